"""ctypes binding of libtritonformer_b200.so (the C ABI declared in include/tritonformer_b200.h; the
tfb_debug_* switches in include/tritonformer_b200_debug.h).

The library is the only implementation: if it is missing the import fails loudly, there is
no Python or CPU fallback for any operator.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtritonformer_b200.so")

F16, BF16, F32 = 0, 1, 2
_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}

_c = ctypes
_vp, _i64, _i32, _f32 = _c.c_void_p, _c.c_int64, _c.c_int, _c.c_float
_pi64 = _c.POINTER(_c.c_int64)
_pi32 = _c.POINTER(_c.c_int)

_SIGNATURES = {
    "tfb_version": (_i32, []),
    "tfb_last_error": (_c.c_char_p, []),
    "tfb_launch_count": (_i64, []),
    "tfb_device_status": (_i32, [_i32]),
    "tfb_debug_set": (None, [_i32, _i32]),
    "tfb_debug_counters": (_i32, [_c.POINTER(_c.c_uint64)]),
    "tfb_debug_wait_probe": (_i32, [_c.c_uint64, _vp, _vp]),
    "tfb_layernorm_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _vp]),
    "tfb_layernorm_bwd_partials": (_i64, [_i64, _i64]),
    "tfb_layernorm_bwd": (_i32, [_vp] * 9 + [_i64] * 6 + [_i32, _vp]),
    "tfb_layernorm_bwd_res": (_i32, [_vp] * 10 + [_i64] * 7 + [_i32, _vp]),
    "tfb_layernorm_bwd_acc": (_i32, [_vp] * 10 + [_i64] * 7 + [_i32, _i32, _vp]),
    "tfb_layernorm_bwd_static": (_i32, [_vp] * 8 + [_i64] * 5 + [_i32, _vp]),
    "tfb_softmax_fwd": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tfb_softmax_bwd": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tfb_cross_entropy_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp]),
    "tfb_cross_entropy_bwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tfb_relu_bwd": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "tfb_colsum_partials": (_i64, [_i64, _i64]),
    "tfb_colsum": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tfb_embedding_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tfb_embedding_bwd_scratch_bytes": (_i64, [_i64] * 4),
    "tfb_embedding_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "tfb_grad_check": (_i32, [_vp, _i64, _i32, _vp, _vp]),
    "tfb_adamw_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _vp, _vp] + [_c.c_double] * 5 + [_vp]),
    "tfb_loss_scale_update": (_i32, [_vp, _vp, _f32, _f32, _i32, _vp]),
    "tfb_gemm": (_i32, [_vp, _vp, _vp, _vp] + [_i64] * 8 + [_i32, _i32, _i32, _vp, _pi32]),
    "tfb_gemm_workspace_bytes": (_i64, []),
    "tfb_gemm_fused": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64] + [_i64] * 8 + [_i32, _i32, _vp, _i64, _vp, _pi32]),
    "tfb_attention_fwd": (_i32, [_vp] * 5 + [_i64] * 4 + [_pi64] * 4 + [_vp, _i32, _vp, _i64, _i64, _i32, _vp, _pi32]),
    "tfb_attention_bwd_scratch_bytes": (_i64, [_i64] * 4),
    "tfb_attention_bwd": (_i32, [_vp] * 9 + [_i64] * 4 + [_pi64] * 8 + [_vp, _i32, _vp, _i64, _i64, _vp, _i64, _i32, _vp, _pi32]),
}

EXPORTS = tuple(sorted(_SIGNATURES))


def _load():
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "tritonformer_b200: %s is missing. Build it with `python tritonformer_b200/build.py` "
            "(needs nvcc); there is no fallback implementation." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
if os.environ.get("TFB_FORCE_GENERIC_GEMM") == "1":  # test switch, see tfb_debug_set
    lib.tfb_debug_set(0, 1)
if os.environ.get("TFB_FORCE_GENERIC_ATTN") == "1":
    lib.tfb_debug_set(1, 1)
if os.environ.get("TFB_SERIALISED_LAUNCHES") == "1":  # no programmatic dependent launch
    lib.tfb_debug_set(3, 1)
if os.environ.get("TFB_GEMM_FREE_SMS"):  # SMs the GEMM grids leave to a collective running beside them
    lib.tfb_debug_set(6, int(os.environ["TFB_GEMM_FREE_SMS"]))
if os.environ.get("TFB_GEMM_SWITCHES"):  # bit 0: whole tiles only, bit 5 (32): no CTA-pair kernel
    lib.tfb_debug_set(4, int(os.environ["TFB_GEMM_SWITCHES"]))


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[t]
    except KeyError:
        raise AssertionError("unsupported dtype %s" % t)


def check(rc: int) -> None:
    """Status -> exception: argument errors surface as AssertionError like the reference's asserts."""
    if rc == 0:
        return
    msg = lib.tfb_last_error().decode("utf-8", "replace")
    if rc in (-1, -2):
        raise AssertionError(msg)
    raise RuntimeError("tritonformer_b200 (%d): %s" % (rc, msg))


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def strides3(t: torch.Tensor):
    """{b,h,t} element strides of a (B,H,T,hd) tensor as a C array."""
    return (_c.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def launch_count() -> int:
    return int(lib.tfb_launch_count())


def device_status(reset: bool = False) -> int:
    """The status word of the current device (synchronises it).  With `reset`, clears a non-zero word and
    zeroes the GEMM workspaces, whose arrival counters an abandoned split product can leave non-zero."""
    code = int(lib.tfb_device_status(1 if reset else 0))
    if reset and code != 0:
        from . import linear
        linear.reset_workspaces()
    return code


_STATUS_TEXT = {0x7100: "a token id outside the embedding table", 0x7e00: "the wait probe of the test suite"}


def check_status() -> None:
    """Raises RuntimeError if a kernel of the library reported a failure on the current device (a bounded wait
    that ran out, a token id outside the embedding table).  Synchronises the device: call it where the host
    waits anyway, e.g. next to the read-back of the loss.  The status stays set until device_status(reset=True)."""
    code = device_status()
    if code != 0:
        what = _STATUS_TEXT.get(code, "a bounded wait inside a kernel ran out")
        raise RuntimeError("tritonformer_b200: device status 0x%x (%s); the tensor-core kernels skip their work "
                           "until the status is cleared with device_status(reset=True)" % (code, what))
