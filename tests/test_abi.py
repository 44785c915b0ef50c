"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments before touching the device."""
import ctypes
import os
import re

import tritonformer_b200._lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tfb_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    operators = _declared("tritonformer_b200.h")
    switches = _declared("tritonformer_b200_debug.h")
    assert len(operators) >= 19
    # the test and tuning switches live in a header of their own, outside the operator interface
    assert switches and all(n.startswith("tfb_debug_") for n in switches)
    assert not any(n.startswith("tfb_debug_") for n in operators)
    names = sorted(operators + switches)
    raw = ctypes.CDLL(L.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), n
    assert sorted(L.EXPORTS) == names


def test_version_and_error_text():
    assert L.lib.tfb_version() >= 1
    rc = L.lib.tfb_gemm(None, None, None, None, 4, 4, 4, 3, 5, 1, 4, 4, 0, 0, 0, None, None)
    assert rc == -1 and b"unit stride" in L.lib.tfb_last_error()
    try:
        L.check(rc)
    except AssertionError as e:
        assert "unit stride" in str(e)
    else:
        raise AssertionError("no exception")


def test_argument_checks_without_device():
    s = (ctypes.c_int64 * 3)(8, 8, 8)
    rc = L.lib.tfb_attention_fwd(None, None, None, None, None, 1, 2, 64, 48, s, s, s, s, None, 0, None, 0, 0, 0,
                                 None, None)
    assert rc == -2 and b"head_dims" in L.lib.tfb_last_error()
    rc = L.lib.tfb_attention_fwd(None, None, None, None, None, 1, 2, 100, 64, s, s, s, s, None, 0, None, 0, 0, 0,
                                 None, None)
    assert rc == -1 and b"multiple of 64" in L.lib.tfb_last_error()
    assert L.lib.tfb_layernorm_fwd(None, None, None, None, None, None, 4, 0, 0, 0, 1e-5, 0, None) == -1
    assert L.lib.tfb_softmax_fwd(None, None, 4, 8, 4, 8, 2, None) == -1  # row stride < cols
    assert L.lib.tfb_cross_entropy_fwd(None, None, None, None, None, 4, 8, 8, 2, None) == -1  # fp32 logits
    assert L.lib.tfb_layernorm_bwd_partials(8192, 1024) > 0
    assert L.lib.tfb_colsum_partials(8192, 4096) > 0
    assert L.lib.tfb_attention_bwd_scratch_bytes(1, 2, 64, 64) == 2 * 64 * 4 + 2 * 64 * 64 * 4  # 512 is 256-aligned
    # embeddings: shape, position count and scratch are checked before anything is launched
    assert L.lib.tfb_embedding_fwd(None, None, None, None, 2, 8, 0, 100, 0, 0, None) == -1  # d = 0
    assert L.lib.tfb_embedding_fwd(None, None, None, None, 0, 8, 64, 100, 0, 0, None) == 0  # no positions: nothing to do
    one = ctypes.c_void_p(16)  # never dereferenced: the row-count check comes before any launch
    rc = L.lib.tfb_embedding_fwd(None, None, one, None, 2, 8, 64, 100, 4, 0, None)
    assert rc == -1 and b"position table" in L.lib.tfb_last_error()
    rc = L.lib.tfb_embedding_bwd(None, None, None, one, None, 0, 2, 8, 64, 100, 4, 0, None)
    assert rc == -1 and b"position table" in L.lib.tfb_last_error()
    assert L.lib.tfb_embedding_bwd_scratch_bytes(2, 8, 64, 100) == 2 * 100 * 4 + 2 * 8 * 64 * 4
    rc = L.lib.tfb_embedding_bwd(None, None, one, None, None, 0, 2, 8, 64, 100, 0, 0, None)
    assert rc == -1 and b"scratch" in L.lib.tfb_last_error()
    assert L.lib.tfb_embedding_bwd(None, None, None, None, None, 0, 2, 8, 64, 100, 0, 0, None) == 0  # both tables frozen
