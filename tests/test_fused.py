"""GPU parity of the fused layer blocks and of the GEMM epilogue options (addend, mask, split-K) against
fp32 formulas built from the oracle operators."""
import ctypes

import pytest
import torch

from oracle import ops
from util import assert_close, norm_rel

pytestmark = pytest.mark.gpu


def _r(*shape, scale=1.0, dtype=torch.float16):
    return (scale * torch.randn(shape, device="cuda")).to(dtype)


@pytest.mark.parametrize("dims", [(2, 256, 512), (3, 100, 203)])
def test_layernorm_fork(dims):
    from tritonformer_b200.fused import LayerNormFork
    b, t, d = dims
    torch.manual_seed(0)
    x = _r(b, t, d).requires_grad_(True)
    al, be = _r(d).requires_grad_(True), _r(d).requires_grad_(True)
    dy, dr = _r(b, t, d), _r(b, t, d)
    y, r = LayerNormFork.apply(x, al, be, 1e-5)
    assert torch.equal(r, x)
    torch.autograd.backward([y, r], [dy, dr])
    xr, ar, br = (v.detach().float().requires_grad_(True) for v in (x, al, be))
    yr = ops.layer_norm(xr, ar, br, 1e-5)
    torch.autograd.backward([yr, xr * 1.0], [dy.float(), dr.float()])
    assert_close(y, yr, 1e-2, "y", rtol=1e-3)
    assert_close(x.grad, xr.grad, 1e-2, "dx", rtol=1e-3)
    assert norm_rel(al.grad, ar.grad) < 1e-3 and norm_rel(be.grad, br.grad) < 1e-3


@pytest.mark.parametrize("dims,bias", [((2, 256, 512, 256), True), ((2, 256, 512, 256), False), ((1, 70, 129, 67), True)])
def test_linear_residual(dims, bias):
    from tritonformer_b200.fused import LinearResidual
    b, t, k, n = dims
    torch.manual_seed(1)
    x, res = _r(b, t, k).requires_grad_(True), _r(b, t, n).requires_grad_(True)
    w = _r(k, n, scale=k ** -0.5).requires_grad_(True)
    bb = _r(n).requires_grad_(True) if bias else None
    dy = _r(b, t, n)
    y = LinearResidual.apply(x, w, bb, res)
    y.backward(dy)
    xr, wr, rr = (v.detach().float().requires_grad_(True) for v in (x, w, res))
    br = bb.detach().float().requires_grad_(True) if bias else None
    yr = ops.linear(xr, wr, br) + rr
    yr.backward(dy.float())
    assert_close(y, yr, 1e-2, "y", rtol=1e-3)
    assert norm_rel(x.grad, xr.grad) < 1e-3 and norm_rel(w.grad, wr.grad) < 1e-3
    assert torch.equal(res.grad, dy)
    if bias:
        assert norm_rel(bb.grad, br.grad) < 1e-3


def test_qkv_projection():
    from tritonformer_b200.fused import QKVProjection
    torch.manual_seed(2)
    x = _r(2, 256, 512).requires_grad_(True)
    ws = [_r(512, 512, scale=512 ** -0.5).requires_grad_(True) for _ in range(3)]
    gs = [_r(2, 256, 512) for _ in range(3)]
    outs = QKVProjection.apply(x, *ws)
    torch.autograd.backward(list(outs), gs)
    xr = x.detach().float().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    outr = [ops.linear(xr, w) for w in wr]
    torch.autograd.backward(outr, [g.float() for g in gs])
    for a, b_ in zip(outs, outr):
        assert norm_rel(a, b_) < 1e-3
    assert norm_rel(x.grad, xr.grad) < 1e-3
    for a, b_ in zip(ws, wr):
        assert norm_rel(a.grad, b_.grad) < 1e-3


@pytest.mark.parametrize("bias", [False, True])
def test_mlp_residual(bias):
    from tritonformer_b200.fused import MLPResidual
    torch.manual_seed(3)
    b, t, d, f = 2, 256, 256, 1024
    x, res = _r(b, t, d).requires_grad_(True), _r(b, t, d).requires_grad_(True)
    w1, w2 = _r(d, f, scale=d ** -0.5).requires_grad_(True), _r(f, d, scale=f ** -0.5).requires_grad_(True)
    b1 = _r(f).requires_grad_(True) if bias else None
    b2 = _r(d).requires_grad_(True) if bias else None
    dy = _r(b, t, d)
    import tritonformer_b200.fused as fused
    pattern = []
    fused.CAPTURE_ACTIVATION_PATTERN = pattern
    try:
        y = MLPResidual.apply(x, w1, b1, w2, b2, res)
    finally:
        fused.CAPTURE_ACTIVATION_PATTERN = None
    y.backward(dy)
    f32 = lambda v: v.detach().float().requires_grad_(True) if v is not None else None
    xr, rr, w1r, w2r, b1r, b2r = map(f32, (x, res, w1, w2, b1, b2))
    pre = ops.linear(xr, w1r, b1r)
    mask = pattern[0]
    assert bool(((pre > 0) == mask)[pre.abs() > 1e-2].all())
    yr = ops.linear(pre * mask, w2r, b2r) + rr   # ReLU with the kernel's own activation pattern
    yr.backward(dy.float())
    assert_close(y, yr, 1e-2, "y", rtol=1e-3)
    for nm, a, b_ in (("dx", x, xr), ("dw1", w1, w1r), ("dw2", w2, w2r)):
        assert norm_rel(a.grad, b_.grad) < 1e-3, nm
    assert torch.equal(res.grad, dy)
    if bias:
        assert norm_rel(b1.grad, b1r.grad) < 1e-3 and norm_rel(b2.grad, b2r.grad) < 1e-3


STREAM_K_SHAPES = [
    (1024, 1024, 8192),    # 32 tiles: every tile shared by four or five SMs
    (256, 1024, 4096),     # 8 tiles
    (1000, 264, 2048),     # ragged M and N, 16 tiles
    (8192, 1024, 1024),    # 256 tiles on 148 SMs: one wave plus a remainder, each tile on at most two SMs
    (4100, 1544, 704),     # 231 tiles, ragged in M, N and K
    (128, 136, 1024),      # two tiles, few k-blocks
    (128, 64, 64),         # a single tile and k-block: nothing to share
    (1024, 3072, 4096),    # 48 tiles of 256 x 256 for 74 pairs of SMs: CTA-pair kernel, K shared between pairs
    (2300, 2056, 1088),    # 81 ragged pair tiles: CTA-pair kernel, whole tiles
]


@pytest.mark.parametrize("shape", STREAM_K_SHAPES)
@pytest.mark.parametrize("layout", ["weight_grad", "forward", "input_grad"])
def test_stream_k_gemm_matches_fp32_and_is_deterministic(shape, layout):
    """Outputs with fewer tiles than SMs (or pairs of SMs) share the contraction of their tiles between SMs through
    fp32 partial tiles in the workspace; large outputs run on the CTA-pair kernel.  The result must match fp32, must not depend on timing, must agree with
    the same kernel run without a workspace (whole tiles only), and the arrival counters must be zero again."""
    import ctypes
    from tritonformer_b200 import _lib, linear as lin
    m, n, k = shape
    torch.manual_seed(4)
    if layout == "weight_grad":
        a = _r(k, m)                       # A(m, k) = a[k, m]  (MN-major)
        a_sm, a_sk, a32 = 1, m, a.float().t()
    else:
        a = _r(m, k)
        a_sm, a_sk, a32 = k, 1, a.float()
    if layout == "input_grad":
        b = _r(n, k, scale=k ** -0.5)      # B(k, n) = b[n, k]  (K-major, a weight read transposed)
        b_sk, b_sn, b32 = 1, k, b.float().t()
    else:
        b = _r(k, n, scale=k ** -0.5)
        b_sk, b_sn, b32 = n, 1, b.float()
    bias, old, mask = _r(n), _r(m, n), _r(m, n)
    want = a32 @ b32
    got1 = lin.gemm(a, a_sm, a_sk, b, b_sk, b_sn, m, n, k)
    got2 = lin.gemm(a, a_sm, a_sk, b, b_sk, b_sn, m, n, k)
    assert torch.equal(got1, got2)
    assert norm_rel(got1, want) < 1e-3
    plain = torch.empty_like(got1)
    _lib.check(_lib.lib.tfb_gemm(a.data_ptr(), b.data_ptr(), plain.data_ptr(), None, m, n, k, a_sm, a_sk, b_sk, b_sn,
                                 n, 0, 0, _lib.dtype_code(a.dtype), _lib.stream_ptr(a.device), None))
    assert_close(got1, plain, 2e-3, "with and without workspace", rtol=2e-3)
    acc = old.clone()
    lin.gemm(a, a_sm, a_sk, b, b_sk, b_sn, m, n, k, out=acc, accumulate=True)
    assert norm_rel(acc, want + old.float()) < 1e-3
    full = lin.gemm(a, a_sm, a_sk, b, b_sk, b_sn, m, n, k, bias=bias, relu=True, addend=old, mask=mask)
    assert_close(full, (torch.relu(want + bias.float()) + old.float()) * (mask > 0), 1e-2, "epilogue", rtol=2e-3)
    ws = lin._gemm_workspace(a.device, _lib.stream_ptr(a.device))
    torch.cuda.synchronize()
    assert int(ws[:8192].count_nonzero()) == 0
    assert _lib.lib.tfb_device_status(0) == 0


@pytest.mark.parametrize("shape", [(512, 384, 320), (130, 72, 100)])
def test_gemm_epilogue_addend_and_mask(shape):
    from tritonformer_b200 import linear as lin
    m, n, k = shape
    torch.manual_seed(5)
    a, b = _r(m, k), _r(k, n, scale=k ** -0.5)
    bias, addend, mask = _r(n), _r(m, n), _r(m, n)
    got = lin.gemm(a, k, 1, b, n, 1, m, n, k, bias=bias, relu=True, addend=addend, mask=mask)
    want = (torch.relu(a.float() @ b.float() + bias.float()) + addend.float()) * (mask > 0)
    assert_close(got, want, 1e-2, "epilogue", rtol=1e-3)
