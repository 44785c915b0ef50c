"""GPU parity: the four Linear Functions vs the oracle (shapes drawn like tritonformer/test_linear.py,
i.e. mostly NOT multiples of 8, plus the model's aligned shapes that run on the tcgen05 kernel)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ops
from util import NUM_TEST, assert_close, golden_arrays, norm_rel

pytestmark = pytest.mark.gpu
rng = np.random.RandomState(0)
RAGGED = [(int(b), int(i), int(j), int(k)) for b in rng.randint(1, 8, size=NUM_TEST)
          for i in rng.randint(64, 2048, size=NUM_TEST) for j in rng.randint(64, 4096, size=NUM_TEST)
          for k in rng.randint(64, 4096, size=NUM_TEST)]
ALIGNED = [(4, 2048, 1024, 1024), (2, 512, 1024, 4096), (2, 512, 4096, 1024), (1, 1024, 1536, 1536),
           (1, 256, 768, 50304), (3, 72, 136, 264), (1, 128, 64, 128), (2, 100, 8, 8), (1, 8, 4096, 16)]


def _functions():
    from tritonformer_b200.linear import LinearBias, LinearBiasReLU, LinearNoBias, LinearNoBiasReLU
    return {(False, False): LinearNoBias, (True, False): LinearBias,
            (False, True): LinearNoBiasReLU, (True, True): LinearBiasReLU}


def _run(dims, has_bias, relu, dtype):
    b, m, n, k = dims
    torch.manual_seed(0)
    x = torch.randn((b, m, n), device="cuda").to(dtype).requires_grad_(True)
    w = (torch.randn((n, k), device="cuda") / n ** 0.5).to(dtype).requires_grad_(True)
    bias = torch.randn((k,), device="cuda").to(dtype).requires_grad_(True) if has_bias else None
    dy = torch.randn((b, m, k), device="cuda").to(dtype)
    keep = dy.clone()
    fn = _functions()[(has_bias, relu)]
    y = fn.apply(x, w, bias) if has_bias else fn.apply(x, w)
    y.backward(dy)
    assert torch.equal(dy, keep), "incoming gradient must not be modified"
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    br = bias.detach().float().requires_grad_(True) if has_bias else None
    yr = ops.linear(xr, wr, br, False)
    if relu:
        # A pre-activation within rounding distance of zero may land on either side in 16-bit
        # arithmetic; the oracle is evaluated with the kernel's own mask so that such units do not
        # turn into whole-row differences of dX.  The masks must agree wherever |pre-act| is not tiny.
        mask = y.detach() > 0
        pre = yr.detach()
        assert bool(((pre > 0) == mask)[pre.abs() > 1e-2].all()), "ReLU mask disagrees away from zero"
        yr = yr * mask
    yr.backward(dy.float())
    got = [y, x.grad, w.grad] + ([bias.grad] if has_bias else [])
    want = [yr, xr.grad, wr.grad] + ([br.grad] if has_bias else [])
    return got, want


def _check(got, want, dtype):
    names = ["y", "dx", "dw", "db"]
    for nm, a, b in zip(names, got, want):
        assert a.shape == b.shape and a.dtype == dtype, nm
        # one rounding of an fp32-accumulated result: 2^-11 (fp16) / 2^-8 (bf16) relative
        assert norm_rel(a, b) < (1e-3 if dtype is torch.float16 else 6e-3), nm
    if dtype is torch.float16:
        assert_close(got[0], want[0], 1e-2, "y", rtol=1e-3)  # the reference tests' atol + one fp16 rounding
        assert_close(got[1], want[1], 1e-2, "dx", rtol=1e-3)


@pytest.mark.parametrize("dims", RAGGED)
@pytest.mark.parametrize("has_bias", [False, True])
def test_linear_ragged_shapes(dims, has_bias):
    got, want = _run(dims, has_bias, False, torch.float16)
    _check(got, want, torch.float16)


@pytest.mark.parametrize("dims", ALIGNED)
@pytest.mark.parametrize("has_bias,relu", [(False, False), (True, False), (False, True), (True, True)])
def test_linear_aligned_shapes(dims, has_bias, relu):
    got, want = _run(dims, has_bias, relu, torch.float16)
    _check(got, want, torch.float16)


@pytest.mark.parametrize("dims", ALIGNED[:4] + RAGGED[:2])
def test_linear_bf16(dims):
    got, want = _run(dims, True, True, torch.bfloat16)
    _check(got, want, torch.bfloat16)


def test_aligned_shapes_take_the_tcgen05_kernel_and_agree_with_the_generic_one():
    import tritonformer_b200._lib as L
    torch.manual_seed(3)
    m, n, k = 512, 384, 320
    a = torch.randn((m, k), device="cuda", dtype=torch.float16)
    b = torch.randn((k, n), device="cuda", dtype=torch.float16) / k ** 0.5
    outs = []
    for force in (0, 1):
        L.lib.tfb_debug_set(0, force)
        c = torch.empty((m, n), device="cuda", dtype=torch.float16)
        path = ctypes.c_int(-1)
        L.check(L.lib.tfb_gemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, m, n, k, k, 1, n, 1, n, 0, 0, 0,
                               L.stream_ptr(a.device), ctypes.byref(path)))
        assert path.value == (0 if force else 1)
        outs.append(c)
    L.lib.tfb_debug_set(0, 0)
    assert L.device_status() == 0
    assert_close(outs[0], outs[1], 2e-3, "tcgen05 vs generic")


def test_gemm_accumulate_and_strided_output():
    import tritonformer_b200._lib as L
    torch.manual_seed(4)
    m, n, k = 256, 128, 192
    a = torch.randn((m, k), device="cuda", dtype=torch.float16)
    b = torch.randn((k, n), device="cuda", dtype=torch.float16) / k ** 0.5
    big = torch.randn((m, n + 64), device="cuda", dtype=torch.float16)
    want = big.clone().float()
    want[:, :n] += a.float() @ b.float()
    L.check(L.lib.tfb_gemm(a.data_ptr(), b.data_ptr(), big.data_ptr(), None, m, n, k, k, 1, n, 1, n + 64, 0, 1, 0,
                           L.stream_ptr(a.device), None))
    assert_close(big, want, 2e-2, "accumulate into a slice")


def test_linear_golden_vector():
    from tritonformer_b200.linear import LinearBias, LinearNoBias
    g = golden_arrays()
    x, w, b = (torch.from_numpy(g[k]).cuda() for k in ("lin_x", "lin_w", "lin_b"))
    assert_close(LinearNoBias.apply(x, w).cpu(), torch.from_numpy(g["lin_out"]), 1e-2, "golden")
    assert_close(LinearBias.apply(x, w, b).cpu(), torch.from_numpy(g["lin_out_bias"]), 1e-2, "golden bias")


def test_dimension_mismatch_raises_like_the_reference():
    from tritonformer_b200.linear import LinearNoBias
    x = torch.randn((1, 8, 16), device="cuda", dtype=torch.float16)
    w = torch.randn((24, 8), device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError, match="Dimension mismatch"):
        LinearNoBias.apply(x, w)
