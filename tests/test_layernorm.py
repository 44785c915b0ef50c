"""GPU parity: LayerNorm Function vs the fp32 oracle (shapes drawn like tritonformer/test_layernorm.py)."""
import numpy as np
import pytest
import torch

from oracle import ops
from util import NUM_TEST, assert_close, golden_arrays, norm_rel

pytestmark = pytest.mark.gpu
rng = np.random.RandomState(0)
DIMS = [(int(b), int(i), int(j)) for b in rng.randint(1, 32, size=NUM_TEST)
        for i in rng.randint(64, 1024, size=NUM_TEST) for j in rng.randint(64, 1024, size=NUM_TEST)]
DIMS += [(4, 2048, 1024), (1, 4096, 1536), (2, 2048, 2048), (2, 1024, 768), (1, 3, 8), (1, 1, 4104)]


def _run(dims, dtype):
    from tritonformer_b200.layernorm import LayerNorm
    b, sq, d = dims
    torch.manual_seed(0)
    x = (3.14 + 0.4 * torch.randn((b, sq, d), device="cuda")).to(dtype).requires_grad_(True)
    alpha = torch.randn((d,), device="cuda").to(dtype).requires_grad_(True)
    beta = torch.randn((d,), device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn((b, sq, d), device="cuda").to(dtype)
    y = LayerNorm.apply(x, alpha, beta, 1e-5)
    y.backward(dy)
    xr, ar, br = (t.detach().float().requires_grad_(True) for t in (x, alpha, beta))
    yr = ops.layer_norm(xr, ar, br, 1e-5)
    yr.backward(dy.float())
    return (y, x.grad, alpha.grad, beta.grad), (yr, xr.grad, ar.grad, br.grad)


@pytest.mark.parametrize("dims", DIMS)
def test_ln_fwd_bwd_fp16(dims):
    (y, dx, da, db), (yr, dxr, dar, dbr) = _run(dims, torch.float16)
    assert y.dtype == torch.float16 and da.shape == dar.shape
    assert_close(y, yr, 1e-2, "y", rtol=1e-3)       # atol of the reference tests + one fp16 rounding
    assert_close(dx, dxr, 1e-2, "dx", rtol=1e-3)
    assert norm_rel(da, dar) < 1e-3 and norm_rel(db, dbr) < 1e-3  # reference: norm-relative < 1e-3


@pytest.mark.parametrize("dims", DIMS[-6:])
def test_ln_fwd_bwd_bf16(dims):
    (y, dx, da, db), (yr, dxr, dar, dbr) = _run(dims, torch.bfloat16)
    assert norm_rel(y, yr) < 4e-3 and norm_rel(dx, dxr) < 6e-3
    assert norm_rel(da, dar) < 4e-3 and norm_rel(db, dbr) < 4e-3


def test_ln_golden_vector():
    from tritonformer_b200.layernorm import LayerNorm
    g = golden_arrays()
    x, a, b = (torch.from_numpy(g[k]).cuda() for k in ("ln_x", "ln_alpha", "ln_beta"))
    y = LayerNorm.apply(x, a, b, 1e-5)
    assert_close(y.cpu(), torch.from_numpy(g["ln_out"]), 1e-2, "golden")


def test_ln_under_autocast_casts_to_fp16():
    from tritonformer_b200.nn import LayerNorm as LNModule
    m = LNModule(256, device="cuda", dtype=torch.float16)
    torch.nn.init.ones_(m.weight), torch.nn.init.zeros_(m.bias)
    x = torch.randn(2, 64, 256, device="cuda")  # fp32 input
    with torch.autocast("cuda", dtype=torch.float16):
        y = m(x)
    assert y.dtype == torch.float16
    with pytest.raises(AssertionError):
        m(x)  # outside autocast nothing is cast, fp32 input is rejected like the reference does


def test_ln_backward_adds_parameter_gradients_into_given_buffers():
    """`into=(dalpha, dbeta)`: the kernel that folds the partial column sums adds them to what the buffers hold
    (gradient accumulation without a separate add), dx is unchanged."""
    from tritonformer_b200.layernorm import layernorm_backward, layernorm_forward
    torch.manual_seed(1)
    x = torch.randn((3, 70, 512), device="cuda").half()
    dy = torch.randn_like(x)
    alpha = torch.randn(512, device="cuda").half()
    beta = torch.randn(512, device="cuda").half()
    _, stats = layernorm_forward(x, alpha, beta, 1e-5)
    dx, da, db = layernorm_backward(dy, x, alpha, stats)
    old_a = torch.randn(512, device="cuda").half()
    old_b = torch.randn(512, device="cuda").half()
    buf_a, buf_b = old_a.clone(), old_b.clone()
    dx2, none_a, none_b = layernorm_backward(dy, x, alpha, stats, into=(buf_a, buf_b))
    assert none_a is None and none_b is None
    assert torch.equal(dx, dx2)
    # one fp32 add of the fp32 column sum and the old value, one rounding
    assert_close(buf_a, old_a.float() + da.float(), 2e-2, "dalpha", rtol=2e-3)
    assert_close(buf_b, old_b.float() + db.float(), 2e-2, "dbeta", rtol=2e-3)
