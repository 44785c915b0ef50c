"""GPU parity: Softmax Function vs the oracle (shapes drawn like tritonformer/test_softmax.py)."""
import numpy as np
import pytest
import torch

from oracle import ops
from util import NUM_TEST, assert_close, golden_arrays

pytestmark = pytest.mark.gpu
rng = np.random.RandomState(0)
DIMS = [(int(b), int(i), int(j)) for b in rng.randint(1, 32, size=NUM_TEST)
        for i in rng.randint(256, 1024, size=NUM_TEST) for j in rng.randint(64, 1024, size=NUM_TEST)]
DIMS += [(2, 512, 1024), (1, 256, 2048), (1, 64, 5000), (3, 7, 4)]


@pytest.mark.parametrize("dims", DIMS)
def test_softmax_fwd_bwd_fp32(dims):
    from tritonformer_b200.softmax import Softmax
    b, sq, d = dims
    torch.manual_seed(0)
    x = torch.randn((b, sq, d), device="cuda", requires_grad=True)
    dy = 0.1 * torch.randn((b, sq, d), device="cuda")
    keep = dy.clone()
    y = Softmax.apply(x)
    y.backward(dy)
    assert torch.equal(dy, keep), "incoming gradient must not be modified"
    xr = x.detach().clone().requires_grad_(True)
    yr = ops.softmax(xr)
    yr.backward(dy)
    assert_close(y, yr, 1e-4, "y")      # atol of the reference test
    assert_close(x.grad, xr.grad, 1e-4, "dx")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_softmax_16bit(dtype):
    from tritonformer_b200.softmax import Softmax
    torch.manual_seed(1)
    x = torch.randn((2, 300, 1000), device="cuda").to(dtype).requires_grad_(True)
    dy = (0.1 * torch.randn((2, 300, 1000), device="cuda")).to(dtype)
    y = Softmax.apply(x)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    yr = ops.softmax(xr)
    yr.backward(dy.float())
    tol = 1e-3 if dtype is torch.float16 else 8e-3
    assert_close(y, yr, tol, "y")
    assert_close(x.grad, xr.grad, tol, "dx")


def test_softmax_golden_vector():
    from tritonformer_b200.softmax import Softmax
    g = golden_arrays()
    y = Softmax.apply(torch.from_numpy(g["sm_x"]).cuda())
    assert_close(y.cpu(), torch.from_numpy(g["sm_out"]), 1e-6, "golden")
