"""GPU parity: CrossEntropyLoss Function vs the oracle (shapes drawn like tritonformer/test_crossentropy.py)."""
import numpy as np
import pytest
import torch

from oracle import ops
from util import NUM_TEST, assert_close, golden_arrays

pytestmark = pytest.mark.gpu
rng = np.random.RandomState(0)
DIMS = [(int(b), int(d)) for b in rng.randint(1, 32, size=NUM_TEST + 2) for d in rng.randint(256, 64000, size=NUM_TEST + 2)]
DIMS += [(64, 50304), (5, 50304 + 3), (1, 8)]


@pytest.mark.parametrize("dims", DIMS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cross_entropy_fwd_bwd(dims, dtype):
    from tritonformer_b200.crossentropy import CrossEntropyLoss, CrossEntropyLossFP32
    n, v = dims
    torch.manual_seed(0)
    logits = torch.randn((n, v), device="cuda").to(dtype).requires_grad_(True)
    labels = torch.randint(0, v, (n,), device="cuda")
    if n > 2:
        labels[1] = -1  # skipped row
    before = logits.detach().clone()
    loss = CrossEntropyLoss.apply(logits, labels)
    assert loss.shape == (n,) and loss.dtype == dtype
    w = torch.randn((n,), device="cuda").to(dtype)
    loss.backward(w)
    assert torch.equal(logits.detach(), before), "saved logits must not be modified"
    lr = logits.detach().float().requires_grad_(True)
    ref = ops.cross_entropy_rows(lr, labels)
    ref.backward(w.float())
    assert_close(loss, ref, 1e-2 if dtype is torch.float16 else 6e-2, "loss")
    assert_close(logits.grad, lr.grad, 1e-2, "dlogits")
    # fp32-loss variant, mean reduction through a stride-0 expanded gradient
    logits.grad = None
    l32 = CrossEntropyLossFP32.apply(logits, labels)
    assert l32.dtype == torch.float32
    assert_close(l32, ref.detach(), 2e-5, "loss fp32")
    (l32.sum() / n).backward()
    lr.grad = None
    (ops.cross_entropy_rows(lr, labels).sum() / n).backward()
    tol = 2e-3 if dtype is torch.float16 else 1.6e-2
    assert (logits.grad.float() - lr.grad).abs().max().item() <= tol * lr.grad.abs().max().item() + 1e-7


def test_cross_entropy_golden_vector():
    from tritonformer_b200.crossentropy import CrossEntropyLossFP32
    g = golden_arrays()
    loss = CrossEntropyLossFP32.apply(torch.from_numpy(g["ce_logits"]).cuda(), torch.from_numpy(g["ce_labels"]).cuda())
    assert abs(loss.mean().item() - float(g["ce_mean"])) < 1e-5
