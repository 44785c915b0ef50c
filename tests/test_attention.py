"""GPU parity: CausalAttention / BiasedCausalAttention vs the fp32 oracle.

Shapes are drawn like tritonformer/test_attention.py and test_biased_attention.py (b in [1,4),
heads in [4,32), seq = 64*[1,32), head_dim in {32,64}) plus head_dim 128, T = 2048, the strided
(B,T,H*hd) views the model passes, bf16, a non-ALiBi dense bias and ALiBi given as slopes."""
import numpy as np
import pytest
import torch

from oracle import ops
from util import NUM_TEST, assert_close, golden_arrays, norm_rel

pytestmark = pytest.mark.gpu
rng = np.random.RandomState(0)
DIMS = [(int(b), int(nh), int(sq), int(hd)) for b in rng.randint(1, 4, size=NUM_TEST)
        for nh in rng.randint(4, 32, size=NUM_TEST) for sq in 64 * rng.randint(1, 32, size=NUM_TEST)
        for hd in rng.choice([32, 64], size=NUM_TEST, replace=True)]
DIMS += [(1, 2, 64, 128), (2, 4, 2048, 64), (1, 3, 1024, 128), (1, 2, 4096, 128), (1, 1, 64, 32), (2, 16, 512, 64)]
# the attention shapes of the named configurations: the fused-op benchmark case and the 410M model (B4 H16 T2048
# hd64), the 840M model (B1 H12 T4096 hd128) and the 1.4B model (B2 H16 T2048 hd128)
NAMED = [(4, 16, 2048, 64), (1, 12, 4096, 128), (2, 16, 2048, 128)]


def _make(dims, dtype, strided):
    b, nh, sq, hd = dims
    torch.manual_seed(0)
    if strided:  # views of (B, T, H*hd), as produced by the model's projections
        mk = lambda: torch.randn((b, sq, nh * hd), device="cuda").to(dtype).view(b, sq, nh, hd).transpose(1, 2)
    else:
        mk = lambda: torch.randn((b, nh, sq, hd), device="cuda").to(dtype)
    q, k, v = (mk().detach().requires_grad_(True) for _ in range(3))
    dy = mk().detach()
    return q, k, v, dy


def _compare(q, k, v, dy, out, bias_f32, dtype):
    out.backward(dy)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = ops.attention(qr, kr, vr, bias_f32)
    ref.backward(dy.float())
    if dtype is torch.float16:
        atol, rel = 1e-2, 2e-3   # atol: the reference tests' own bound
    else:
        atol, rel = 8e-2, 1.2e-2
    assert_close(out, ref, atol, "out")
    assert norm_rel(out, ref) < rel
    for nm, a, b_ in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        assert a.stride() == getattr(q if nm == "dq" else k if nm == "dk" else v, "stride")()
        assert norm_rel(a, b_) < 2.5 * rel, nm
        if dtype is torch.float16:
            # the reference tests' own bound (atol 1e-2 against a torch fp16 product) plus one fp16 rounding of
            # gradients whose magnitude is above 1 (sums over up to thousands of positions)
            assert_close(a, b_, 1e-2, nm, rtol=2e-3)


@pytest.mark.parametrize("dims", DIMS)
@pytest.mark.parametrize("strided", [False, True])
def test_causal_attention_fp16(dims, strided):
    from tritonformer_b200.attention import CausalAttention
    q, k, v, dy = _make(dims, torch.float16, strided)
    out = CausalAttention.apply(q, k, v)
    assert out.stride() == q.stride()
    _compare(q, k, v, dy, out, None, torch.float16)


@pytest.mark.parametrize("dims", NAMED)
@pytest.mark.parametrize("alibi", [False, True])
def test_attention_shapes_of_the_named_configurations(dims, alibi):
    """fp16 without bias and with the ALiBi slopes 2^(-8(i+1)/H) of the benchmark case; the 1.4B shape in bf16
    with the reference's (H, T, T) table."""
    from tritonformer_b200 import attention as A
    b, nh, sq, hd = dims
    bf16_table = alibi and dims == (2, 16, 2048, 128)
    dtype = torch.bfloat16 if bf16_table else torch.float16
    q, k, v, dy = _make(dims, dtype, True)
    if not alibi:
        out, bias_ref = A.CausalAttention.apply(q, k, v), None
    elif bf16_table:
        table = ops.alibi_table(sq, nh, torch.float16, "cuda")
        out, bias_ref = A.BiasedCausalAttention.apply(q, k, v, table), table.float()
    else:
        slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / nh) for i in range(nh)], device="cuda")
        pos = torch.arange(sq, device="cuda")
        bias_ref = -slopes[:, None, None] * (pos.view(sq, 1) - pos.view(1, sq)).clamp_min(0).float()
        out = A.BiasedCausalAttention.apply(q, k, v, slopes)
    _compare(q, k, v, dy, out, bias_ref, dtype)


@pytest.mark.parametrize("dims", DIMS[-6:])
def test_causal_attention_bf16(dims):
    from tritonformer_b200.attention import CausalAttention
    q, k, v, dy = _make(dims, torch.bfloat16, True)
    _compare(q, k, v, dy, CausalAttention.apply(q, k, v), None, torch.bfloat16)


@pytest.mark.parametrize("dims", DIMS[::2])
@pytest.mark.parametrize("form", ["table", "slopes", "dense"])
def test_biased_attention_fp16(dims, form):
    from tritonformer_b200 import attention as A
    b, nh, sq, hd = dims
    q, k, v, dy = _make(dims, torch.float16, True)
    if form == "table":      # the reference's (H, P, P) ALiBi table, P > T: recognised, computed in-kernel
        table = ops.alibi_table(sq + 64, nh, torch.float16, "cuda")
        bias_arg, bias_ref = table, table[:, :sq, :sq].float()
        assert A._resolve_bias(table, nh, sq, torch.float16).rounded
    elif form == "slopes":   # exact fp32 ALiBi from per-head slopes
        slopes = torch.tensor(ops.get_slopes(nh), device="cuda", dtype=torch.float32)
        pos = torch.arange(sq, device="cuda")
        bias_arg = slopes
        bias_ref = -slopes[:, None, None] * (pos.view(sq, 1) - pos.view(1, sq)).clamp_min(0).float()
    else:                    # arbitrary dense bias without -inf: still causally masked
        bias_arg = (0.5 * torch.randn((nh, sq, sq), device="cuda")).half()
        bias_ref = bias_arg.float()
        assert A._resolve_bias(bias_arg, nh, sq, torch.float16).table is not None
    out = A.BiasedCausalAttention.apply(q, k, v, bias_arg)
    _compare(q, k, v, dy, out, bias_ref, torch.float16)


def test_attention_golden_vectors():
    from tritonformer_b200.attention import BiasedCausalAttention, CausalAttention
    g = golden_arrays()
    for tag in ("a", "b"):
        q, k, v = (torch.from_numpy(g[f"attn_{tag}_{n}"]).cuda() for n in "qkv")
        assert_close(CausalAttention.apply(q, k, v).cpu(), torch.from_numpy(g[f"attn_{tag}_out"]), 1e-2, "golden")
        q, k, v = (torch.from_numpy(g[f"battn_{tag}_{n}"]).cuda() for n in "qkv")
        bias = torch.from_numpy(g[f"battn_{tag}_bias"]).cuda()
        out = BiasedCausalAttention.apply(q, k, v, bias)
        assert_close(out.cpu(), torch.from_numpy(g[f"battn_{tag}_out"]), 1e-2, "golden bias")


def test_reference_asserts_are_kept():
    from tritonformer_b200.attention import BiasedCausalAttention, CausalAttention
    mk = lambda *s: torch.randn(s, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError, match="multiple of 64"):
        CausalAttention.apply(mk(1, 2, 96, 64), mk(1, 2, 96, 64), mk(1, 2, 96, 64))
    with pytest.raises(AssertionError, match="head_dims"):
        CausalAttention.apply(mk(1, 2, 64, 48), mk(1, 2, 64, 48), mk(1, 2, 64, 48))
    with pytest.raises(AssertionError, match="number of heads"):
        BiasedCausalAttention.apply(mk(1, 2, 64, 64), mk(1, 2, 64, 64), mk(1, 2, 64, 64), mk(3, 64, 64))


@pytest.mark.parametrize("dims", [(2, 4, 2048, 64), (1, 5, 640, 64), (2, 16, 512, 64), (1, 3, 1024, 128)])
@pytest.mark.parametrize("alibi", [False, True])
def test_forward_is_independent_of_the_order_of_its_items(dims, alibi):
    """The forward kernel's persistent CTAs walk (query tile, batch*head) items longest walk first; a switch makes
    them walk slice by slice instead.  The arithmetic of an item does not depend on which CTA runs it or when, so
    both orders give the same bits; output and log-sum-exp match the oracle."""
    from tritonformer_b200 import _lib
    from tritonformer_b200.attention import _Bias, attention_forward
    b, nh, sq, hd = dims
    q, k, v, _ = _make(dims, torch.float16, True)
    q, k, v = q.detach(), k.detach(), v.detach()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / nh) for i in range(nh)], device="cuda") if alibi else None
    bias = _Bias(slopes=slopes)
    out1, lse1, _ = attention_forward(q, k, v, bias)
    _lib.lib.tfb_debug_set(2, 32)
    try:
        out2, lse2, _ = attention_forward(q, k, v, bias)
    finally:
        _lib.lib.tfb_debug_set(2, 0)
    torch.cuda.synchronize()
    assert _lib.lib.tfb_device_status(0) == 0
    assert torch.equal(out1, out2) and torch.equal(lse1, lse2)
    bias_f32 = None
    if alibi:
        pos = torch.arange(sq, device="cuda")
        dist = (pos.view(sq, 1) - pos.view(1, sq)).clamp(min=0).float()
        bias_f32 = -dist.view(1, sq, sq) * slopes.view(nh, 1, 1)
    ref = ops.attention(q.float(), k.float(), v.float(), bias_f32)
    assert_close(out1, ref, 1e-2, "out")
    assert norm_rel(out1, ref) < 2e-3
    scores = torch.einsum("bhid,bhjd->bhij", q.float(), k.float()) / hd ** 0.5
    if bias_f32 is not None:
        scores = scores + bias_f32
    causal = torch.ones((sq, sq), dtype=torch.bool, device="cuda").tril()
    lse_ref = torch.logsumexp(scores.masked_fill(~causal, float("-inf")), dim=-1)
    assert_close(lse1, lse_ref, 2e-3, "lse")


def test_alibi_finding_is_tied_to_the_tensor_object():
    """The "this table is ALiBi" finding lives on the tensor object: a different table that reuses the same
    address is examined afresh, and an in-place write makes the finding stale."""
    from tritonformer_b200 import attention as A
    nh, sq = 4, 128
    table = ops.alibi_table(sq, nh, torch.float16, "cuda")
    assert A._resolve_bias(table, nh, sq, torch.float16).slopes is not None
    addr = table.data_ptr()
    del table
    dense = torch.randn((nh, sq, sq), device="cuda").half()  # the caching allocator hands the block out again
    res = A._resolve_bias(dense, nh, sq, torch.float16)
    assert res.table is not None and res.slopes is None, (addr, dense.data_ptr())
    table = ops.alibi_table(sq, nh, torch.float16, "cuda")
    assert A._resolve_bias(table, nh, sq, torch.float16).slopes is not None
    table[:, 5, 2] = 0.25  # no longer ALiBi; the write bumps the version counter
    assert A._resolve_bias(table, nh, sq, torch.float16).table is not None
