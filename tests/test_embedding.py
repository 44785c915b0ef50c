"""GPU parity: the embedding Function (token + learned position tables) vs the oracle."""
import pytest
import torch

from oracle import ops

pytestmark = pytest.mark.gpu

# (batch, seq, d, vocab, position rows or None)
CASES = [
    (4, 64, 1024, 50304, 128),   # model-like, almost no token held twice
    (3, 50, 96, 17, 64),         # every token held many times
    (2, 33, 100, 40, 33),        # d not a multiple of 8: element-wise kernels
    (1, 1, 8, 1, None),
    (5, 128, 256, 300, None),    # no position table (the ALiBi configuration)
    (2, 2048, 64, 50304, 2048),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_embedding_fwd_bwd(case, dtype):
    from tritonformer_b200.embedding import Embedding
    b, t, d, v, p = case
    torch.manual_seed(0)
    ids = torch.randint(0, v, (b, t), device="cuda")
    tok = (torch.randn((v, d), device="cuda") * 0.5).to(dtype).requires_grad_(True)
    pos = (torch.randn((p, d), device="cuda") * 0.5).to(dtype).requires_grad_(True) if p else None
    out = Embedding.apply(ids, tok, pos)
    assert out.shape == (b, t, d) and out.dtype == dtype
    tok32 = tok.detach().float().requires_grad_(True)
    pos32 = pos.detach().float().requires_grad_(True) if p else None
    ref = ops.embedding(ids, tok32, pos32)
    # one rounding of an exact fp32 sum of two 16-bit values: bit-exact
    assert torch.equal(out, ref.to(dtype))
    w = torch.randn((b, t, d), device="cuda").to(dtype)
    out.backward(w)
    ref.backward(w.float())
    # fp32 sums rounded once to 16 bits: within one unit in the last place of the exact sum
    ulp = 2.0 ** -10 if dtype is torch.float16 else 2.0 ** -7
    for name, got, want in (("token", tok.grad, tok32.grad), ("position", pos.grad if p else None, pos32.grad if p else None)):
        if want is None:
            continue
        err = (got.float() - want).abs()
        assert (err <= ulp * want.abs() + 1e-6).all(), "%s table gradient: worst %g" % (name, err.max().item())
        assert torch.equal(got == 0, want == 0) or (want.abs()[got == 0] < 1e-6).all()


def test_embedding_adds_to_existing_gradients():
    """The C entry point adds to what the gradient buffers hold and leaves untouched rows alone."""
    from tritonformer_b200.embedding import embedding_backward
    b, t, d, v = 2, 16, 64, 100
    torch.manual_seed(1)
    ids = torch.randint(0, 10, (b, t), device="cuda")  # only rows 0..9 are touched
    dout = torch.randn((b, t, d), device="cuda").half()
    dtok = torch.randn((v, d), device="cuda").half()
    dpos = torch.randn((32, d), device="cuda").half()
    tok0, pos0 = dtok.clone(), dpos.clone()
    embedding_backward(ids, dout, dtok, dpos)
    want_tok = tok0.float().index_add_(0, ids.view(-1), dout.float().view(-1, d))
    want_pos = pos0.float()
    want_pos[:t] += dout.float().sum(0)
    assert torch.equal(dtok[10:], tok0[10:]) and torch.equal(dpos[t:], pos0[t:])
    assert (dtok.float() - want_tok).abs().max().item() < 2e-2
    assert (dpos.float() - want_pos).abs().max().item() < 1e-2


def test_embedding_token_out_of_range_is_reported():
    """A token id outside the table gives a zero row and a sticky status instead of a device fault."""
    from tritonformer_b200 import _lib
    from tritonformer_b200.embedding import embedding_forward
    tok = torch.ones((10, 16), device="cuda", dtype=torch.float16)
    ids = torch.tensor([[1, 10, 3, -1]], device="cuda")
    out = embedding_forward(ids, tok)
    assert _lib.lib.tfb_device_status(1) == 0x7100
    assert _lib.lib.tfb_device_status(0) == 0
    assert out[0, 0].eq(1).all() and out[0, 1].eq(0).all() and out[0, 3].eq(0).all()


def test_embedding_empty_batch():
    """No positions: nothing is launched, shapes and gradients are still well-formed."""
    from tritonformer_b200.embedding import Embedding
    tok = torch.randn((10, 16), device="cuda").half().requires_grad_(True)
    pos = torch.randn((4, 16), device="cuda").half().requires_grad_(True)
    out = Embedding.apply(torch.zeros((0, 4), device="cuda", dtype=torch.int64), tok, pos)
    assert out.shape == (0, 4, 16)
    out.sum().backward()
    assert tok.grad.eq(0).all() and pos.grad.eq(0).all()


def test_embedding_frozen_token_table_gets_no_gradient_buffer():
    """A token table that needs no gradient is neither indexed nor written; the position table still gets its sums."""
    from tritonformer_b200.embedding import Embedding
    torch.manual_seed(2)
    ids = torch.randint(0, 50, (3, 24), device="cuda")
    tok = torch.randn((50, 64), device="cuda").half()  # frozen
    pos = torch.randn((32, 64), device="cuda").half().requires_grad_(True)
    out = Embedding.apply(ids, tok, pos)
    w = torch.randn_like(out)
    out.backward(w)
    assert tok.grad is None
    want = torch.zeros((32, 64), device="cuda")
    want[:24] = w.float().sum(0)
    assert (pos.grad.float() - want).abs().max().item() < 1e-2


def test_embedding_fp32_tables_under_autocast():
    """A model kept in fp32 under autocast: the tables are cast like the inputs of the other Functions and the
    gradients come back in fp32."""
    from tritonformer_b200.embedding import Embedding
    torch.manual_seed(3)
    ids = torch.randint(0, 40, (2, 16), device="cuda")
    tok = torch.randn((40, 32), device="cuda").requires_grad_(True)
    pos = torch.randn((16, 32), device="cuda").requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.float16):
        out = Embedding.apply(ids, tok, pos)
    assert out.dtype is torch.float16
    ref = ops.embedding(ids, tok.detach().half().float(), pos.detach().half().float())
    assert torch.equal(out, ref.half())
    out.float().sum().backward()
    assert tok.grad.dtype is torch.float32 and pos.grad.dtype is torch.float32
    counts = torch.bincount(ids.view(-1), minlength=40).float()
    assert torch.equal(tok.grad, counts[:, None].expand(40, 32))
    assert torch.equal(pos.grad, torch.full((16, 32), 2.0, device="cuda"))
