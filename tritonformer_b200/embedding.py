"""Token (+ learned position) embedding as one autograd Function.

Stands in for the two `torch.nn.Embedding` lookups and their sum at the head of the reference model
(transformer.py:259-272, 311-321): one gather kernel forward; backward adds the token-table and
position-table gradients in one pass over the incoming gradient, without a sort.
"""
import torch
from torch.autograd import Function

from . import _lib
from . import linear as _linear
from ._amp import amp_backward, amp_forward


def embedding_forward(input_ids, tok, pos=None):
    assert input_ids.is_cuda and input_ids.dtype == torch.int64 and input_ids.dim() == 2, \
        "embedding expects a CUDA int64 (batch, seq) tensor of token ids"
    assert tok.dim() == 2 and tok.dtype in (torch.float16, torch.bfloat16), \
        "embedding expects a (vocab, d) fp16/bf16 table"
    batch, seq = input_ids.shape
    vocab, d = tok.shape
    if pos is not None:
        assert pos.dtype == tok.dtype and pos.dim() == 2 and pos.shape[1] == d, "position table mismatch"
        assert pos.shape[0] >= seq, "sequence longer than the position table"
        pos = pos.contiguous()
    ids = input_ids.contiguous()
    tok = tok.contiguous()
    out = torch.empty((batch, seq, d), device=tok.device, dtype=tok.dtype)
    _lib.check(_lib.lib.tfb_embedding_fwd(
        ids.data_ptr(), tok.data_ptr(), pos.data_ptr() if pos is not None else None, out.data_ptr(),
        batch, seq, d, vocab, pos.shape[0] if pos is not None else 0, _lib.dtype_code(tok.dtype),
        _lib.stream_ptr(tok.device)))
    return out


def embedding_backward(input_ids, dout, dtok, dpos=None, vocab=None):
    """ADDS the gradients to `dtok` (vocab, d) and `dpos` (>= seq, d) in place.  Either may be None (a frozen
    table); with `dtok` None the vocabulary size comes from `vocab`."""
    batch, seq = input_ids.shape
    ref = dtok if dtok is not None else dpos
    if ref is None:
        return
    d = ref.shape[1]
    vocab = dtok.shape[0] if dtok is not None else int(vocab)
    assert (dtok is None or dtok.is_contiguous()) and (dpos is None or dpos.is_contiguous())
    assert dpos is None or dpos.shape[0] >= seq, "sequence longer than the position table"
    ids = input_ids.contiguous()
    dout = dout.to(ref.dtype).contiguous()
    nbytes = int(_lib.lib.tfb_embedding_bwd_scratch_bytes(batch, seq, d, vocab))
    scratch = torch.empty(nbytes, device=ref.device, dtype=torch.uint8)
    _lib.check(_lib.lib.tfb_embedding_bwd(
        ids.data_ptr(), dout.data_ptr(), dtok.data_ptr() if dtok is not None else None,
        dpos.data_ptr() if dpos is not None else None, scratch.data_ptr(), nbytes, batch, seq, d, vocab,
        dpos.shape[0] if dpos is not None else 0, _lib.dtype_code(ref.dtype), _lib.stream_ptr(ref.device)))


def _grad_target(p):
    """(buffer to add into, whether it is p.grad itself)."""
    if _linear.accumulating() and p.grad is not None and p.grad.is_contiguous() \
            and p.grad.dtype == p.dtype and p.grad.shape == p.shape:
        return p.grad, True
    return torch.zeros_like(p, memory_format=torch.contiguous_format), False


class Embedding(Function):
    """out[b, t] = tok[input_ids[b, t]] (+ pos[t]).  `pos` may be None.

    Under autocast the tables are cast to the region's 16-bit type like the inputs of the other Functions, so
    a model kept in fp32 works; the table gradients come back in the tables' own dtype."""

    @staticmethod
    @amp_forward
    def forward(ctx, input_ids, tok, pos):
        ctx.save_for_backward(input_ids, tok, pos)
        return embedding_forward(input_ids, tok, pos)

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        input_ids, tok, pos = ctx.saved_tensors
        dtok, tok_in_place = (None, True)  # a frozen table gets no gradient buffer at all
        if ctx.needs_input_grad[1]:
            dtok, tok_in_place = _grad_target(tok)
        dpos, pos_in_place = (None, True)
        if pos is not None and ctx.needs_input_grad[2]:
            dpos, pos_in_place = _grad_target(pos)
        embedding_backward(input_ids, grad_output, dtok, dpos, vocab=tok.shape[0])
        return None, None if tok_in_place else dtok, None if pos_in_place else dpos
