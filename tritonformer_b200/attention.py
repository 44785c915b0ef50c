"""Causal attention autograd Functions (drop-in for tritonformer/attention.py:13-60).

q, k, v are (B, H, T, head_dim) with any {b,h,t} strides (the model passes strided views of its
(B, T, H*head_dim) projections); the output keeps q's layout.  The saved statistic is the fp32
log-sum-exp per row.  `BiasedCausalAttention` takes either the reference's dense (H, T, T) bias
table or a (H,) tensor of ALiBi slopes; a table that is exactly the ALiBi table of
transformer.generate_alibi_mask is recognised once (per buffer) and computed in-kernel from its
slopes with the same rounding, so the table is never read again (the finding is kept on the tensor
object itself and is redone after an in-place write).
"""
import ctypes

import torch
from torch.autograd import Function

from . import _lib
from ._amp import amp_backward, amp_forward


# When set to a list, every attention forward / backward call is bracketed by two CUDA events on its stream and
# appends (start, end, "fwd" | "bwd", flops): the benchmark sums the elapsed times of an eager step.
TIMING = None


def _timed(kind, shape, call):
    if TIMING is None:
        return call()
    b, h, t, hd = shape
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = call()
    e1.record()
    TIMING.append((e0, e1, kind, (2.0 if kind == "fwd" else 5.0) * b * h * t * t * hd))  # causal: half of 4 / 10
    return out


def _check_qkv(q, k, v):
    assert q.is_cuda and q.dim() == 4, "attention expects (B, H, T, head_dim) CUDA tensors"
    assert q.shape == k.shape == v.shape, "q, k, v must have the same shape"
    assert q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype, \
        "attention expects matching fp16/bf16 inputs"
    assert q.shape[-1] in (32, 64, 128), "Only head_dims of [32,64,128] are supported."
    assert q.shape[2] % 64 == 0, "Number of elements in sequence must be a multiple of 64"


def _unit_inner(t):
    return t if t.stride(-1) == 1 else t.contiguous()


class _Bias:
    """Resolved form of the attn_bias argument."""
    __slots__ = ("slopes", "rounded", "table")

    def __init__(self, slopes=None, rounded=0, table=None):
        self.slopes, self.rounded, self.table = slopes, rounded, table


def _resolve_bias(attn_bias, heads, seq, dtype):
    if attn_bias is None:
        return _Bias()
    if attn_bias.dim() == 1:
        assert attn_bias.shape[0] == heads, \
            f"Expected attention bias to have leading dimension equal to number of heads ({heads})"
        return _Bias(slopes=attn_bias.to(torch.float32).contiguous())
    assert attn_bias.dim() == 3, "attention bias must be (H,) slopes or an (H, T, T) table"
    assert attn_bias.shape[0] == heads, \
        f"Expected attention bias to have leading dimension equal to number of heads ({heads})"
    assert attn_bias.shape[1] == attn_bias.shape[2], (
        f"Expected attention bias to be a square but got nr = {attn_bias.shape[1]} and nc = {attn_bias.shape[2]}")
    assert attn_bias.shape[1] >= seq, "attention bias is smaller than the sequence"
    # The verdict is remembered ON the tensor object (with the version counter it was taken at), so it dies
    # with the tensor: another table that later lands at the same address is a different object and is
    # examined afresh.  In-place writes bump the counter; writes through `.data` do not and are not seen.
    memo = getattr(attn_bias, "_tfb_alibi", None)
    if memo is None or memo[0] != attn_bias._version:
        memo = (attn_bias._version, _detect_alibi(attn_bias))
        attn_bias._tfb_alibi = memo
    hit = memo[1]
    if hit is not False:
        return _Bias(slopes=hit, rounded=1 if attn_bias.dtype is torch.float16 else 2)
    table = attn_bias if attn_bias.dtype == dtype else attn_bias.to(dtype)
    return _Bias(table=_unit_inner(table))


def _detect_alibi(table):
    """Returns fp32 slopes if `table` equals the ALiBi table built from them, else False.

    Costs one host synchronisation, paid once per bias buffer."""
    h, p, _ = table.shape
    if p < 2 or table.dtype not in (torch.float16, torch.bfloat16):
        return False
    slopes = -table[:, 1, 0]
    dist = -torch.tril(torch.arange(p, device=table.device).view(p, 1)
                       - torch.arange(p, device=table.device).view(1, p)).to(table.dtype)
    want = dist * slopes[:, None, None]
    lower = torch.ones((p, p), dtype=torch.bool, device=table.device).tril()
    same = bool(((table == want) | ~lower).all().item())
    return slopes.to(torch.float32).contiguous() if same else False


def attention_forward(q, k, v, bias: _Bias):
    _check_qkv(q, k, v)
    q, k, v = _unit_inner(q), _unit_inner(k), _unit_inner(v)
    b, h, t, hd = q.shape
    out = torch.empty_like(q)  # keeps q's (dense, permuted) strides
    if out.stride(-1) != 1:
        out = torch.empty(q.shape, device=q.device, dtype=q.dtype)
    lse = torch.empty((b, h, t), device=q.device, dtype=torch.float32)
    path = ctypes.c_int(0)
    tab = bias.table
    _timed("fwd", q.shape, lambda: _lib.check(_lib.lib.tfb_attention_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), b, h, t, hd,
        _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out),
        bias.slopes.data_ptr() if bias.slopes is not None else None, int(bias.rounded),
        tab.data_ptr() if tab is not None else None,
        tab.stride(0) if tab is not None else 0, tab.stride(1) if tab is not None else 0,
        _lib.dtype_code(q.dtype), _lib.stream_ptr(q.device), ctypes.byref(path))))
    return out, lse, (q, k, v)


def _are_column_blocks(q, k, v):
    """q, k, v of shape (B, H, T, hd) are the views [.., 0:d], [.., d:2d], [.., 2d:3d] of one (B, T, 3 d) tensor."""
    b, h, t, hd = q.shape
    d = h * hd
    want = (t * 3 * d, hd, 3 * d, 1)
    es = q.element_size()
    return (q.shape == k.shape == v.shape and q.stride() == want and k.stride() == want and v.stride() == want
            and k.data_ptr() == q.data_ptr() + d * es and v.data_ptr() == q.data_ptr() + 2 * d * es)


def attention_backward(d_out, out, q, k, v, lse, bias: _Bias):
    b, h, t, hd = q.shape
    d_out = _unit_inner(d_out.to(q.dtype))
    if _are_column_blocks(q, k, v):
        # q, k, v are column blocks of one (B, T, 3 H hd) projection output: lay their gradients out the same
        # way, so that the projection's backward is one product over the whole block
        grads = torch.empty((b, t, 3, h, hd), device=q.device, dtype=q.dtype)
        dq, dk, dv = (grads[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    else:
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    nbytes = _lib.lib.tfb_attention_bwd_scratch_bytes(b, h, t, hd)
    scratch = torch.empty((nbytes,), device=q.device, dtype=torch.uint8)
    path = ctypes.c_int(0)
    tab = bias.table
    _timed("bwd", q.shape, lambda: _lib.check(_lib.lib.tfb_attention_bwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(), lse.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), b, h, t, hd,
        _lib.strides3(q), _lib.strides3(k), _lib.strides3(v), _lib.strides3(out), _lib.strides3(d_out),
        _lib.strides3(dq), _lib.strides3(dk), _lib.strides3(dv),
        bias.slopes.data_ptr() if bias.slopes is not None else None, int(bias.rounded),
        tab.data_ptr() if tab is not None else None,
        tab.stride(0) if tab is not None else 0, tab.stride(1) if tab is not None else 0,
        scratch.data_ptr(), nbytes, _lib.dtype_code(q.dtype), _lib.stream_ptr(q.device),
        ctypes.byref(path))))
    return dq, dk, dv


class CausalAttention(Function):
    """softmax(causal(q kᵀ / sqrt(hd))) v"""

    @staticmethod
    @amp_forward
    def forward(ctx, query, key, value):
        out, lse, (q, k, v) = attention_forward(query, key, value, _Bias())
        ctx.save_for_backward(lse, q, k, v, out)
        return out

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        lse, q, k, v, out = ctx.saved_tensors
        return attention_backward(grad_output, out, q, k, v, lse, _Bias())


class BiasedCausalAttention(Function):
    """softmax(causal(q kᵀ / sqrt(hd) + bias)) v; no gradient for the bias; no autocast handling."""

    @staticmethod
    def forward(ctx, query, key, value, attn_bias):
        bias = _resolve_bias(attn_bias, query.shape[1], query.shape[2], query.dtype)
        out, lse, (q, k, v) = attention_forward(query, key, value, bias)
        ctx.save_for_backward(lse, q, k, v, out)
        ctx.bias = bias
        return out

    @staticmethod
    def backward(ctx, grad_output):
        lse, q, k, v, out = ctx.saved_tensors
        dq, dk, dv = attention_backward(grad_output, out, q, k, v, lse, ctx.bias)
        return dq, dk, dv, None
