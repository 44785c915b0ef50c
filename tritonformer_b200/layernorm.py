"""LayerNorm autograd Function (drop-in for tritonformer/layernorm.py:7-26)."""
import torch
from torch.autograd import Function

from . import _lib
from ._amp import amp_backward, amp_forward


def _rows(t: torch.Tensor) -> torch.Tensor:
    d = t.shape[-1]
    t2 = t.reshape(-1, d)
    if t2.stride(1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < d):
        t2 = t2.contiguous()
    return t2


def layernorm_forward(x, alpha, beta, eps):
    assert x.is_cuda and x.dtype in (torch.float16, torch.bfloat16), "LayerNorm expects a CUDA fp16/bf16 input"
    assert alpha.dtype == x.dtype and beta.dtype == x.dtype, "LayerNorm parameters must match the input dtype"
    d = x.shape[-1]
    assert alpha.numel() == d and beta.numel() == d, "LayerNorm parameter size mismatch"
    x2 = _rows(x)
    rows = x2.shape[0]
    y = torch.empty((rows, d), device=x.device, dtype=x.dtype)
    stats = torch.empty((2, rows), device=x.device, dtype=torch.float32)
    alpha, beta = alpha.contiguous(), beta.contiguous()
    _lib.check(_lib.lib.tfb_layernorm_fwd(
        x2.data_ptr(), alpha.data_ptr(), beta.data_ptr(), y.data_ptr(), stats[0].data_ptr(),
        stats[1].data_ptr(), rows, d, x2.stride(0) if rows > 1 else d, d, float(eps),
        _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device)))
    return y.view(x.shape), stats


def layernorm_backward(dy, x, alpha, stats, dres=None, into=None, overwrite=False):
    """dx, dalpha, dbeta; `dres` (same shape as x) is added to dx inside the kernel.  `into` = (dalpha, dbeta)
    buffers to ADD the parameter gradients to, or with `overwrite` to write them to (then returned as None,
    None)."""
    d = x.shape[-1]
    x2, dy2 = _rows(x), _rows(dy)
    r2 = _rows(dres) if dres is not None else None
    rows = x2.shape[0]
    dx = torch.empty((rows, d), device=x.device, dtype=x.dtype)
    if into is None:
        dalpha = torch.empty((d,), device=x.device, dtype=x.dtype)
        dbeta = torch.empty_like(dalpha)
    else:
        dalpha, dbeta = into
    n = _lib.lib.tfb_layernorm_bwd_partials(rows, d)
    partials = torch.empty((n, 2, d), device=x.device, dtype=torch.float32)
    alpha = alpha.contiguous()
    _lib.check(_lib.lib.tfb_layernorm_bwd_acc(
        dy2.data_ptr(), x2.data_ptr(), alpha.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(),
        r2.data_ptr() if r2 is not None else None,
        dx.data_ptr(), dalpha.data_ptr(), dbeta.data_ptr(), partials.data_ptr(), n, rows, d,
        dy2.stride(0) if rows > 1 else d, x2.stride(0) if rows > 1 else d,
        (r2.stride(0) if rows > 1 else d) if r2 is not None else 0, d,
        1 if (into is not None and not overwrite) else 0, _lib.dtype_code(x.dtype), _lib.stream_ptr(x.device)))
    if into is not None:
        return dx.view(x.shape), None, None
    return dx.view(x.shape), dalpha, dbeta


class LayerNorm(Function):
    """y = alpha * (x - mean) / sqrt(var + eps) + beta over the last dimension."""

    @staticmethod
    @amp_forward
    def forward(ctx, input, alpha, beta, eps):
        y, stats = layernorm_forward(input, alpha, beta, eps)
        ctx.save_for_backward(input, alpha, stats)
        return y

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        x, alpha, stats = ctx.saved_tensors
        dx, dalpha, dbeta = layernorm_backward(grad_output.to(x.dtype), x, alpha, stats)
        return dx, dalpha.view(alpha.shape), dbeta.view(alpha.shape), None
