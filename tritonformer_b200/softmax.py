"""Softmax autograd Function over the last dimension (drop-in for tritonformer/softmax.py:6-21).

No autocast decoration, as in the reference; fp32, fp16 and bf16 inputs are accepted.  The
backward writes a new tensor instead of overwriting the incoming gradient.
"""
import torch
from torch.autograd import Function

from . import _lib


def _rows(t):
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(1) == 1 else t2.contiguous()


class Softmax(Function):
    @staticmethod
    def forward(ctx, input):
        assert input.is_cuda, "Softmax expects a CUDA tensor"
        x2 = _rows(input)
        rows, cols = x2.shape
        y = torch.empty((rows, cols), device=input.device, dtype=input.dtype)
        _lib.check(_lib.lib.tfb_softmax_fwd(x2.data_ptr(), y.data_ptr(), rows, cols,
                                            x2.stride(0) if rows > 1 else cols, cols,
                                            _lib.dtype_code(input.dtype), _lib.stream_ptr(input.device)))
        y = y.view(input.shape)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        (y,) = ctx.saved_tensors
        g2, y2 = _rows(grad_output.to(y.dtype)), _rows(y)
        rows, cols = y2.shape
        dx = torch.empty((rows, cols), device=y.device, dtype=y.dtype)
        _lib.check(_lib.lib.tfb_softmax_bwd(g2.data_ptr(), y2.data_ptr(), dx.data_ptr(), rows, cols,
                                            g2.stride(0) if rows > 1 else cols,
                                            y2.stride(0) if rows > 1 else cols, cols,
                                            _lib.dtype_code(y.dtype), _lib.stream_ptr(y.device)))
        return dx.view(y.shape)
