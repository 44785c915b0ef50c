"""Softmax cross-entropy autograd Functions (drop-in for tritonformer/crossentropy.py:9-24).

`CrossEntropyLoss.apply(logits (N,V), labels (N,))` returns the per-row losses in the logits'
dtype, as the reference does.  `CrossEntropyLossFP32` is the same operator returning the
unrounded fp32 per-row losses (used by the model so the mean is taken in fp32).
A label outside [0, V) marks a row to skip: zero loss, zero gradient.
"""
import torch
from torch.autograd import Function

from . import _lib
from ._amp import amp_backward, amp_forward


def _ce_forward(ctx, logits, labels, want_f32):
    assert logits.is_cuda and logits.dim() == 2, "cross entropy expects a 2-D CUDA logits tensor"
    assert logits.dtype in (torch.float16, torch.bfloat16), "cross entropy expects fp16/bf16 logits"
    assert labels.dim() == 1 and labels.shape[0] == logits.shape[0], "labels must be (N,)"
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    labels = labels.to(torch.int64).contiguous()
    n, v = logits.shape
    loss = torch.empty((n,), device=logits.device, dtype=logits.dtype)
    extra = torch.empty((2 if want_f32 else 1, n), device=logits.device, dtype=torch.float32)
    lse = extra[0]
    loss32 = extra[1] if want_f32 else None
    _lib.check(_lib.lib.tfb_cross_entropy_fwd(
        logits.data_ptr(), labels.data_ptr(), loss.data_ptr(),
        loss32.data_ptr() if want_f32 else None, lse.data_ptr(), n, v,
        logits.stride(0) if n > 1 else v, _lib.dtype_code(logits.dtype), _lib.stream_ptr(logits.device)))
    ctx.save_for_backward(logits, labels, lse)
    return loss32 if want_f32 else loss


def _ce_backward(ctx, grad_output):
    logits, labels, lse = ctx.saved_tensors
    n, v = logits.shape
    g = grad_output.to(logits.dtype)  # keeps a stride-0 expand as it is
    gs = g.stride(0) if g.dim() == 1 and n > 1 else 0
    dlogits = torch.empty((n, v), device=logits.device, dtype=logits.dtype)
    _lib.check(_lib.lib.tfb_cross_entropy_bwd(
        logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), g.data_ptr(), gs, dlogits.data_ptr(),
        n, v, logits.stride(0) if n > 1 else v, v, _lib.dtype_code(logits.dtype),
        _lib.stream_ptr(logits.device)))
    return dlogits, None


class CrossEntropyLoss(Function):
    """Softmax Cross Entropy; per-row loss in the dtype of the logits."""

    @staticmethod
    @amp_forward
    def forward(ctx, input, labels):
        return _ce_forward(ctx, input, labels, False)

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        return _ce_backward(ctx, grad_output)


class CrossEntropyLossFP32(Function):
    """Softmax Cross Entropy; per-row loss in fp32."""

    @staticmethod
    @amp_forward
    def forward(ctx, input, labels):
        return _ce_forward(ctx, input, labels, True)

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        return _ce_backward(ctx, grad_output)
