"""Autocast behaviour of the autograd Functions.

The reference decorates its Functions with custom_fwd(cast_inputs=torch.float16) / custom_bwd
(tritonformer/linear.py:14,20; layernorm.py:9,18; attention.py:15,24; crossentropy.py:13,20):
inside an autocast region floating CUDA tensors are cast to fp16 and the body runs with autocast
off; outside it nothing is touched.  Here the cast target is the region's own dtype when that is
bfloat16 (so a bf16 autocast region computes in bf16) and float16 otherwise.
"""
import functools

import torch


def _cast(value, dtype):
    if isinstance(value, torch.Tensor):
        if value.is_floating_point() and value.is_cuda and value.dtype is not torch.float64:
            return value.to(dtype)
        return value
    if isinstance(value, (list, tuple)):
        return type(value)(_cast(v, dtype) for v in value)
    return value


def amp_forward(fwd):
    @functools.wraps(fwd)
    def wrapper(ctx, *args):
        ctx._amp_dtype = torch.get_autocast_dtype("cuda")
        ctx._amp_used = False  # the body itself never runs under autocast
        if torch.is_autocast_enabled("cuda"):
            target = torch.bfloat16 if ctx._amp_dtype is torch.bfloat16 else torch.float16
            with torch.autocast(device_type="cuda", enabled=False):
                return fwd(ctx, *_cast(args, target))
        return fwd(ctx, *args)

    return wrapper


def amp_backward(bwd):
    @functools.wraps(bwd)
    def wrapper(ctx, *grads):
        with torch.autocast(device_type="cuda", enabled=ctx._amp_used, dtype=ctx._amp_dtype):
            return bwd(ctx, *grads)

    return wrapper
