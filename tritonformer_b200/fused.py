"""Fused building blocks of the transformer layer (no counterpart in the reference, which runs each of
these steps as its own kernel).  Same arithmetic as the plain Functions, fewer passes over HBM:

* `LayerNormFork`   (y, r) = (LayerNorm(x), x): the pre-LN fork.  Its backward adds the gradient that
                    arrives through the residual branch inside the LayerNorm backward kernel.
* `LinearResidual`  x @ W (+ b) + residual with the add in the GEMM epilogue.
* `QKVProjection`   the three projections of one input; the backward chains the three input-gradient
                    products through the GEMM epilogue's addend instead of summing them afterwards.
* `MLPResidual`     relu(x W1 + b1) W2 + b2 + residual; the backward applies the ReLU mask in the
                    epilogue of the product that yields the hidden gradient.
"""
import torch
from torch.autograd import Function

from . import linear as L
from ._amp import amp_backward, amp_forward
from .layernorm import layernorm_backward, layernorm_forward


# Test hook: when set to a list, MLPResidual.forward appends the boolean activation pattern (act > 0)
# of every call, so a reference can be evaluated with the same pattern.
CAPTURE_ACTIVATION_PATTERN = None


class LayerNormFork(Function):
    @staticmethod
    @amp_forward
    def forward(ctx, x, alpha, beta, eps):
        y, stats = layernorm_forward(x, alpha, beta, eps)
        ctx.save_for_backward(x, alpha, stats)
        return y, x.view_as(x)

    @staticmethod
    @amp_backward
    def backward(ctx, dy, dres):
        x, alpha, stats = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        dres = dres.to(x.dtype) if dres is not None else None
        dx, dalpha, dbeta = layernorm_backward(dy.to(x.dtype), x, alpha, stats, dres)
        return dx, dalpha.view(alpha.shape), dbeta.view(alpha.shape), None


class LinearResidual(Function):
    @staticmethod
    @amp_forward
    def forward(ctx, x, weight, bias, residual):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return L.linear_forward(x, weight, bias, False, residual=residual)

    @staticmethod
    @amp_backward
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.to(x.dtype)
        dx = L.input_grad(dy, w, x.shape) if ctx.needs_input_grad[0] else None
        dw = L.weight_grad(x, dy, w) if ctx.needs_input_grad[1] else None
        db = L.column_sum(dy) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, dy


class QKVProjection(Function):
    @staticmethod
    @amp_forward
    def forward(ctx, x, wq, wk, wv):
        ctx.save_for_backward(x, wq, wk, wv)
        return (L.linear_forward(x, wq, None, False), L.linear_forward(x, wk, None, False),
                L.linear_forward(x, wv, None, False))

    @staticmethod
    @amp_backward
    def backward(ctx, dq, dk, dv):
        x, wq, wk, wv = ctx.saved_tensors
        dx = None
        if ctx.needs_input_grad[0]:
            for g, w in ((dq, wq), (dk, wk), (dv, wv)):
                if g is not None:
                    dx = L.input_grad(g.to(x.dtype), w, x.shape, addend=dx, out=dx)
        grads = [L.weight_grad(x, g.to(x.dtype), w) if (g is not None and need) else None
                 for g, w, need in ((dq, wq, ctx.needs_input_grad[1]), (dk, wk, ctx.needs_input_grad[2]),
                                    (dv, wv, ctx.needs_input_grad[3]))]
        return (dx, *grads)


class MLPResidual(Function):
    @staticmethod
    @amp_forward
    def forward(ctx, x, w1, b1, w2, b2, residual):
        act = L.linear_forward(x, w1, b1, True)
        if CAPTURE_ACTIVATION_PATTERN is not None:
            CAPTURE_ACTIVATION_PATTERN.append((act > 0).detach())
        y = L.linear_forward(act, w2, b2, False, residual=residual)
        ctx.save_for_backward(x, w1, w2, act)
        ctx.has_bias = (b1 is not None, b2 is not None)
        return y

    @staticmethod
    @amp_backward
    def backward(ctx, dy):
        x, w1, w2, act = ctx.saved_tensors
        dy = dy.to(x.dtype)
        need = ctx.needs_input_grad
        dz = L.input_grad(dy, w2, act.shape, mask=act)  # hidden gradient with the ReLU mask applied
        dw2 = L.weight_grad(act, dy, w2) if need[3] else None
        db2 = L.column_sum(dy) if ctx.has_bias[1] and need[4] else None
        dx = L.input_grad(dz, w1, x.shape) if need[0] else None
        dw1 = L.weight_grad(x, dz, w1) if need[1] else None
        db1 = L.column_sum(dz) if ctx.has_bias[0] and need[2] else None
        return dx, dw1, db1, dw2, db2, dy
