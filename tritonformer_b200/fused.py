"""Fused building blocks of the transformer layer (no counterpart in the reference, which runs each of
these steps as its own kernel).  Same arithmetic as the plain Functions, fewer passes over HBM:

* `LayerNormFork`   (y, r) = (LayerNorm(x), x): the pre-LN fork.  Its backward adds the gradient that
                    arrives through the residual branch inside the LayerNorm backward kernel.
* `LinearResidual`  x @ W (+ b) + residual with the add in the GEMM epilogue.
* `QKVProjection`   the three projections of one input as one product with the concatenated weight; the
                    backward is one product for the input gradient and one for the three weight gradients.
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
        ctx.save_for_backward(x, alpha, beta, stats)
        return y, x.view_as(x)

    @staticmethod
    @amp_backward
    def backward(ctx, dy, dres):
        x, alpha, beta, stats = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        dres = dres.to(x.dtype) if dres is not None else None
        into = None
        if L.accumulating() and ctx.needs_input_grad[1] and ctx.needs_input_grad[2]:
            ga, gb = alpha.grad, beta.grad
            if ga is not None and gb is not None and ga.is_contiguous() and gb.is_contiguous() \
                    and ga.dtype == x.dtype and gb.dtype == x.dtype and ga.shape == alpha.shape == gb.shape:
                into = (ga, gb)  # the column sums are added to .grad by the kernel that folds them
        dx, dalpha, dbeta = layernorm_backward(dy.to(x.dtype), x, alpha, stats, dres, into=into,
                                               overwrite=L.overwriting())
        if into is not None and L.overwriting():
            L.note_written(*into)
        if into is not None:
            return dx, None, None, None
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
        dx, dw = L.linear_backward(dy, x, w, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        db = L.column_sum(dy) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, dy


def _adjacent_columns(parts, width):
    """True if `parts` are the column blocks [0, w), [w, 2w), ... of one row-major matrix of `width` columns."""
    first = parts[0]
    es = first.element_size()
    for i, t in enumerate(parts):
        if t is None or t.dtype != first.dtype or t.shape != first.shape or t.stride(-1) != 1:
            return False
        if t.data_ptr() != first.data_ptr() + i * first.shape[-1] * es:
            return False
        lead = t.reshape(-1, t.shape[-1]) if t.dim() > 2 else t
        if lead.stride(0) != width or (t.dim() > 2 and lead.data_ptr() != t.data_ptr()):
            return False
    return True


class QKVProjection(Function):
    """q, k, v = x Wq, x Wk, x Wv as ONE product with the concatenated weight [Wq | Wk | Wv]: the three outputs
    are column blocks of one (rows, 3 d) buffer.  When the three incoming gradients are again column blocks of
    one buffer (the attention backward allocates them that way), the input gradient and the three weight
    gradients are one product each as well; otherwise the input-gradient products are chained through the GEMM
    epilogue's addend."""

    @staticmethod
    @amp_forward
    def forward(ctx, x, wq, wk, wv):
        same = wq.shape == wk.shape == wv.shape and wq.dtype == wk.dtype == wv.dtype
        if not same:
            ctx.fused = False
            ctx.save_for_backward(x, wq, wk, wv)
            return (L.linear_forward(x, wq, None, False), L.linear_forward(x, wk, None, False),
                    L.linear_forward(x, wv, None, False))
        ctx.fused = True
        d = wq.shape[1]
        if _adjacent_columns((wq, wk, wv), 3 * d):
            # the three weights already are the column blocks of one (in, 3 d) matrix
            # (Transformer.fuse_projection_weights): no copy
            w = torch.as_strided(wq, (wq.shape[0], 3 * d), (3 * d, 1))
        else:
            w = torch.cat((wq, wk, wv), dim=1)  # (in, 3 d)
        y = L.linear_forward(x, w, None, False)
        ctx.save_for_backward(x, w, wq, wk, wv)
        return y[..., :d], y[..., d:2 * d], y[..., 2 * d:]

    @staticmethod
    @amp_backward
    def backward(ctx, dq, dk, dv):
        need = ctx.needs_input_grad
        if ctx.fused:
            x, w, wq, wk, wv = ctx.saved_tensors
            d = wq.shape[1]
            grads = [g.to(x.dtype) if g is not None else None for g in (dq, dk, dv)]
            if all(g is not None for g in grads) and _adjacent_columns(grads, 3 * d):
                rows = x.numel() // x.shape[-1]
                dy = torch.as_strided(grads[0], (rows, 3 * d), (3 * d, 1))
                dws = [None, None, None]
                pgrads = [p.grad for p in (wq, wk, wv)]
                one_product = L.accumulating() and all(need[1:4]) and all(g is not None for g in pgrads) \
                    and pgrads[0].dtype == x.dtype and pgrads[0].shape == wq.shape \
                    and _adjacent_columns(pgrads, 3 * d)
                fork = L._WeightGradFork(dy.device, need[0] and one_product)
                mark = fork.mark()
                dx = L.input_grad(dy, w, x.shape) if need[0] else None
                if one_product:
                    # the three .grad are column blocks of one (in, 3 d) matrix (GradBuckets column_blocks):
                    # one product that adds straight into it (on the side stream, beside the input gradient)
                    into = torch.as_strided(pgrads[0], (wq.shape[0], 3 * d), (3 * d, 1))

                    def product():
                        x2 = x.reshape(-1, x.shape[-1])  # (a copy, if one is needed, belongs to the stream it is used on)
                        L.gemm(x2, x2.stride(1), x2.stride(0), dy, dy.stride(0), dy.stride(1), wq.shape[0], 3 * d, rows,
                               out=into, accumulate=not L.overwriting())
                    fork.run(mark, product, (x, dy))
                    fork.join()
                    if L.overwriting():
                        L.note_written(*pgrads)
                elif any(need[1:4]):
                    dw = L.weight_grad(x, dy, w)  # (in, 3 d); w is a temporary, so this is a fresh tensor
                    for i, p in enumerate((wq, wk, wv)):
                        if not need[1 + i]:
                            continue
                        part = dw[:, i * d:(i + 1) * d]
                        if L.accumulating() and p.grad is not None and p.grad.dtype == part.dtype \
                                and p.grad.shape == part.shape:
                            p.grad.add_(part)
                        else:
                            dws[i] = part
                return (dx, *dws)
            ws = (wq, wk, wv)
        else:
            x, *ws = ctx.saved_tensors
            grads = (dq, dk, dv)
        dx = None
        if need[0]:
            for g, w_ in zip(grads, ws):
                if g is not None:
                    dx = L.input_grad(g.to(x.dtype), w_, x.shape, addend=dx, out=dx)
        dws = [L.weight_grad(x, g.to(x.dtype), w_) if (g is not None and n) else None
               for g, w_, n in zip(grads, ws, need[1:4])]
        return (dx, *dws)


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
        # the two weight gradients run on the side stream beside the input-gradient products (see linear.py)
        fork = L._WeightGradFork(dy.device, need[1] and need[3] and L._grad_goes_into_buffer(w1, x)
                                 and L._grad_goes_into_buffer(w2, x))
        m0 = fork.mark()
        dz = L.input_grad(dy, w2, act.shape, mask=act)  # hidden gradient with the ReLU mask applied
        m1 = fork.mark()
        dw2 = fork.run(m0, lambda: L.weight_grad(act, dy, w2), (act, dy)) if need[3] else None
        db2 = L.column_sum(dy) if ctx.has_bias[1] and need[4] else None
        dx = L.input_grad(dz, w1, x.shape) if need[0] else None
        dw1 = fork.run(m1, lambda: L.weight_grad(x, dz, w1), (x, dz)) if need[1] else None
        db1 = L.column_sum(dz) if ctx.has_bias[0] and need[2] else None
        fork.join()
        return dx, dw1, db1, dw2, db2, dy
