"""Linear autograd Functions (drop-in for tritonformer/linear.py:10-102).

Weights are stored (in_features, out_features) and applied as x @ W.  Every product -- forward,
input gradient and weight gradient -- is one call of the same GEMM entry point with different
operand strides; the weight gradient contracts over all B*T rows at once in fp32 instead of
producing per-batch partials and summing them.  Bias and ReLU are applied in the GEMM epilogue.
The incoming gradient is never modified (the reference masks it in place).
"""
import collections
import os
import contextlib
import ctypes

import torch
from torch.autograd import Function

from . import _lib
from ._amp import amp_backward, amp_forward


def _as_rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 and x2.stride(0) != 1:
        x2 = x2.contiguous()
    return x2


# When set to a list, every GEMM call appends a description of itself (shape, operand strides,
# epilogue options): the benchmark replays that list to time the kernel family on its own.
PROFILE = None
# When set to a list, every GEMM call is bracketed by two CUDA events on its stream and appends
# (start, end, flops): the benchmark sums the elapsed times of one eager step to time the kernels on
# the step's own operands.
TIMING = None


def replay(calls, device):
    """Re-issues the recorded GEMM calls on scratch operands of the same shapes and strides."""
    cache = {}

    def buf(key, numel, dtype):
        t = cache.get((key, dtype))
        if t is None or t.numel() < numel:
            t = torch.randn(numel, device=device).to(dtype) * 0.05
            cache[(key, dtype)] = t
        return t

    for c in calls:
        m, n, k, dt = c["m"], c["n"], c["k"], c["dtype"]
        a = buf("a", m * k, dt)
        b = buf("b", k * n, dt)
        out = buf("c", m * n, dt)[: m * n].view(m, n)
        addend = out if c["accumulate"] else (buf("x", m * n, dt)[: m * n].view(m, n) if c["addend"] else None)
        mask = buf("m", m * n, dt)[: m * n].view(m, n) if c["mask"] else None
        bias = buf("bias", n, dt)[:n] if c["bias"] else None
        gemm(a, c["a"][0], c["a"][1], b, c["b"][0], c["b"][1], m, n, k, bias=bias, relu=c["relu"], out=out,
             addend=addend, mask=mask)


# Inside `with accumulate_into_grad():` a weight gradient is added straight into an existing, contiguous
# `.grad` by the GEMM epilogue (one rounding of accumulator + old value) and the Function reports no
# gradient for the weight, so autograd launches no separate accumulation kernel.  Off outside the block,
# because parameter hooks do not fire for gradients delivered this way; `dp.GradBuckets.accumulate()`
# is the same block for a model whose gradients live in flat buckets.
_accumulate_depth = 0
_overwrite = False
_written = None  # where the block in force records the .grad buffers that kernels WROTE (data pointers), or None


def accumulating() -> bool:
    return _accumulate_depth > 0


def overwriting() -> bool:
    return _accumulate_depth > 0 and _overwrite


def note_written(*grads):
    """Called by the kernels' wrappers for every `.grad` buffer they overwrote."""
    if _written is not None:
        for g in grads:
            _written.add(g.data_ptr())


@contextlib.contextmanager
def accumulate_into_grad(enabled: bool = True, overwrite: bool = False, written=None,
                         defer_weight_grads: bool = False):
    """Weight, LayerNorm-parameter and embedding gradients produced inside the block are added into the
    existing `.grad` buffers by the kernels that compute them.

    `overwrite`: linear-weight and LayerNorm-parameter gradients are WRITTEN to `.grad` instead of added: the
    buffers need not be cleared before the step and the product's epilogue does not read them.  Only valid when
    each such parameter receives exactly one gradient per block (no weight shared between two layers, one
    micro-batch per block); the data pointers of the buffers written are added to the set `written` when one is
    given; everything else is still added and still needs a cleared buffer."""
    global _accumulate_depth, _overwrite, _written, DEFER_WEIGHT_GRAD_JOIN
    if not enabled:
        yield
        return
    previous = (_overwrite, _written, DEFER_WEIGHT_GRAD_JOIN)
    _accumulate_depth += 1
    _overwrite, _written = bool(overwrite), (written if overwrite else None)
    DEFER_WEIGHT_GRAD_JOIN = bool(defer_weight_grads)
    try:
        yield
    finally:
        _accumulate_depth -= 1
        _overwrite, _written, DEFER_WEIGHT_GRAD_JOIN = previous
        join_weight_grads()


# GEMM scratch, newest last; at most _MAX_WORKSPACES are kept per process.  An entry that falls out is
# returned to the caching allocator, which hands it out again only in the order of the stream it was
# allocated on, so kernels still in flight on that stream keep their scratch.
_workspaces = collections.OrderedDict()
_MAX_WORKSPACES = 8


def _gemm_workspace(device, stream):
    """Scratch the GEMM uses to share the contraction of a tile between SMs: arrival counters (kept zero by
    the kernels, so cleared only here) and one fp32 partial tile per SM.  One per device and stream, since calls
    that share it must be stream-ordered."""
    key = (device, stream)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(int(_lib.lib.tfb_gemm_workspace_bytes()), device=device, dtype=torch.uint8)
        _workspaces[key] = ws
        while len(_workspaces) > _MAX_WORKSPACES:
            _workspaces.popitem(last=False)
    else:
        _workspaces.move_to_end(key)
    return ws


def reset_workspaces():
    """Zeroes every cached GEMM workspace.  For use after the device status word was cleared: a split product
    that gave up can leave arrival counters non-zero."""
    for ws in _workspaces.values():
        ws.zero_()


def gemm(a, a_sm, a_sk, b, b_sk, b_sn, m, n, k, bias=None, relu=False, out=None, accumulate=False,
         addend=None, mask=None):
    """C[m,n] = mask(act(sum_k A(m,k) B(k,n) + bias) + addend) with element strides for A and B.

    `addend` and `mask` are (m, n) tensors with unit inner stride; `accumulate` adds into `out`."""
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=a.dtype)
    if accumulate:
        addend = out
    path = ctypes.c_int(0)
    stream = _lib.stream_ptr(a.device)
    ws = _gemm_workspace(a.device, stream)
    if TIMING is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    _lib.check(_lib.lib.tfb_gemm_fused(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None,
        addend.data_ptr() if addend is not None else None, addend.stride(0) if addend is not None else 0,
        mask.data_ptr() if mask is not None else None, mask.stride(0) if mask is not None else 0,
        m, n, k, a_sm, a_sk, b_sk, b_sn, out.stride(0), 1 if relu else 0, _lib.dtype_code(a.dtype),
        ws.data_ptr(), ws.numel(), stream, ctypes.byref(path)))
    if TIMING is not None:
        e1.record()
        TIMING.append((e0, e1, 2.0 * m * n * k))
    if PROFILE is not None:
        PROFILE.append({"m": m, "n": n, "k": k, "a": (a_sm, a_sk), "b": (b_sk, b_sn), "bias": bias is not None,
                        "relu": bool(relu), "addend": addend is not None, "accumulate": addend is out,
                        "mask": mask is not None, "dtype": a.dtype, "path": path.value})
    return out


def _check_linear(x, w, bias):
    assert x.is_cuda and w.is_cuda, "Linear expects CUDA tensors"
    assert x.dim() >= 2 and w.dim() == 2, "Incorrect number of dimensions for LHS or RHS"
    assert x.shape[-1] == w.shape[0], (
        f"Dimension mismatch. Expected a.shape[2] ({x.shape[-1]}) to be equal to b.shape[0] ({w.shape[0]})")
    assert x.dtype in (torch.float16, torch.bfloat16) and w.dtype == x.dtype, "Linear expects matching fp16/bf16"
    if bias is not None:
        assert bias.dtype == x.dtype and bias.numel() == w.shape[1], "bias must be (out_features,)"


def linear_forward(x, w, bias, relu, residual=None):
    _check_linear(x, w, bias)
    x2 = _as_rows(x)
    if w.stride(0) != 1 and w.stride(1) != 1:
        w = w.contiguous()
    m, k = x2.shape
    n = w.shape[1]
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, n)
        if res2.stride(1) != 1:
            res2 = res2.contiguous()
    y = gemm(x2, x2.stride(0), x2.stride(1), w, w.stride(0), w.stride(1), m, n, k,
             bias=bias.contiguous() if bias is not None else None, relu=relu, addend=res2)
    return y.view(*x.shape[:-1], n)


def input_grad(dy, w, x_shape, mask=None, addend=None, out=None):
    """dX = dY Wᵀ (optionally masked by a saved ReLU output, optionally added to `addend`)."""
    dy2 = _as_rows(dy)
    m, n = dy2.shape
    k = w.shape[0]
    m2 = mask.reshape(m, k) if mask is not None else None
    a2 = addend.reshape(m, k) if addend is not None else None
    o2 = out.reshape(m, k) if out is not None else None
    # B(kk, nn) = W[nn, kk]
    return gemm(dy2, dy2.stride(0), dy2.stride(1), w, w.stride(1), w.stride(0), m, k, n, mask=m2, addend=a2,
                out=o2).view(x_shape)


def weight_grad(x, dy, w):
    """dW = Xᵀ dY over every row of the flattened batch.  Returns None when the product was added
    straight into `w.grad` (see accumulate_into_grad)."""
    x2, dy2 = _as_rows(x), _as_rows(dy)
    m, k = x2.shape
    n = dy2.shape[1]
    into = None
    if accumulating() and w.grad is not None and w.grad.is_contiguous() and w.grad.dtype == x.dtype \
            and w.grad.shape == (k, n):
        into = w.grad
    # A(mm, kk) = X[kk, mm]
    dw = gemm(x2, x2.stride(1), x2.stride(0), dy2, dy2.stride(0), dy2.stride(1), k, n, m, out=into,
              accumulate=into is not None and not overwriting())
    if into is not None and overwriting():
        note_written(into)
    return None if into is not None else dw


# The two products of a linear layer's backward are independent.  When the weight gradient goes straight into an
# existing `.grad` buffer (so that nothing is allocated for it), it is launched on a side stream: both products are
# persistent kernels that fill every SM, and on one stream the second can only start when the first has ended
# completely, paying its start-up after the other's last epilogue; side by side, its CTAs take over the SMs one by
# one as the first kernel's CTAs finish.  The compute stream joins the side stream before the backward function
# returns, so the operands cannot be recycled under the side kernel.
# `accumulate_into_grad(defer_weight_grads=True)` goes one step further: the compute stream does not wait at the end
# of each backward function but only where the gradients are needed - at the end of the block and before a bucket
# is reduced (`join_weight_grads`) - so the weight-gradient products fill the gaps of the whole backward pass.  Their
# operands are marked as in use by the side stream (`record_stream`), which keeps the allocator from recycling them
# under the side kernels; what nothing guards against is a later IN-PLACE write to such an operand on the compute
# stream (autograd adds a second gradient contribution into the first one's buffer when it can), so this is for
# graphs whose gradient tensors are only read after they were handed to a linear layer's backward - the fused
# blocks of `transformer.py` are such a graph (the residual sums happen inside kernels, into fresh tensors).
FORK_WEIGHT_GRAD = os.environ.get("TFB_FORK_DW", "1") != "0"
DEFER_WEIGHT_GRAD_JOIN = False  # set by the accumulate_into_grad block in force
_side_streams = {}
_unjoined = {}  # (device index, compute stream handle) -> (compute stream, side stream) with work not yet joined


def join_weight_grads():
    """Makes every compute stream wait for the weight-gradient products that still run on its side stream."""
    for main, side in list(_unjoined.values()):
        main.wait_stream(side)
    _unjoined.clear()


class _WeightGradFork:
    """`mark()` before the kernels that the side work does not depend on; `run(mark, fn)` launches fn on the side
    stream after that point; `join()` makes the compute stream wait for it."""

    def __init__(self, device, enabled=True):
        self.on = bool(enabled) and FORK_WEIGHT_GRAD and accumulating() and device.type == "cuda"
        self.used = False
        if self.on:
            self.main = torch.cuda.current_stream(device)
            key = (device.index, self.main.cuda_stream)
            side = _side_streams.get(key)
            if side is None:
                side = _side_streams[key] = torch.cuda.Stream(device)
            self.side = side

    def mark(self):
        return self.main.record_event() if self.on else None

    def run(self, mark, fn, operands=()):
        if not self.on:
            return fn()
        self.side.wait_event(mark)
        with torch.cuda.stream(self.side):
            out = fn()
        self.used = True
        if DEFER_WEIGHT_GRAD_JOIN:
            for t in operands:
                t.record_stream(self.side)
        return out

    def join(self):
        if self.on and self.used:
            if DEFER_WEIGHT_GRAD_JOIN:
                _unjoined[(self.main.device.index, self.main.cuda_stream)] = (self.main, self.side)
            else:
                self.main.wait_stream(self.side)


def _grad_goes_into_buffer(w, x):
    """The conditions under which weight_grad writes into `w.grad` and returns nothing (only then may it run on the
    side stream: a tensor it allocated there would be used on the compute stream)."""
    return accumulating() and w.grad is not None and w.grad.is_contiguous() and w.grad.dtype == x.dtype \
        and w.grad.shape == w.shape and w.dim() == 2 and x.shape[-1] == w.shape[0]


def linear_backward(dy, x, w, need_dx=True, need_dw=True):
    """dX = dY Wᵀ, dW = Xᵀ dY (contraction over every row of the flattened batch)."""
    fork = _WeightGradFork(dy.device, need_dx and need_dw and _grad_goes_into_buffer(w, x))
    mark = fork.mark()
    dx = input_grad(dy, w, x.shape) if need_dx else None
    dw = fork.run(mark, lambda: weight_grad(x, dy, w), (x, dy)) if need_dw else None
    fork.join()
    return dx, dw


def relu_backward(dy, act):
    dy = dy.contiguous()
    act = act.contiguous()
    dz = torch.empty_like(dy)
    _lib.check(_lib.lib.tfb_relu_bwd(dy.data_ptr(), act.data_ptr(), dz.data_ptr(), dy.numel(),
                                     _lib.dtype_code(dy.dtype), _lib.stream_ptr(dy.device)))
    return dz


def column_sum(x):
    """Sum over every leading dimension -> (last_dim,), fp32 accumulation."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows, cols = x2.shape
    out = torch.empty((cols,), device=x.device, dtype=x.dtype)
    n = _lib.lib.tfb_colsum_partials(rows, cols)
    partials = torch.empty((n, cols), device=x.device, dtype=torch.float32)
    _lib.check(_lib.lib.tfb_colsum(x2.data_ptr(), out.data_ptr(), partials.data_ptr(), n, rows, cols,
                                   x2.stride(0) if rows > 1 else cols, _lib.dtype_code(x.dtype),
                                   _lib.stream_ptr(x.device)))
    return out


def _backward(ctx, grad_output, has_bias, has_relu):
    if has_relu:
        x, w, act = ctx.saved_tensors
        dz = relu_backward(grad_output.to(x.dtype), act)
    else:
        x, w = ctx.saved_tensors
        dz = grad_output.to(x.dtype)
    dx, dw = linear_backward(dz, x, w, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
    if not has_bias:
        return dx, dw
    db = column_sum(dz) if ctx.needs_input_grad[2] else None
    return dx, dw, db


class LinearNoBias(Function):
    """y = x @ W"""

    @staticmethod
    @amp_forward
    def forward(ctx, input, weight):
        ctx.save_for_backward(input, weight)
        return linear_forward(input, weight, None, False)

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        return _backward(ctx, grad_output, False, False)


class LinearBias(Function):
    """y = x @ W + b"""

    @staticmethod
    @amp_forward
    def forward(ctx, input, weight, bias):
        ctx.save_for_backward(input, weight)
        return linear_forward(input, weight, bias, False)

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        return _backward(ctx, grad_output, True, False)


class LinearNoBiasReLU(Function):
    """y = relu(x @ W)"""

    @staticmethod
    @amp_forward
    def forward(ctx, input, weight):
        out = linear_forward(input, weight, None, True)
        ctx.save_for_backward(input, weight, out)
        return out

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        return _backward(ctx, grad_output, False, True)


class LinearBiasReLU(Function):
    """y = relu(x @ W + b)"""

    @staticmethod
    @amp_forward
    def forward(ctx, input, weight, bias):
        out = linear_forward(input, weight, bias, True)
        ctx.save_for_backward(input, weight, out)
        return out

    @staticmethod
    @amp_backward
    def backward(ctx, grad_output):
        return _backward(ctx, grad_output, True, True)
