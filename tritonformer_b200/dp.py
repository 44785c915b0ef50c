"""Batch-sharded data parallelism for the fwd+bwd path: every rank holds a replica and its own
(B, T) token batch; the only exchange is the all-reduce (mean) of the parameter gradients.

The gradients of all parameters live in a few flat buffers (`.grad` of each parameter is a view
into one), so the weight-gradient GEMMs write where the collective reads and a step needs one
all-reduce per bucket instead of one per parameter.  Works over NCCL (GPU) and gloo (CPU tests).
The reference has no distributed code; this module exists because the benchmark is defined at
1, 2, 4 and 8 GPUs.
"""
from typing import List

import torch
import torch.distributed as dist


class GradBuckets:
    def __init__(self, params, bucket_bytes: int = 32 << 20, column_blocks=()):
        """`column_blocks`: tuples of 2-D parameters of one shape (in, d) whose gradients are laid out as the column
        blocks of ONE (in, len * d) matrix inside the bucket (the q/k/v projection weights: their gradients are then
        a single product that accumulates straight into the bucket)."""
        self.params = [p for p in params if p.requires_grad]
        self.buckets: List[torch.Tensor] = []
        self.members: List[list] = []  # parameters of each bucket
        self._views = []
        self._blocks = []  # (bucket index, first element, elements, parameters) of every column-block matrix
        self._written = set()  # data pointers of the .grad views that kernels overwrite (accumulate(overwrite=True))
        block_of = {}
        for blk in column_blocks:
            blk = tuple(blk)
            if len(blk) > 1 and all(q.dim() == 2 and q.shape == blk[0].shape and q.dtype == blk[0].dtype
                                    and q.requires_grad for q in blk):
                for q in blk:
                    block_of[id(q)] = blk
        groups, cur, cur_bytes = [], [], 0
        for p in reversed(self.params):  # backward produces gradients roughly in reverse order
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > bucket_bytes or cur[0].dtype != p.dtype):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            groups.append(cur)
        pad = lambda n: -(-n // 8) * 8  # keep every view 16-byte aligned
        for group in groups:
            total = sum(pad(p.numel()) for p in group)
            flat = torch.zeros(total, device=group[0].device, dtype=group[0].dtype)
            in_group = {id(p) for p in group}
            placed = set()
            off = 0
            for p in group:
                if id(p) in placed:
                    continue
                blk = block_of.get(id(p))
                if blk is not None and all(id(q) in in_group for q in blk) and p.numel() % 8 == 0:
                    rows, d = p.shape
                    mat = flat[off:off + len(blk) * p.numel()].view(rows, len(blk) * d)
                    for i, q in enumerate(blk):
                        view = mat[:, i * d:(i + 1) * d]
                        q.grad = view
                        self._views.append((q, view))
                        placed.add(id(q))
                    self._blocks.append((len(self.buckets), off, len(blk) * p.numel(), tuple(blk)))
                    off += len(blk) * pad(p.numel())
                    continue
                view = flat[off:off + p.numel()].view_as(p)
                p.grad = view
                self._views.append((p, view))
                placed.add(id(p))
                off += pad(p.numel())
            self.buckets.append(flat)
            self.members.append(list(group))

    def zero(self, skip_written: bool = False):
        """Clears the buckets.  `skip_written`: leaves out the gradients that the kernels overwrite anyway
        (`accumulate(overwrite=True)`; known once one step has run that way) and clears only the rest - the
        embedding tables, biases and the padding between views."""
        if not skip_written:
            for b in self.buckets:
                b.zero_()
            return
        for b, ranges in zip(self.buckets, self._ranges_to_clear()):
            for lo, hi in ranges:
                b[lo:hi].zero_()

    def _ranges_to_clear(self):
        written = self._written
        if getattr(self, "_clear_key", None) == len(written):
            return self._clear_ranges
        es = {id(b): b.element_size() for b in self.buckets}
        base = {id(b): b.data_ptr() for b in self.buckets}
        out = []
        for b, members in zip(self.buckets, self.members):
            keep = []  # element ranges of this bucket that are overwritten
            for p in members:
                g = p.grad
                if g is not None and g.data_ptr() in written and g.is_contiguous():
                    lo = (g.data_ptr() - base[id(b)]) // es[id(b)]
                    keep.append((lo, lo + g.numel()))
            # column blocks of one matrix are not contiguous each, but written together: the matrix as a whole
            for bi, lo, n, blk in self._blocks:
                if self.buckets[bi] is b and all(q.grad is not None and q.grad.data_ptr() in written for q in blk):
                    keep.append((lo, lo + n))
            keep.sort()
            ranges, at = [], 0
            for lo, hi in keep:
                if lo > at:
                    ranges.append((at, lo))
                at = max(at, hi)
            if at < b.numel():
                ranges.append((at, b.numel()))
            out.append(ranges)
        self._clear_key, self._clear_ranges = len(written), out
        return out

    def accumulate(self, overwrite: bool = False, defer_weight_grads: bool = False):
        """Context manager for the forward+backward of a step: the kernels that produce weight, LayerNorm and
        embedding gradients add them straight into the bucket views (`linear.accumulate_into_grad`), so no
        separate accumulation kernels run.  Clear the buckets with `zero()` at the start of a step.

        `overwrite`: linear-weight and LayerNorm gradients are written instead of added (one gradient per
        parameter and step: no shared weights, one micro-batch); after a first step run this way,
        `zero(skip_written=True)` clears only what is still added to.  `defer_weight_grads`: see
        `linear.accumulate_into_grad` (for graphs that never write a gradient tensor in place)."""
        from . import linear
        return linear.accumulate_into_grad(overwrite=overwrite, written=self._written,
                                           defer_weight_grads=defer_weight_grads)

    def check_views(self):
        """Autograd must have accumulated in place: every .grad still aliases its bucket."""
        for p, view in self._views:
            if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                raise RuntimeError("a parameter gradient left its bucket (set_to_none or replaced)")

    @staticmethod
    def reduce_bucket(b, group=None):
        """Mean of one flat bucket over the ranks of `group` (NCCL averages in the collective)."""
        if dist.get_backend(group) == "nccl":
            dist.all_reduce(b, op=dist.ReduceOp.AVG, group=group)
        else:
            dist.all_reduce(b, op=dist.ReduceOp.SUM, group=group)
            b.div_(dist.get_world_size(group))

    def all_reduce_mean(self, group=None):
        """Average every bucket over the ranks of `group`."""
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        for b in self.buckets:
            self.reduce_bucket(b, group)


class OverlappedReducer:
    """Starts each bucket's all-reduce as soon as the backward pass has produced all of its gradients.

    `stages` are the modules of the model in forward order (the transformer layers).  A hook on the
    input of stage i fires when the gradient with respect to that input exists, i.e. when every kernel
    that writes a gradient of stages i, i+1, ... has been enqueued; every bucket made only of such
    parameters is then reduced on a side stream (after an event on the compute stream), overlapping
    the rest of the backward pass.  `finish()` reduces what is left (the embeddings) and makes the
    compute stream wait for the collectives.  On CUDA the whole pattern is stream-ordered and can be
    captured in a CUDA graph together with the step.
    """

    def __init__(self, buckets: GradBuckets, stages, group=None, on_collectives=None, high_priority=False):
        """`on_collectives(active)`: called with True when the first collective of a step is enqueued and with
        False from finish(), on the thread that enqueues the kernels; the benchmark uses it to size the GEMM
        grids for the SMs the collectives leave."""
        self.buckets, self.group = buckets, group
        self.on_collectives = on_collectives
        stage_of = {}
        for i, m in enumerate(stages):
            for p in m.parameters():
                stage_of[id(p)] = i
        # a bucket is ready once the backward pass has gone below its earliest stage; parameters that
        # belong to no stage and sit before the stages (embeddings) make their bucket wait for finish()
        n = len(stages)
        order = {id(p): j for j, p in enumerate(buckets.params)}        # registration (forward) order
        first_stage_param = min((order[id(p)] for m in stages for p in m.parameters() if id(p) in order), default=0)
        self.ready_at = []
        for members in buckets.members:
            at = n
            for p in members:
                if id(p) in stage_of:
                    at = min(at, stage_of[id(p)])
                elif order[id(p)] < first_stage_param:
                    at = -1            # used before the stages (embeddings): gradient arrives last
                # else: used after the stages (final norm, head): gradient arrives first, no constraint
            self.ready_at.append(at)
        self.launched = [False] * len(buckets.buckets)
        self.enabled = True  # set False around a step that only some ranks run (no collectives then)
        # `high_priority`: the collectives' CTAs are placed ahead of waiting compute CTAs whenever an SM frees up
        self.side = (torch.cuda.Stream(priority=-1 if high_priority else 0)
                     if buckets.buckets and buckets.buckets[0].is_cuda else None)
        self._handles = [m.register_forward_pre_hook(self._make_pre_hook(i)) for i, m in enumerate(stages)]

    def _make_pre_hook(self, i):
        def pre_hook(module, args):
            x = args[0] if args else None
            # A hook on a non-leaf input runs just before the node that produced it is executed in
            # backward; by then the gradient accumulators of every later parameter have run (they have
            # the highest priority in the autograd queue).  A leaf input gives no such ordering against
            # this stage's own parameters, so its stage is left to finish().
            if isinstance(x, torch.Tensor) and x.requires_grad and not x.is_leaf:
                x.register_hook(lambda g: self._stage_done(i))
        return pre_hook

    def _reduce(self, k):
        b = self.buckets.buckets[k]
        if self.on_collectives is not None and not any(self.launched):
            self.on_collectives(True)
        self.launched[k] = True
        if self.side is not None:
            from . import linear
            linear.join_weight_grads()  # weight gradients still in flight on their side stream
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                self.buckets.reduce_bucket(b, self.group)
        else:
            self.buckets.reduce_bucket(b, self.group)

    def _stage_done(self, i):
        if not self.enabled or not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return
        for k, at in enumerate(self.ready_at):
            if not self.launched[k] and at >= i:
                self._reduce(k)

    def finish(self):
        """Call after backward(): reduces the remaining buckets and joins the side stream."""
        if self.enabled and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            for k in range(len(self.launched)):
                if not self.launched[k]:
                    self._reduce(k)
            if self.side is not None:
                torch.cuda.current_stream().wait_stream(self.side)
        if self.on_collectives is not None and any(self.launched):
            self.on_collectives(False)
        self.launched = [False] * len(self.launched)

    def remove(self):
        for h in self._handles:
            h.remove()


def broadcast_parameters(module: torch.nn.Module, src: int = 0, group=None):
    """Make every replica start from rank `src`'s parameters and buffers."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        if t.data.is_contiguous():
            dist.broadcast(t.data, src=src, group=group)
        else:  # e.g. a projection weight that is a column block of a shared buffer
            tmp = t.data.contiguous()
            dist.broadcast(tmp, src=src, group=group)
            t.data.copy_(tmp)


def shard_batch(global_ids: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank r takes sequences [r*B, (r+1)*B) of a (world*B, T) global batch."""
    assert global_ids.shape[0] % world == 0, "global batch must divide evenly over the ranks"
    per = global_ids.shape[0] // world
    return global_ids[rank * per:(rank + 1) * per]
