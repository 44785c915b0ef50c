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
    def __init__(self, params, bucket_bytes: int = 256 << 20):
        self.params = [p for p in params if p.requires_grad]
        self.buckets: List[torch.Tensor] = []
        self._views = []
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
        for group in groups:
            total = sum(-(-p.numel() // 8) * 8 for p in group)  # keep every view 16-byte aligned
            flat = torch.zeros(total, device=group[0].device, dtype=group[0].dtype)
            off = 0
            for p in group:
                view = flat[off:off + p.numel()].view_as(p)
                p.grad = view
                self._views.append((p, view))
                off += -(-p.numel() // 8) * 8
            self.buckets.append(flat)

    def zero(self):
        for b in self.buckets:
            b.zero_()

    def check_views(self):
        """Autograd must have accumulated in place: every .grad still aliases its bucket."""
        for p, view in self._views:
            if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                raise RuntimeError("a parameter gradient left its bucket (set_to_none or replaced)")

    def all_reduce_mean(self, group=None, async_op: bool = False):
        """Average every bucket over the ranks of `group`."""
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return []
        world = dist.get_world_size(group)
        avg = dist.get_backend(group) == "nccl"
        works = []
        for b in self.buckets:
            if avg:
                works.append(dist.all_reduce(b, op=dist.ReduceOp.AVG, group=group, async_op=async_op))
            else:
                w = dist.all_reduce(b, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
                if async_op:
                    w.wait()
                b.div_(world)
        return works if async_op else []


def broadcast_parameters(module: torch.nn.Module, src: int = 0, group=None):
    """Make every replica start from rank `src`'s parameters and buffers."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        dist.broadcast(t.data, src=src, group=group)


def shard_batch(global_ids: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank r takes sequences [r*B, (r+1)*B) of a (world*B, T) global batch."""
    assert global_ids.shape[0] % world == 0, "global batch must divide evenly over the ranks"
    per = global_ids.shape[0] // world
    return global_ids[rank * per:(rank + 1) * per]
