"""Batch sharding and the slow-weight gradient bucket for multi-GPU runs.

Every (batch, head) sequence is independent, so the path shards over the batch with no
exchange inside the recurrence.  The one collective of a training step is the sum
all-reduce of the slow-weight gradients: the callers build the per-sample state with
``W.repeat(bsz, 1, 1, 1)`` (supervised_learning/layer.py:174-177), whose backward is a sum
over the batch.  ``GradBucket`` keeps one flat fp32 buffer; each layer's per-sample state
gradients are reduced over the local batch straight into its slice (one kernel through
the C ABI on CUDA), and the bucket is all-reduced once per step.

The host logic here is backend-agnostic: with CPU tensors (gloo) the local reduction is a
plain ``sum(0)``, which is what the CPU tests exercise.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(global_batch: int, world_size: int, rank: int):
    """Contiguous batch slice [lo, hi) of ``rank``; the first ``global_batch % world_size``
    ranks take one extra sample."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("bad rank / world size")
    base, rem = divmod(global_batch, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class GradBucket:
    """Flat fp32 bucket of slow-weight gradients, all-reduced once per step."""

    def __init__(self, shapes, device):
        self.shapes = [tuple(s) for s in shapes]
        self.offsets = []
        off = 0
        for s in self.shapes:
            n = 1
            for d in s:
                n *= d
            self.offsets.append((off, n))
            off += (n + 3) // 4 * 4          # keep every slice 16-byte aligned
        self.flat = torch.zeros(off, device=device, dtype=torch.float32)
        self.work = None

    def view(self, i):
        off, n = self.offsets[i]
        return self.flat[off:off + n].view(self.shapes[i])

    def reduce_into(self, i, per_sample_grad, accumulate=False):
        """bucket[i] (+)= per_sample_grad.sum(0); per_sample_grad is [B_local, *shape]."""
        dst = self.view(i)
        if per_sample_grad.device.type == "cuda":
            from .ops import reduce_batch
            reduce_batch(per_sample_grad, dst, accumulate=accumulate)
        else:
            s = per_sample_grad.sum(0, dtype=torch.float32)
            if accumulate:
                dst.add_(s)
            else:
                dst.copy_(s)

    def all_reduce(self, group=None, async_op=False):
        """Sum over ranks (no-op without an initialised process group or at world size 1)."""
        if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        self.work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        return self.work

    def wait(self):
        if self.work is not None:
            self.work.wait()
            self.work = None
