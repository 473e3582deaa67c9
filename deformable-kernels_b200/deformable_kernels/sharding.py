"""Batch sharding of the deformable-kernel operators across ranks.

Every output of the path except the bank gradient depends on one sample only
(y, grad-input, offset gradients; nd-linear's output and coordinate gradient), so rank r of R
simply owns a contiguous slice of the batch and no data-path collective is needed.  The bank
gradient (and nd-linear's data gradient) is a sum over the batch: each rank holds a partial sum,
which training code all-reduces together with its other parameter gradients.
"""
import torch
import torch.distributed as dist


def shard_bounds(batch, rank, world):
    """Contiguous slice [lo, hi) of `batch` samples owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(tensors, rank, world):
    """Slice every tensor along dim 0 to this rank's share (None entries pass through)."""
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        lo, hi = shard_bounds(t.size(0), rank, world)
        out.append(t[lo:hi].contiguous())
    return out


def allreduce_bank_grad(grad, group=None, average=False):
    """Sum (or average) the per-rank partial bank gradient in place; a no-op without a process group."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=group)
        if average:
            grad.div_(dist.get_world_size(group))
    return grad
