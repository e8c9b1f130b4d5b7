"""Multi-GPU helpers for the PAM path: one process per GPU over ``torch.distributed``.

The path shards by rows with no exchange — every output row of a PAM matrix product, every element
of an elementwise op and every LayerNorm / softmax row depends on its own input row only — so the
sweeps split the row range across ranks and never communicate (`shard_rows`).  The one real
exchange of a full training step is the data-parallel gradient sum, which the reference leaves to
its frameworks' DistributedDataParallel (NCCL all-reduce); `all_reduce_gradients` is that step for
a hand-rolled loop: one flat bucket per dtype, summed in place over NVLink by NCCL (gloo on CPU).
The reference's fairseq path sums gradients and never rescales them by the sample count
(fairseq/optim/fairseq_optimizer.py:103-119 discards the product), hence ``average=False`` by
default.
"""
import torch
import torch.distributed as dist


def shard_rows(total, rank, world):
    """[start, stop) of rank's contiguous block when `total` rows are dealt as evenly as possible
    (the first total % world ranks get one extra row)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def all_reduce_gradients(params, group=None, average=False):
    """Sums (or averages) the gradients of `params` over the process group, in place, with one
    collective per dtype.  Parameters without a gradient on this rank contribute zeros, so every
    rank issues the same collective."""
    if not dist.is_available() or not dist.is_initialized():
        return
    world = dist.get_world_size(group)
    if world == 1:
        return
    params = [p for p in params if p.requires_grad]
    buckets = {}
    for p in params:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        buckets.setdefault((p.grad.dtype, p.grad.device), []).append(p.grad)
    for grads in buckets.values():
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
        offset = 0
        for g in grads:
            g.copy_(flat[offset:offset + g.numel()].view_as(g))
            offset += g.numel()


def max_over_ranks(value, device, group=None):
    """The largest `value` on any rank (used for timing: a multi-GPU time is the slowest rank's)."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
