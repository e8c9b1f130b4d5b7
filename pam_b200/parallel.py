"""Multi-GPU helpers for the PAM path: one process per GPU over ``torch.distributed``.

The path shards by rows with no exchange — every output row of a PAM matrix product, every element
of an elementwise op and every LayerNorm / softmax row depends on its own input row only — so the
sweeps split the row range across ranks and never communicate (`shard_rows`).  The one real
exchange of a full training step is the data-parallel gradient sum, which the reference leaves to
its frameworks' DistributedDataParallel (NCCL all-reduce); `all_reduce_gradients` is that step for
a hand-rolled loop: one flat bucket per dtype, summed in place over NVLink by NCCL (gloo on CPU);
`GradientBuckets` is the same sum started bucket by bucket while the backward pass is still running
(what DistributedDataParallel does, fairseq/models/distributed_fairseq_model.py:60-70).
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


class GradientBuckets:
    """Data-parallel gradient sum overlapped with the backward pass.

    Parameters are grouped, in reverse order of registration (roughly the order in which their
    gradients become ready), into buckets of about `bucket_bytes` (default: 25 MB, or an eighth of all
    gradients if that is less).  A hook on each parameter fires
    when its gradient has been accumulated; when the last gradient of a bucket arrives the bucket is
    flattened and its all-reduce is started asynchronously, so it travels over NVLink while the rest
    of the backward pass computes.  `finish()` waits for the reductions and copies the sums back into
    the `.grad` tensors.  The result equals `all_reduce_gradients` (a sum, optionally averaged); the
    sum of a bucket is the same collective on every rank, so replicas stay identical.

        buckets = GradientBuckets(params)        # once
        loss.backward(); buckets.finish()        # every step, before the optimizer
    """

    def __init__(self, params, bucket_bytes=None, group=None, average=False):
        self.group, self.average = group, average
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.params = [p for p in params if p.requires_grad]
        if bucket_bytes is None:
            # 25 MB as DistributedDataParallel takes, but at least eight buckets, so that a model whose
            # gradients fit one such bucket (DeiT-tiny: 23 MB) still overlaps its reduction with the backward pass
            total = sum(p.numel() * p.element_size() for p in self.params)
            bucket_bytes = min(25 << 20, max(1 << 20, total // 8))
        self.buckets, self.owner = [], {}
        current, size = [], 0
        for p in reversed(self.params):
            current.append(p)
            size += p.numel() * p.element_size()
            if size >= bucket_bytes:
                self.buckets.append(current)
                current, size = [], 0
        if current:
            self.buckets.append(current)
        for index, bucket in enumerate(self.buckets):
            for p in bucket:
                self.owner[p] = index
        self.pending = [len(b) for b in self.buckets]
        self.inflight = []
        self.handles = [p.register_post_accumulate_grad_hook(self._ready) for p in self.params] if self.active else []

    def _ready(self, param):
        index = self.owner[param]
        self.pending[index] -= 1
        if self.pending[index] == 0:
            self._launch(index)

    def _launch(self, index):
        grads = []
        for p in self.buckets[index]:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            grads.append(p.grad)
        flat = torch.cat([g.reshape(-1) for g in grads])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.inflight.append((index, flat, grads, work))

    def finish(self):
        """Completes the step's reductions (buckets whose gradients never arrived, e.g. unused
        parameters, are reduced now with zeros) and re-arms the hooks' counters."""
        if not self.active:
            return
        launched = {index for index, *_ in self.inflight}
        for index in range(len(self.buckets)):
            if index not in launched:
                self._launch(index)
        world = dist.get_world_size(self.group)
        for _, flat, grads, work in self.inflight:
            work.wait()
            if self.average:
                flat /= world
            offset = 0
            for g in grads:
                g.copy_(flat[offset:offset + g.numel()].view_as(g))
                offset += g.numel()
        self.inflight = []
        self.pending = [len(b) for b in self.buckets]

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles = []


def max_over_ranks(value, device, group=None):
    """The largest `value` on any rank (used for timing: a multi-GPU time is the slowest rank's)."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
