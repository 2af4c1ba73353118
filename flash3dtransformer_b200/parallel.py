"""Scene-sharded data parallelism over the GPUs of one node (one process per GPU, torch.distributed).

The reference has no distributed code at all.  Scenes are independent everywhere on the hot path (PSH counters,
sub-buckets and attention scopes never cross a scene... except that the reference hashes against the bounding box
and the mean scene size of the WHOLE batch, flash3dxfmr/psh/psh_main.py:100-104,117-118), so a batch is split into
contiguous runs of scenes along `seps`, balanced by point count, and every rank runs the unchanged single-GPU path
on its run.  Collectives are used only where the path has a real exchange:
  * `global_psh_stats`   6-value bounding box (min / max all-reduce) + scene count and point count, so that bucket ids
                         do not depend on the sharding;
  * `gather_rows`        variable-length all-gather of per-rank output rows;
  * `allreduce_gradients` bucketed fp32 all-reduce of parameter gradients after the backward pass;
  * `GradientBucketReducer` the same reduction overlapped with the backward pass: gradients live in flat fp32 buckets
                         and a bucket's all-reduce starts as soon as the backward has produced its last gradient.
Everything works with the `nccl` backend on CUDA tensors and with `gloo` on CPU tensors (used by the CPU tests).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_scenes(sizes: Sequence[int], world_size: int) -> List[Tuple[int, int]]:
    """Contiguous scene ranges [start, end) per rank, balanced by point count: rank r ends at the first scene
    boundary whose cumulative point count reaches (r+1)/world of the total.  Ranks may be empty when there are
    fewer scenes than ranks."""
    total = float(sum(sizes))
    bounds, acc, scene = [], 0.0, 0
    n = len(sizes)
    for r in range(world_size):
        start = scene
        target = total * (r + 1) / world_size
        while scene < n and (acc + sizes[scene] / 2.0 <= target or r == world_size - 1):
            acc += sizes[scene]
            scene += 1
        bounds.append((start, scene))
    return bounds


def shard_batch(coords: torch.Tensor, seps: torch.Tensor, rank: int, world_size: int):
    """(rows, re-based separators, (row0, row1), index of the first scene) of `rank`'s scenes.  `seps` may live on
    any device; planning is on the host.  The first-scene index goes to DeviceManagerSingleton.set_scene_base so that
    the PSH rebalance draws the same random numbers as in an unsharded run."""
    wide = seps.detach().to("cpu", torch.int64)
    sizes = torch.diff(wide, prepend=wide.new_zeros(1)).tolist()
    s0, s1 = shard_scenes(sizes, world_size)[rank]
    row0 = int(wide[s0 - 1]) if s0 > 0 else 0
    row1 = int(wide[s1 - 1]) if s1 > 0 else 0
    row1 = max(row1, row0)
    local_seps = (wide[s0:s1] - row0).to(seps.dtype).to(seps.device)
    return coords[row0:row1].contiguous(), local_seps, (row0, row1), s0


def global_psh_stats(coords: torch.Tensor, seps: torch.Tensor, group=None, total_scenes: Optional[int] = None,
                     total_points: Optional[int] = None):
    """Bounding box (fp16 min, max) and mean scene size over all ranks' scenes.  Passing them to
    `batch_bucket_scatter(..., bbox=, mean_n=)` / `Flash3D.forward(..., bbox=, mean_n=)` makes a shard's bucket ids
    identical to the ones a single process would compute for the same scenes inside the full batch.

    The box is one 6-value MAX all-reduce (the minimum travels negated) and stays on the device.  The mean scene size
    sizes the bucket tables, so it is needed on the host: a caller that knows the global batch (a data loader does)
    passes `total_scenes` / `total_points` and the step has no host synchronisation; otherwise the two counts are
    summed over the ranks and read back."""
    big = torch.finfo(torch.float32).max
    if coords.shape[0]:
        lo, hi = torch.aminmax(coords.float(), dim=0)
    else:
        lo = torch.full((3,), big, device=coords.device)
        hi = -lo
    distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    if distributed:
        box = torch.cat([-lo, hi])
        dist.all_reduce(box, op=dist.ReduceOp.MAX, group=group)
        lo, hi = -box[:3], box[3:]
    if total_scenes is not None and total_points is not None:
        return (lo.half(), hi.half()), float(total_points) / max(float(total_scenes), 1.0)
    counts = torch.tensor([float(seps.shape[0]), float(coords.shape[0])], device=coords.device)
    if distributed:
        dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=group)
    scenes, points = counts.tolist()
    return (lo.half(), hi.half()), points / max(scenes, 1.0)


def gather_rows(local: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenation over ranks of [rows_r, C] tensors with different row counts (rank order)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    n = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    counts = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(counts, n, group=group)
    counts = [int(c) for c in counts]
    width = max(counts)
    padded = local.new_zeros((width,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)


def allreduce_gradients(params, group=None, bucket_bytes: int = 64 << 20, average: bool = True) -> int:
    """Sum (or average) parameter gradients over ranks in fp32 buckets of about `bucket_bytes`.  Parameters without
    a gradient contribute zeros so that every rank issues the same collectives.  Returns the number of buckets."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return 0
    world = dist.get_world_size(group)
    params = [p for p in params if p.requires_grad]
    buckets, cur, cur_bytes = [], [], 0
    for p in params:
        cur.append(p)
        cur_bytes += p.numel() * 4
        if cur_bytes >= bucket_bytes:
            buckets.append(cur)
            cur, cur_bytes = [], 0
    if cur:
        buckets.append(cur)
    for bucket in buckets:
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float() for p in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
        off = 0
        for p in bucket:
            g = flat[off: off + p.numel()].view_as(p).to(p.dtype)
            off += p.numel()
            if p.grad is None:
                p.grad = g
            else:
                p.grad.copy_(g)
    return len(buckets)


class GradientBucketReducer:
    """Gradient all-reduce overlapped with the backward pass.

    Parameters are grouped, in reverse order of registration (the order in which a backward pass produces gradients),
    into flat fp32 buckets of about `bucket_bytes`; every parameter's `.grad` is a view into its bucket, so nothing is
    concatenated or copied.  A hook on each parameter counts finished gradients; when a bucket is complete its
    all-reduce is issued asynchronously (NCCL runs it on its own stream while the backward continues).  Buckets are
    always issued in bucket order, whichever completes first, so every rank issues the same collectives in the same
    order; `finish()` issues what is left (parameters that received no gradient contribute zeros), waits, and averages.

    Usage per step:   reducer.zero();  [micro-batch backward passes, the last one inside `with reducer.reducing():`];
                      reducer.finish();  optimizer.step()
    """

    def __init__(self, params, group=None, bucket_bytes: int = 32 << 20, average: bool = True):
        self.group = group
        self.average = average
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.params = [p for p in params if p.requires_grad]
        self.buckets = []          # (flat buffer, [params])
        self._bucket_of = {}
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            cur.append(p)
            cur_bytes += p.numel() * 4
            if cur_bytes >= bucket_bytes:
                self._make_bucket(cur)
                cur, cur_bytes = [], 0
        if cur:
            self._make_bucket(cur)
        self._armed = False
        self._pending = [0] * len(self.buckets)
        self._next = 0
        self._works = []
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params]

    def _make_bucket(self, plist):
        dev = plist[0].device
        flat = torch.zeros(sum(p.numel() for p in plist), dtype=torch.float32, device=dev)
        off = 0
        for p in plist:
            view = flat[off: off + p.numel()].view_as(p)
            off += p.numel()
            p.grad = view if p.dtype == torch.float32 else None
            self._bucket_of[id(p)] = (len(self.buckets), view)
        self.buckets.append((flat, list(plist)))

    def zero(self):
        """Clear every bucket (in place of optimizer.zero_grad: the gradients must stay views of the buckets)."""
        for flat, plist in self.buckets:
            flat.zero_()
            for p in plist:
                view = self._bucket_of[id(p)][1]
                if p.dtype == torch.float32 and (p.grad is None or p.grad.data_ptr() != view.data_ptr()):
                    p.grad = view
        self._pending = [len(plist) for _, plist in self.buckets]
        self._next = 0
        self._works = []

    class _Arm:
        def __init__(self, owner):
            self.owner = owner

        def __enter__(self):
            self.owner._armed = True

        def __exit__(self, *exc):
            self.owner._armed = False

    def reducing(self):
        """Context of the LAST backward pass of a step (with gradient accumulation, earlier micro-batches only add)."""
        return GradientBucketReducer._Arm(self)

    def _issue_ready(self, force: bool = False):
        while self._next < len(self.buckets) and (force or self._pending[self._next] <= 0):
            flat = self.buckets[self._next][0]
            if self.world > 1:
                self._works.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            self._next += 1

    def _on_grad(self, p):
        idx, view = self._bucket_of[id(p)]
        if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
            # autograd installed its own tensor (first gradient of a parameter whose .grad was None, or a parameter
            # that is not fp32): fold it into the bucket and point .grad back at the bucket for fp32 parameters
            view.add_(p.grad.to(torch.float32))
            p.grad = view if p.dtype == torch.float32 else None
        if not self._armed:
            return
        self._pending[idx] -= 1
        self._issue_ready()

    def finish(self) -> int:
        """Issue the remaining buckets, wait for all of them and average.  Returns the number of buckets."""
        self._issue_ready(force=True)
        for w in self._works:
            w.wait()
        self._works = []
        if self.average and self.world > 1:
            for flat, _ in self.buckets:
                flat.div_(self.world)
        for flat, plist in self.buckets:          # parameters that are not fp32 get their gradient back in their own dtype
            for p in plist:
                if p.dtype != torch.float32:
                    p.grad = self._bucket_of[id(p)][1].to(p.dtype)
        return len(self.buckets)

    def close(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []
