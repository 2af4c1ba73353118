"""The whole inference forward as one CUDA graph.

A forward of the backbone is a few hundred kernel launches (PSH, sub-bucket build, pooling, attention, projections)
whose shapes depend only on the batch signature: the scene sizes.  For a server or a benchmark that feeds batches of one
signature, `GraphedForward` records those launches once and replays them per batch: the host then issues one graph launch
instead of every kernel, which matters for small batches, where the launches take longer than the kernels.

What makes the forward capturable: the layers plan their buffers from the host copy of the scene separators that travels
with the device copy (psh.batching.attach_host_seps), so nothing is read back from the device; the level buffers of a
signature come from the pool (psh/plan.py); the library's scratch blocks are sized by the warm-up runs on the capture
stream and pinned by the capture.  The bounding box of the batch is computed on the device inside the graph; in a
scene-sharded run, where it takes an all-reduce, the caller computes it (parallel.global_psh_stats) and passes it to every
call, and it is copied into the graph's static input.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .psh import batching


class GraphedForward:
    """model(coords, None, seps) as a CUDA graph for batches whose scene sizes equal those of `seps`.

    coords fp16 [N, 3] and seps uint32 [B] are an example batch on the model's device; seps must carry its host copy
    (attach_host_seps) or be readable once here.  `bbox` = (lo, hi) device tensors and `mean_n` as returned by
    parallel.global_psh_stats make the graph take the bounding box as an input instead of computing it."""

    def __init__(self, model: torch.nn.Module, coords: torch.Tensor, seps: torch.Tensor, *, bbox: Optional[Tuple] = None,
                 mean_n=None, scene_base=None, warmup: int = 2):
        if not coords.is_cuda:
            raise RuntimeError("GraphedForward needs a CUDA batch")
        self.model = model
        self.device = coords.device
        host = batching.host_seps(seps).clone()
        self._host_seps = host
        self.coords = coords.clone()
        self.seps = batching.attach_host_seps(seps.clone(), host)
        self._bbox = None if bbox is None else (bbox[0].clone(), bbox[1].clone())
        self._mean_n, self._scene_base = mean_n, scene_base
        self.stream = torch.cuda.Stream(self.device)
        self.graph = torch.cuda.CUDAGraph()
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream), torch.no_grad():
            # warm-up on the capture stream: kernel attributes, the library's per-stream scratch blocks, the level
            # buffers of this signature and every cached weight form exist before the capture starts
            for _ in range(max(1, warmup)):
                self._run()
        self.stream.synchronize()
        with torch.cuda.graph(self.graph, stream=self.stream), torch.no_grad():
            self.out = self._run()
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def _run(self):
        return self.model(self.coords, None, self.seps, bbox=self._bbox, mean_n=self._mean_n, scene_base=self._scene_base)

    def matches(self, seps: torch.Tensor) -> bool:
        """True when a batch with these separators has the recorded signature."""
        host = getattr(seps, "_f3d_host", None)
        host = host if host is not None else batching.host_seps(seps)
        return host.shape == self._host_seps.shape and bool(torch.equal(host.to(torch.int64), self._host_seps.to(torch.int64)))

    def __call__(self, coords: torch.Tensor, bbox: Optional[Tuple] = None) -> torch.Tensor:
        """Copy the batch into the graph's input and replay it on the current stream.  Returns the graph's output
        buffer, which the next call overwrites: consume or copy it first (work queued on the current stream is ordered
        before the next replay by the stream)."""
        if coords.shape != self.coords.shape:
            raise RuntimeError(f"GraphedForward was recorded for {tuple(self.coords.shape)} coordinates, got {tuple(coords.shape)}")
        if (bbox is None) != (self._bbox is None):
            raise RuntimeError("GraphedForward: pass a bounding box exactly when the graph was recorded with one")
        self.coords.copy_(coords, non_blocking=True)
        if bbox is not None:
            self._bbox[0].copy_(bbox[0], non_blocking=True)
            self._bbox[1].copy_(bbox[1], non_blocking=True)
        self.graph.replay()
        return self.out
