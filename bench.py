#!/usr/bin/env python
"""Benchmark of the Flash3D hot path on B200.

    python bench.py --gpus N --steps K --warmup W            this build (one process per GPU; torchrun for N > 1)
    python bench.py --impl reference --gpus N --steps K ...   CPU restatement of the reference's path (rank 0 only)

A step is one forward pass of the 5-stage Flash3D hourglass backbone (channels 32/64/128/256/512, depths
2/2/2/6/2, bucket 512, scope 8, bf16) over one batch of 16 synthetic LiDAR-like scans of 120,000 points per GPU
(PSH bucketing + scatter, 28 transformer blocks of LayerNorm / QKV GEMM / bucketed attention / projection /
SwiGLU MLP, 4 sub-bucket poolings and the matching unpoolings).  With N GPUs every rank processes its own batch of
scenes (weak scaling, scenes sharded along batch_sep); the only collective in the step is the 6-value bounding-box
all-reduce that keeps bucket ids independent of the sharding.

Rank 0 prints one JSON line: whole-job points/s with inputs resident in HBM (`value`), the same metric through the
public API from pinned host buffers to a pinned host copy of the output features (`e2e`), the roofline position of the
dominant kernel family (`roofline`), the CPU restatement timed on the host cores (`cpu_baseline`) and, under `extras`,
short runs of the other configurations after the headline measurement: `strong` (the 16-scan batch sharded over the N
ranks, output rows gathered), `train_step` (forward + backward + overlapped gradient all-reduce + SGD on this rank's
share of 64 scans of 200,000 points) and, on one GPU, `attn_layer` (one attention layer forward + backward on 8 scans)
and `psh_pool` (PSH + 3 poolings + 3 unpoolings on 8 scenes of 1,000,000 points).  `--no-extras` skips them.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "points/sec (Flash3D backbone fwd)"
SCENES_PER_GPU = 16
POINTS_PER_SCENE = 120_000
CHANNELS = (32, 64, 128, 256, 512)
DEPTHS = (2, 2, 2, 6, 2)
BUCKET, SCOPE, HASH_OP = 512, 8, 2
ATTN_FWD_TRAFFIC_PER_OPERAND_BYTE = 0.9245     # dram bytes / operand bytes of the attention forward in its profiler capture


# ----------------------------------------------------------------------------------------------------- helpers
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()            # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clk, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clk = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(clocks)) if clocks else None, "sm_max_mhz": max_clk,
                "samples": len(clocks), "reasons": sorted(reasons)}


def make_batch(rank: int, scenes: int, points: int):
    from flash3dtransformer_b200 import synthetic
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [points] * scenes, seed=1000 * rank)
    return coords32.astype(np.float16), seps.astype(np.uint32)


def build_model(device):
    from flash3dtransformer_b200 import configs
    torch.manual_seed(0)
    model = configs.flash3d_backbone(CHANNELS, DEPTHS, BUCKET, SCOPE, HASH_OP)
    return model.to(device).eval()


# ------------------------------------------------------------------------------------- kernel-family timing
class FamilyTimer:
    """Wraps the operator module's entry points with CUDA events on the launching stream and records the
    algorithmic work of every call, so that per-family time shares and the dominant family's roofline position
    come from the timed region itself."""

    def __init__(self, pshattn):
        self.p = pshattn
        self.records = []
        self.enabled = False
        self._orig = {}

    def _wrap(self, name, work_fn, family):
        orig = getattr(self.p, name)
        self._orig[name] = orig

        def wrapped(*a, **kw):
            if not self.enabled:
                return orig(*a, **kw)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            r = orig(*a, **kw)
            e.record()
            flops, nbytes = work_fn(*a, **kw)
            self.records.append((family, s, e, flops, nbytes))
            return r

        setattr(self.p, name, wrapped)

    def install(self):
        def attn(Q, K, V, O, L, scopes, bucket):
            b, l, h, d = Q.shape
            w = scopes.shape[1] * bucket
            tokens = scopes.shape[0] * w * b
            return 4.0 * tokens * w * h * d, 4.0 * b * l * h * d * 2 + b * l * h * 4

        def gemm(x, w, bias, out, residual=None, nsplit=1, epilogue=0):
            m, k = x.shape
            n = w.shape[0]
            by = 2.0 * (m * k + out.numel() + (0 if residual is None else residual.numel()))
            return 2.0 * m * n * k, by

        def gemm_fused(x, w, bias, out, residual=None, nsplit=1, epilogue=0, ln_stats=None, ln_colsum=None, ln_eps=1e-5,
                       stats_out=None):
            m, k = x.shape
            n = w.shape[0]
            by = 2.0 * (m * k + out.numel() + (0 if residual is None else residual.numel()))
            by += 8.0 * m * ((ln_stats is not None) + (stats_out is not None))       # row sums read / written
            return 2.0 * m * n * k, by

        def ln(x, w, b, out, eps=1e-5, gelu=False):
            return 0.0, 4.0 * x.numel()

        def stats(x, st):
            return 0.0, 2.0 * x.numel() + 8.0 * x.shape[0]

        def pool(coord, feat, seps, maxn, S, nv, bmin, bmax, sid, soff, rsep, rcoord, rfeat, ind, ht, op):
            n = coord.shape[0]
            e = feat.element_size()
            c = feat.shape[1]
            return 0.0, n * (19.0 + c * e + c * e / S + 4)

        def unpool(res, down, up, ind, S, covered_rows=None):
            e = res.element_size()
            c = res.shape[1]
            return 0.0, res.shape[0] * (2.0 * c * e + c * e / S + 4)

        def psh(coord, *rest):
            return 0.0, 18.0 * coord.shape[0]

        self._wrap("buck_swin_fwd", attn, "attention_fwd")
        self._wrap("linear_bf16", gemm, "gemm")
        self._wrap("linear_fused", gemm_fused, "gemm")
        self._wrap("layernorm_bf16", ln, "layernorm")
        self._wrap("row_stats_bf16", stats, "layernorm")
        self._wrap("batch_subbuck_reduce", pool, "subbuck_pool")
        self._wrap("additive_unpool_fwd", unpool, "unpool")
        self._wrap("batch_psh_scatter_pad_hash", psh, "psh_scatter")

    def summary(self):
        fam = {}
        for family, s, e, flops, nbytes in self.records:
            ms = s.elapsed_time(e)
            f = fam.setdefault(family, {"ms": 0.0, "flops": 0.0, "bytes": 0.0, "launches": 0})
            f["ms"] += ms
            f["flops"] += flops
            f["bytes"] += nbytes
            f["launches"] += 1
        return fam


# ------------------------------------------------------------------------------------------- CPU restatement
def cpu_backbone_points_per_s(points: int, steps: int, warmup: int = 0):
    """Times the CPU restatement of the path (oracle/backbone_oracle.py) on one synthetic scan."""
    from flash3dtransformer_b200 import configs, synthetic
    from oracle import backbone_oracle
    torch.manual_seed(0)
    model = configs.flash3d_backbone(CHANNELS, DEPTHS, BUCKET, SCOPE, HASH_OP).eval()
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [points], seed=0)
    c16 = coords32.astype(np.float16)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for _ in range(warmup):
        backbone_oracle.flash3d_forward(model, c16, seps)
    t0 = time.perf_counter()
    for _ in range(steps):
        backbone_oracle.flash3d_forward(model, c16, seps)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return points / dt, dt, torch.get_num_threads()


def headline_config(args, world: int):
    return {"workload": f"flash3d_backbone_fwd_5stage_{args.scenes}x{args.points // 1000}k_per_gpu",
            "scenes_per_gpu": args.scenes, "points_per_scene": args.points, "channels": list(CHANNELS),
            "depths": list(DEPTHS), "bucket_size": BUCKET, "scope_size": SCOPE, "hash_op": HASH_OP,
            "parallelism": f"scene-sharded x{world}",
            "l2": "activations per layer (>= 124 MB) exceed the 126 MB L2 across a step; no explicit flush"}


def run_reference(args, rank: int):
    """The CPU arm: the same model and metric on the host cores, each step one scan of `--ref-points` points (a bounded
    sample of the workload: points/s of this path does not depend on how many scans a step holds, scenes are
    independent).  Loads no part of the CUDA library."""
    if rank != 0:
        return
    pts = args.ref_points
    value, dt, cores = cpu_backbone_points_per_s(pts, args.steps, args.warmup)
    sample = (f"each step = 1 scan of {pts} points of the workload's distribution through the full 5-stage backbone forward, "
              f"fp32 torch/numpy CPU restatement (oracle/backbone_oracle.py), {cores} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "points/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": "points/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "points/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path and cannot be built here (empty ThunderKittens "
                "submodule, attention kernels absent); this arm times the CPU restatement used as the parity oracle",
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------- GPU arm
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch.distributed as dist
    from flash3dtransformer_b200.lib import _cabi, pshattn
    from flash3dtransformer_b200.psh import batching

    _cabi.load()                                  # no fallback: fails loudly when the extension is missing
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    model = build_model(dev)
    c16, seps = make_batch(rank, args.scenes, args.points)
    n_points = int(c16.shape[0])
    host_coords = torch.from_numpy(c16).pin_memory()
    host_seps = torch.from_numpy(seps).pin_memory()
    coords = host_coords.to(dev)
    seps_dev = host_seps.to(dev)
    batching.host_seps(seps_dev)

    from flash3dtransformer_b200 import parallel

    def step(c, s):
        # bounding box over all ranks' scenes (one 6-value all-reduce when world > 1); the global scene and point counts
        # are known to every rank, so the step has no host synchronisation
        bbox, mean_n = parallel.global_psh_stats(c, s, total_scenes=args.scenes * world, total_points=n_points * world)
        with torch.no_grad():
            return model(c, None, s, bbox=bbox, mean_n=mean_n, scene_base=rank * args.scenes)

    timer = FamilyTimer(pshattn)
    timer.install()
    for _ in range(args.warmup):
        out = step(coords, seps_dev)
    torch.cuda.synchronize()
    pshattn.device_status()

    def barrier():
        if world > 1:
            dist.barrier()

    # ---- device-resident timing
    sampler = ClockSampler(local_rank)
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    launches0 = pshattn.launch_count()
    timer.enabled = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step(coords, seps_dev)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    timer.enabled = False
    launches = pshattn.launch_count() - launches0
    clocks = sampler.stop()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = ms.item() / args.steps
    pshattn.device_status()

    # ---- end to end: pinned host buffers in, the step's output features back in pinned host memory, every step.
    # The copy-back runs on its own stream into one of two host buffers, so step i+1 computes while step i's features
    # leave the device; the timed region ends when the last copy has landed.
    host_out = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream(dev)
    done = [None, None]
    main_stream = torch.cuda.current_stream(dev)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        c = host_coords.to(dev, non_blocking=True)
        # the loader's host copy of the separators travels with the device copy (psh.scan_io does the same), so the
        # layers plan their buffers without reading anything back
        s = batching.attach_host_seps(host_seps.to(dev, non_blocking=True), host_seps)
        o = step(c, s)
        if done[i % 2] is not None:
            done[i % 2].synchronize()                    # the host buffer of two steps ago has been filled
        copy_stream.wait_stream(main_stream)
        with torch.cuda.stream(copy_stream):
            host_out[i % 2].copy_(o, non_blocking=True)
            o.record_stream(copy_stream)
            done[i % 2] = torch.cuda.Event()
            done[i % 2].record(copy_stream)
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_per_step = e2e_s.item() / args.steps
    d2h_bytes = int(out.numel() * out.element_size())
    out_cpu = out.cpu()
    last = host_out[(args.steps - 1) % 2]
    checksum = float(last[:n_points].float().mean())      # read on the host, outside the timed region
    if not torch.equal(last, out_cpu):
        raise RuntimeError("the features copied back in the end-to-end loop differ from the device-resident run")
    extras = None
    if not args.no_extras:
        del out, o, host_out, last, out_cpu, model, coords
        torch.cuda.empty_cache()
        extras = run_extras(args, rank, world, local_rank)

    if rank != 0:
        return
    fam = timer.summary()
    total_fam_ms = sum(f["ms"] for f in fam.values()) or 1.0
    peaks = measured_peaks()
    dominant = max(fam, key=lambda k: fam[k]["ms"]) if fam else None
    roofline = None
    if dominant:
        f = fam[dominant]
        sec = f["ms"] * 1e-3
        traffic = None
        if dominant == "attention_fwd":
            achieved, peak, unit, bound = f["flops"] / sec / 1e12, peaks["tflops"], "TFLOP/s", "tensor"
            # DRAM read + write bytes of this kernel from a profiler capture of a smaller launch of the same kernel
            # (2 scans instead of 16: 236.2 MB measured against 255.5 MB of operands), scaled to this launch by its
            # operand bytes; traffic grows in proportion to the tokens because every CTA reads its own Q / K / V once
            traffic = ATTN_FWD_TRAFFIC_PER_OPERAND_BYTE * f["bytes"] / f["launches"]
        else:
            achieved, peak, unit, bound = f["bytes"] / sec / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
        roofline = {"kernel": dominant, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                    "frac": achieved / peak, "traffic": traffic,
                    "traffic_source": "profiler capture of a smaller launch, scaled by operand bytes" if traffic else None,
                    "peak_source": peaks["source"],
                    "launches": f["launches"], "avg_launch_ms": f["ms"] / f["launches"],
                    "share_of_kernel_time": f["ms"] / total_fam_ms}
    kernels = {k: {"ms_per_step": v["ms"] / args.steps, "share": v["ms"] / total_fam_ms,
                   "launches_per_step": v["launches"] / args.steps,
                   "tflops": v["flops"] / (v["ms"] * 1e-3) / 1e12 if v["ms"] else 0.0,
                   "gbs": v["bytes"] / (v["ms"] * 1e-3) / 1e9 if v["ms"] else 0.0} for k, v in fam.items()}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        v, dt, cores = cpu_backbone_points_per_s(args.ref_points, 1, 0)
        cpu = {"value": v, "unit": "points/s", "cores": cores, "kind": "port",
               "sample": f"1 scan of {args.ref_points} points, full backbone forward, fp32 torch/numpy CPU restatement, "
                         f"{dt:.1f} s"}
    total_points = n_points * world
    line = {
        "metric": METRIC, "value": total_points / (ms_per_step * 1e-3), "unit": "points/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(args, world),
        "e2e": {"value": total_points / e2e_per_step, "unit": "points/s", "h2d_bytes_per_step": int(c16.nbytes + seps.nbytes),
                "d2h_bytes_per_step": d2h_bytes, "ms_per_step": e2e_per_step * 1e3, "checksum": checksum,
                "result": "output features [rows, 32] bf16 copied to pinned host memory every step (copy overlapped with the next step)"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "kernels": kernels,
        "cpu_baseline": cpu,
        "extras": extras,
    }
    print(json.dumps(line), flush=True)


def run_extras(args, rank: int, world: int, local_rank: int):
    """Short runs of the other configurations, after the headline's timed regions; every rank takes part in the
    multi-GPU ones, rank 0 returns the results."""
    import copy
    import torch.distributed as dist
    res = {}
    ex = copy.copy(args)
    ex.steps, ex.warmup = 3, 3
    t0 = time.perf_counter()
    res["strong"] = strong_scaling_measure(ex, rank, world, local_rank)
    torch.cuda.empty_cache()
    tr = copy.copy(args)
    tr.steps, tr.warmup = 3, 1
    tr.scenes, tr.points = max(1, 64 // world), 200_000
    tr.micro_scenes = min(8, tr.scenes)
    res["train_step"] = train_step_measure(tr, rank, world, local_rank)
    torch.cuda.empty_cache()
    if world == 1:
        al = copy.copy(args)
        al.steps, al.warmup = 5, 3
        res["attn_layer"] = attn_layer_measure(al)
        torch.cuda.empty_cache()
        pp = copy.copy(args)
        pp.steps, pp.warmup, pp.points = 5, 3, POINTS_PER_SCENE
        res["psh_pool"] = psh_pool_measure(pp)
        torch.cuda.empty_cache()
        res["graphed_forward"] = graphed_forward_measure(local_rank)
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    res["seconds"] = time.perf_counter() - t0
    return res if rank == 0 else None


def graphed_forward_measure(local_rank: int):
    """The backbone forward of ONE 20,000-point scan (the size of the CPU-runnable configuration), issued kernel by kernel
    and replayed as one CUDA graph (flash3dtransformer_b200.graph.GraphedForward): at this size the host's launches take
    longer than the kernels.  Latency per forward, device-timed, coordinates already on the device."""
    from flash3dtransformer_b200 import graph
    from flash3dtransformer_b200.psh import batching
    dev = torch.device(f"cuda:{local_rank}")
    model = build_model(dev)
    c16, seps = make_batch(0, 1, 20_000)
    coords = torch.from_numpy(c16).to(dev)
    host = torch.from_numpy(seps)
    seps_dev = batching.attach_host_seps(host.to(dev), host)

    def eager():
        with torch.no_grad():
            return model(coords, None, seps_dev)

    def timed(fn, n=30, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    ms_eager = timed(eager)
    ref = eager().clone()
    gf = graph.GraphedForward(model, coords, seps_dev)
    ms_graph = timed(lambda: gf(coords))
    same = bool(torch.equal(gf(coords), ref))
    torch.cuda.synchronize()
    return {"workload": "backbone forward, 1 scan x 20,000 points", "ms_per_forward_eager": ms_eager,
            "ms_per_forward_graph": ms_graph, "points_per_s_graph": 20_000 / (ms_graph * 1e-3), "same_bits": same}


def strong_scaling_measure(args, rank: int, world: int, local_rank: int):
    """The 16 x 120k-point batch of the headline as ONE global batch: sharded by scene over the ranks
    (parallel.shard_batch), forward on every rank's shard, output rows of all ranks gathered (parallel.gather_rows).
    Fixed total work: strong scaling.  Reports ms/step and the gather's share."""
    import torch.distributed as dist
    from flash3dtransformer_b200 import parallel
    from flash3dtransformer_b200.psh import batching
    dev = torch.device(f"cuda:{local_rank}")
    model = build_model(dev)
    c16, seps = make_batch(0, SCENES_PER_GPU, POINTS_PER_SCENE)          # the same global batch on every rank
    coords_all = torch.from_numpy(c16)
    seps_all = torch.from_numpy(seps)
    local, lseps, (r0, r1), scene0 = parallel.shard_batch(coords_all, seps_all, rank, world)
    local = local.to(dev)
    lseps_dev = batching.attach_host_seps(lseps.to(dev), lseps)
    total_points = int(c16.shape[0])
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]

    def step(timed):
        bbox, mean_n = parallel.global_psh_stats(local, lseps_dev, total_scenes=SCENES_PER_GPU, total_points=total_points)
        with torch.no_grad():
            o = model(local, None, lseps_dev, bbox=bbox, mean_n=mean_n, scene_base=scene0)
        if timed:
            ev[2].record()
        g = parallel.gather_rows(o)
        if timed:
            ev[3].record()
        return g

    for _ in range(args.warmup):
        g = step(False)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    gather_ms = 0.0
    ev[0].record()
    for _ in range(args.steps):
        g = step(True)
        torch.cuda.synchronize()
        gather_ms += ev[2].elapsed_time(ev[3])
    ev[1].record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([ev[0].elapsed_time(ev[1]), gather_ms], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = ms[0].item() / args.steps
    return {"metric": METRIC, "value": total_points / (ms_per_step * 1e-3), "unit": "points/s", "n_gpus": world,
            "scaling": "strong", "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "gather_ms_per_step": ms[1].item() / args.steps, "gathered_rows": int(g.shape[0]),
            "gathered_bytes": int(g.numel() * g.element_size()),
            "config": {"workload": f"flash3d_backbone_fwd_5stage_{SCENES_PER_GPU}x{POINTS_PER_SCENE // 1000}k_global_batch",
                       "parallelism": f"scene-sharded x{world}, outputs all-gathered"}}


# ------------------------------------------------------------------------------- secondary workloads (1 GPU)
def _time_ms(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_attn_layer(args):
    print(json.dumps(attn_layer_measure(args)), flush=True)


def attn_layer_measure(args):
    """One bucketed-attention layer forward + backward on 8 LiDAR-like scans of 120,000 points: dim 256, 8 heads x
    head_dim 32, bf16, bucket 512 (scope of one bucket).  Reports tokens/s and the attention kernels' TFLOP/s."""
    from flash3dtransformer_b200.lib import pshattn
    dev = torch.device("cuda:0")
    peaks = measured_peaks()
    ks = args.layer_scope
    l, h, d, c, bucket = args.layer_scenes * 120000 // (512 * ks) * (512 * ks), 8, 32, 256, 512
    g = torch.Generator(dev).manual_seed(0)
    x = torch.randn(l, c, device=dev, generator=g).bfloat16()
    wqkv = (torch.randn(3 * c, c, device=dev, generator=g) / c ** 0.5).bfloat16()
    wp = (torch.randn(c, c, device=dev, generator=g) / c ** 0.5).bfloat16()
    bqkv, bp = torch.zeros(3 * c, device=dev), torch.zeros(c, device=dev)
    scopes = torch.arange(l // bucket, dtype=torch.int64).reshape(-1, ks).to(torch.uint32).to(dev)
    qkv = torch.empty(3, l, c, device=dev, dtype=torch.bfloat16)
    o = torch.empty(1, l, h, d, device=dev, dtype=torch.bfloat16)
    lse = torch.zeros(1, l, h, device=dev)
    out = torch.empty(l, c, device=dev, dtype=torch.bfloat16)
    do = torch.randn(1, l, h, d, device=dev, generator=g).bfloat16()
    delta = torch.zeros(1, l, h, device=dev)
    dq, dk, dv = (torch.zeros_like(o) for _ in range(3))
    q, k, v = (qkv[i].view(1, l, h, d) for i in range(3))

    def fwd_attn():
        pshattn.buck_swin_fwd(q, k, v, o, lse, scopes, bucket)

    def bwd_attn():
        pshattn.buck_swin_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, scopes, bucket)

    def layer():
        pshattn.linear_bf16(x, wqkv, bqkv, qkv, nsplit=3)
        fwd_attn()
        pshattn.linear_bf16(o.view(l, c), wp, bp, out)
        bwd_attn()
        # gradients of the two projections (plain library GEMMs, as in the layer's autograd backward)
        gx = out @ wp
        gw = out.t() @ o.view(l, c)
        gq = qkv.permute(1, 0, 2).reshape(l, 3 * c)
        gx2 = gq @ wqkv
        gw2 = gq.t() @ x
        return gx, gw, gx2, gw2

    t_f = _time_ms(fwd_attn, args.steps, args.warmup)
    t_b = _time_ms(bwd_attn, args.steps, args.warmup)
    t_l = _time_ms(layer, args.steps, args.warmup)
    pshattn.device_status()
    flops_f = 4.0 * l * bucket * ks * h * d
    line = {
        "metric": "tokens/sec (bucketed-attention layer fwd+bwd)", "value": l / (t_l * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_l, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": f"attn_layer_fwd_bwd_{args.layer_scenes}x120k_dim256_h8_d32_bucket512_scope{ks}"},
        "attention_fwd": {"ms": t_f, "tflops": flops_f / (t_f * 1e-3) / 1e12, "frac_of_peak": flops_f / (t_f * 1e-3) / 1e12 / peaks["tflops"]},
        "attention_bwd": {"ms": t_b, "tflops": 2.5 * flops_f / (t_b * 1e-3) / 1e12,
                          "frac_of_peak": 2.5 * flops_f / (t_b * 1e-3) / 1e12 / peaks["tflops"]},
        "peak_tflops": peaks["tflops"], "peak_source": peaks["source"],
    }
    return line


def run_gemm_mix(args):
    """The projection GEMMs of one backbone forward (16 x 120k points: qkv, proj, fc1 with SwiGLU, fc2 at the five
    levels), each timed alone.  `--level L` restricts to one level (for a small profiler capture)."""
    from flash3dtransformer_b200.lib import pshattn
    dev = torch.device("cuda:0")
    peaks = measured_peaks()
    g = torch.Generator(dev).manual_seed(0)
    levels = [(1941504, 32, 4), (974848, 64, 4), (487424, 128, 4), (245760, 256, 12), (122880, 512, 4)]
    if args.level >= 0:
        levels = [levels[args.level]]
    # The measured HBM peak is a copy: half reads, half writes.  A pure store stream is slower on this part, and the
    # projections that write more than they read are bound by it, so it is measured here (a 1 GB fill) and each shape
    # gets a second roofline: the slower of (all bytes at the copy peak) and (written bytes at the store peak).
    fill = torch.empty(500_000_000, dtype=torch.bfloat16, device=dev)
    store_gbs = fill.numel() * 2 / _time_ms(lambda: fill.fill_(1.0), 10, 3) / 1e6
    del fill
    rows, total_ms, roof_ms, roof_store_ms = [], 0.0, 0.0, 0.0
    for m, c, blocks in levels:
        m = m // args.shrink
        for name, n, k, ns, epi, res in (("qkv", 3 * c, c, 3, 0, False), ("proj", c, c, 1, 0, True),
                                         ("fc1_swiglu", 8 * c, c, 1, 2, False), ("fc2", c, 4 * c, 1, 0, True)):
            a = torch.randn(m, k, device=dev, generator=g).bfloat16()
            w = (torch.randn(n, k, device=dev, generator=g) / k ** 0.5).bfloat16()
            b = torch.randn(n, device=dev, generator=g)
            out_n = n // 2 if epi == 2 else n
            out = torch.empty(m, out_n, device=dev, dtype=torch.bfloat16)
            r = torch.randn(m, out_n, device=dev, generator=g).bfloat16() if res else None
            t = _time_ms(lambda: pshattn.linear_bf16(a, w, b, out, residual=r, nsplit=ns, epilogue=epi), args.steps, args.warmup)
            byt = 2.0 * (m * k + m * out_n + (m * out_n if res else 0))
            flop = 2.0 * m * n * k
            roof = max(byt / (peaks["hbm_gbs"] * 1e9), flop / (peaks["tflops"] * 1e12)) * 1e3
            roof_store = max(roof, 2.0 * m * out_n / (store_gbs * 1e9) * 1e3)
            rows.append({"shape": f"{name} M={m} N={n} K={k}", "ms": t, "gbs": byt / t / 1e6, "tflops": flop / t / 1e9,
                         "roofline_ms": roof, "frac": roof / t, "roofline_store_ms": roof_store, "frac_store": roof_store / t})
            total_ms += t * blocks
            roof_ms += roof * blocks
            roof_store_ms += roof_store * blocks
    pshattn.device_status()
    print(json.dumps({"metric": "ms of projection GEMMs per backbone forward", "value": total_ms, "unit": "ms", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": "gemm_mix_backbone_16x120k", "level": args.level, "shrink": args.shrink},
                      "roofline": {"bound": "hbm", "roofline_ms": roof_ms, "frac": roof_ms / total_ms, "peak_source": peaks["source"],
                                   "store_peak_gbs_measured_here": store_gbs, "roofline_store_ms": roof_store_ms,
                                   "frac_store": roof_store_ms / total_ms},
                      "shapes": rows}), flush=True)


def run_train_step(args, rank: int, world: int, local_rank: int):
    line = train_step_measure(args, rank, world, local_rank)
    if rank == 0:
        print(json.dumps(line), flush=True)


def train_step_measure(args, rank: int, world: int, local_rank: int):
    """Backbone forward + backward + gradient all-reduce + SGD step (the backward configuration): `--scenes` scans of
    `--points` points per GPU, scene-sharded; NCCL carries only the PSH bounding box and the gradient all-reduce, which
    is issued bucket by bucket from gradient hooks while the backward pass of the last micro-batch is still running.
    `grad_allreduce_exposed_ms_per_step` is the time between the end of that backward pass and the last bucket."""
    import torch.distributed as dist
    from flash3dtransformer_b200 import parallel
    from flash3dtransformer_b200.lib import _cabi, pshattn
    from flash3dtransformer_b200.psh import batching
    _cabi.load()
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    model = build_model(dev).train()
    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    reducer = parallel.GradientBucketReducer(model.parameters())
    c16, seps = make_batch(rank, args.scenes, args.points)
    coords = torch.from_numpy(c16).to(dev)
    seps_dev = torch.from_numpy(seps).to(dev)
    batching.host_seps(seps_dev)
    # micro-batches of whole scenes: gradients accumulate over them, so a rank's share of a large batch (64 scenes of
    # 200k points on one GPU) runs in the memory of one micro-batch; every micro-batch uses the global PSH statistics
    micro = args.micro_scenes if args.micro_scenes > 0 else args.scenes
    chunks = []
    for s0 in range(0, args.scenes, micro):
        s1 = min(args.scenes, s0 + micro)
        lo = int(seps[s0 - 1]) if s0 else 0
        sp = torch.from_numpy((seps[s0:s1].astype(np.int64) - lo).astype(np.uint32)).to(dev)
        batching.host_seps(sp)
        chunks.append((coords[lo:int(seps[s1 - 1])], sp, rank * args.scenes + s0))
    total_rows = float(coords.shape[0])
    n_params = sum(p.numel() for p in model.parameters())
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    t_ar = [0.0]

    def step(timed: bool):
        reducer.zero()
        bbox, mean_n = parallel.global_psh_stats(coords, seps_dev, total_scenes=args.scenes * world,
                                                 total_points=args.scenes * args.points * world)
        loss = None
        for i, (c, sp, base) in enumerate(chunks):
            out = model(c, None, sp, bbox=bbox, mean_n=mean_n, scene_base=base)
            part = out.float().square().mean() * (c.shape[0] / total_rows)
            if i == len(chunks) - 1:
                with reducer.reducing():          # buckets leave as soon as their last gradient exists
                    part.backward()
            else:
                part.backward()
            loss = part.detach() if loss is None else loss + part.detach()
        if timed:
            ev[2].record()
        reducer.finish()
        if timed:
            ev[3].record()
        opt.step()
        return loss

    for _ in range(args.warmup):
        loss = step(False)
    torch.cuda.synchronize()
    pshattn.device_status()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ar_ms = 0.0
    ev[0].record()
    for _ in range(args.steps):
        loss = step(True)
        torch.cuda.synchronize()
        ar_ms += ev[2].elapsed_time(ev[3])
    ev[1].record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([ev[0].elapsed_time(ev[1]), ar_ms], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    pshattn.device_status()
    reducer.close()
    ms_per_step = ms[0].item() / args.steps
    pts = args.scenes * args.points * world
    return {"metric": "points/sec (Flash3D backbone fwd+bwd+SGD)", "value": pts / (ms_per_step * 1e-3), "unit": "points/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if args.scenes * world == 64 else "weak", "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"flash3d_backbone_train_step_{args.scenes}x{args.points // 1000}k_per_gpu",
                       "global_batch_scenes": args.scenes * world, "micro_batch_scenes": micro, "parameters": n_params,
                       "grad_allreduce_bytes": 4 * n_params, "grad_buckets": len(reducer.buckets)},
            "peak_memory_gb": torch.cuda.max_memory_allocated(dev) / 1e9,
            "grad_allreduce_exposed_ms_per_step": ms[1].item() / args.steps, "loss": float(loss.detach())}


def run_psh_pool(args):
    print(json.dumps(psh_pool_measure(args)), flush=True)


def psh_pool_measure(args):
    """PSH build + scatter, three rounds of stride-2 sub-bucket pooling and the matching unpools on 8 scenes of
    1,000,000 points with heavy-tailed (Zipf 1.5) voxel occupancy, feature dim 128 fp32.  Reports points/s and the
    algorithmic HBM GB/s of every kernel family."""
    from flash3dtransformer_b200 import synthetic
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import psh_main, subbuck as sbm
    dev = torch.device("cuda:0")
    peaks = measured_peaks()
    scenes, pts, c, bucket = 8, args.points if args.points != POINTS_PER_SCENE else 1_000_000, 128, 2048
    c32, seps = synthetic.batch(synthetic.zipf_voxels, [pts] * scenes, seed=0)
    coords = torch.from_numpy(c32.astype(np.float16)).to(dev)
    sp = torch.from_numpy(seps.astype(np.uint32)).to(dev)
    n = coords.shape[0]
    feat = torch.randn(n, c, device=dev, generator=torch.Generator(dev).manual_seed(0))
    _, max_n, nb, div = psh_main.bucket_plan(sp, bucket)
    buf = psh_main.BucketScatterBuffers.create_buffers(coords, sp, bucket, n, nb)
    lo, hi = torch.aminmax(coords, dim=0)

    def psh():
        pshattn.batch_psh_scatter_pad_hash(coords, buf.bucket_id, buf.bucket_cntr, buf.bucket_offs, sp, max_n, nb, div, bucket,
                                           0xFFFF, lo, hi, buf.probe_offs, buf.bucket_cumsum, buf.scattered_coord, 0.0, 1)

    levels = []
    cc, ff, ss = coords, feat, sp
    for _ in range(3):
        sb = sbm.SubbuckBuffers.create_subbuck_buff(cc, ff, ss, 2)
        levels.append((cc, ff, ss, sb, int(sbm.calc_red_sep_sizes(ss, 1)[1].to(torch.int64).max())))
        pshattn.batch_subbuck_reduce(cc, ff, ss, int(levels[-1][4]), 2, 0xFFFF, sb.bbox_min, sb.bbox_max, sb.subbuck_id, sb.subbuck_off,
                                     sb.reduced_sep, sb.reduced_coord, sb.reduced_feat, sb.unpool_ind, 1, 1)
        cc, ff, ss = sb.reduced_coord, sb.reduced_feat, sb.reduced_sep
    ups = [torch.empty_like(lv[1]) for lv in levels]

    def pools():
        for cc_, ff_, ss_, sb_, mx in levels:
            pshattn.batch_subbuck_reduce(cc_, ff_, ss_, int(mx), 2, 0xFFFF, sb_.bbox_min, sb_.bbox_max, sb_.subbuck_id, sb_.subbuck_off,
                                         sb_.reduced_sep, sb_.reduced_coord, sb_.reduced_feat, sb_.unpool_ind, 1, 1)

    def unpools():
        down = levels[-1][3].reduced_feat
        for (cc_, ff_, ss_, sb_, mx), up in zip(reversed(levels), reversed(ups)):
            pshattn.additive_unpool_fwd(ff_, down, up, sb_.unpool_ind, 2)
            down = up

    # scatter index of the bucket order, features scattered through it and brought back to the input order
    psh()
    out2in = torch.empty(n, dtype=torch.uint32, device=dev)
    in2out = torch.empty(n, dtype=torch.uint32, device=dev)
    feat_sc, feat_back = torch.empty_like(feat), torch.empty_like(feat)

    def index():
        pshattn.scatter_index(buf.bucket_id, buf.bucket_offs, buf.bucket_cumsum, sp, out2in, in2out)

    def gathers():
        pshattn.gather_rows(feat, out2in, feat_sc)
        pshattn.gather_rows(feat_sc, in2out, feat_back)

    # scan records (x, y, z, intensity as fp32) to fp16 coordinates + intensity: the front end of a real data loader
    records = torch.cat([coords.float(), torch.rand(n, 1, device=dev)], dim=1).contiguous()
    rec_coords = torch.empty(n, 3, dtype=torch.float16, device=dev)
    rec_extra = torch.empty(n, 1, dtype=torch.float32, device=dev)

    def collate():
        pshattn.collate_points_f32(records, rec_coords, rec_extra)

    t_collate = _time_ms(collate, args.steps, args.warmup)
    if not torch.equal(rec_coords, coords):
        raise RuntimeError("collated coordinates differ from the input coordinates")
    t_psh = _time_ms(psh, args.steps, args.warmup)
    t_index = _time_ms(index, args.steps, args.warmup)
    t_gather = _time_ms(gathers, args.steps, args.warmup)
    if not torch.equal(feat_back, feat):
        raise RuntimeError("feature scatter followed by its inverse did not reproduce the input")
    t_pool = _time_ms(pools, args.steps, args.warmup)
    t_unpool = _time_ms(unpools, args.steps, args.warmup)
    rows = [lv[0].shape[0] for lv in levels]
    by_pool = sum(r * (19.0 + c * 4 + c * 4 / 2 + 4) for r in rows)
    by_unpool = sum(r * (2.0 * c * 4 + c * 4 / 2 + 4) for r in rows)
    total_ms = t_psh + t_pool + t_unpool
    fam = {"psh_scatter": {"ms": t_psh, "gbs": 18.0 * n / (t_psh * 1e-3) / 1e9},
           "collate_points": {"ms": t_collate, "gbs": 26.0 * n / (t_collate * 1e-3) / 1e9},
           "scatter_index": {"ms": t_index, "gbs": 18.0 * n / (t_index * 1e-3) / 1e9},
           "feat_scatter_and_restore": {"ms": t_gather, "gbs": 2.0 * n * (2 * c * 4 + 4) / (t_gather * 1e-3) / 1e9},
           "subbuck_pool_x3": {"ms": t_pool, "gbs": by_pool / (t_pool * 1e-3) / 1e9},
           "unpool_x3": {"ms": t_unpool, "gbs": by_unpool / (t_unpool * 1e-3) / 1e9}}
    for f in fam.values():
        f["frac_of_hbm_peak"] = f["gbs"] / peaks["hbm_gbs"]
    line = {"metric": "points/sec (PSH + 3x pool + 3x unpool)", "value": n / (total_ms * 1e-3), "unit": "points/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms, "higher_is_better": True, "dtype": "f32",
            "data": "synthetic", "config": {"workload": f"psh_pool_unpool_8x{pts // 1000}k_zipf_c128_fp32_bucket2048"},
            "kernels": fam, "peak_hbm_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"]}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scenes", type=int, default=SCENES_PER_GPU)
    ap.add_argument("--points", type=int, default=POINTS_PER_SCENE)
    ap.add_argument("--micro-scenes", type=int, default=0, help="train_step: scenes per micro-batch (gradient accumulation); 0 = all")
    ap.add_argument("--ref-points", type=int, default=20000, help="points of the CPU arm's bounded sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="backbone: skip the short runs of the other configurations")
    ap.add_argument("--workload", default="backbone", choices=["backbone", "attn_layer", "psh_pool", "gemm_mix", "train_step"],
                    help="backbone = the headline metric; the others are single-GPU side measurements")
    ap.add_argument("--layer-scenes", type=int, default=8, help="attn_layer: number of 120k-point scans (fewer for a profiler capture)")
    ap.add_argument("--layer-scope", type=int, default=1, help="attn_layer: buckets per attention scope (1 in the layer configuration, 8 in the backbone)")
    ap.add_argument("--level", type=int, default=-1, help="gemm_mix: only this backbone level (0..4)")
    ap.add_argument("--shrink", type=int, default=1, help="gemm_mix: divide the row counts (small profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "train_step":
        if world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        try:
            run_train_step(args, rank, world, local_rank)
        finally:
            if world > 1:
                import torch.distributed as dist
                dist.destroy_process_group()
        return
    if args.workload != "backbone":
        if rank == 0:
            from flash3dtransformer_b200.lib import _cabi
            _cabi.load()
            {"attn_layer": run_attn_layer, "psh_pool": run_psh_pool, "gemm_mix": run_gemm_mix}[args.workload](args)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
