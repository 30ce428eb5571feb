#!/usr/bin/env python
"""Benchmark of the grouped_mm forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Metric: useful TFLOP/s of the 2D x 3D MoE grouped_mm (Mixtral-shape up-projection: 8 experts,
32768 routed rows, K=4096, N=14336, bf16 in/out, seeded multinomial-over-Dirichlet group sizes).
One step = one forward call over one batch. Prints ONE JSON line on rank 0.

  value     device-timed throughput with inputs resident in HBM (CUDA events, max over ranks)
  e2e       the same metric through the public operator with HOST buffers: pinned host inputs are
            copied to the device, the operator runs, the result is copied back, every step
  roofline  tensor-core roofline of the one kernel a step launches
  cpu_baseline  the CPU oracle (per-group fp32 torch.matmul) timed on a bounded sample
  triton_reference  the reference package's own Triton kernel on the same inputs (rank 0, N=1)

With N > 1 (torchrun, one rank per GPU) groups are sharded expert-parallel: every rank holds its
own experts' weights and rows and runs the same per-GPU workload ("weak" scaling: the job has
N x 8 experts and N x 32768 rows); no collective is inside the timed region. A "strong" split of
the single 8-expert workload across ranks is timed afterwards and reported under
`strong_scaling`, with the row imbalance of the split.

`--impl reference` times the CPU restatement of the reference's path (the reference has no CPU
compute path of its own) on the host cores, each step a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from grouped_mm_bf16_b200.workloads import (group_sizes, imbalance, make_workload, partition_groups,  # noqa: E402
                                             partition_rows)

METRIC = "useful TFLOP/s, 2Dx3D MoE grouped_mm forward (Mixtral-shape)"
UNIT = "TFLOP/s"

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the tcgen05 kernel comes
# from an ncu capture whose summary under profiles/ records, beside the figure, a hash of the kernel
# sources it was taken from; the figure is reported only while the sources still have that hash.
TRAFFIC_SUMMARIES = {"mixtral": "gmm_sm100_pair_kernel_mixtral.md"}


def kernel_sources_hash() -> str:
    """sha256 over the CUDA sources of the library (names and contents, sorted)."""
    import hashlib

    h = hashlib.sha256()
    csrc = ROOT / "grouped_mm_bf16_b200" / "csrc"
    for f in sorted(list(csrc.glob("*.cu")) + list(csrc.glob("*.cuh"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def ncu_traffic_bytes(workload: str):
    """(bytes per launch or None, note) from the workload's ncu summary, if it matches the sources."""
    import re

    name = TRAFFIC_SUMMARIES.get(workload)
    path = ROOT / "profiles" / name if name else None
    if path is None or not path.exists():
        return None, "no ncu capture of this workload"
    text = path.read_text()
    m_bytes = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)", text)
    m_hash = re.search(r"kernel_sources_sha256_16:\s*([0-9a-f]{16})", text)
    if not (m_bytes and m_hash):
        return None, f"profiles/{name} records no traffic figure"
    if m_hash.group(1) != kernel_sources_hash():
        return None, f"profiles/{name} was captured from other kernel sources ({m_hash.group(1)}); not carried over"
    return float(m_bytes.group(1)), f"ncu capture summarised in profiles/{name}"


def read_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return dict(tflops=float(d["bf16_tflops"]), tflops_sustained=float(d.get("bf16_tflops_sustained", 0) or 0),
                    hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            uuid = torch.cuda.get_device_properties(index).uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def sample(self):
        if self._nv is None:
            return
        try:
            self.samples.append(int(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM)))
            getter = getattr(self._nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                self._nv.nvmlDeviceGetCurrentClocksThrottleReasons
            mask = int(getter(self._h))
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            time.sleep(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return dist, rank, world, local
    torch.cuda.set_device(0)
    return None, 0, 1, 0


def barrier_sync(dist):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(dist, value: float) -> float:
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, value: float) -> float:
    if dist is None:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def rank_stats(dist, value: float):
    """{"min", "median", "max"} of one number per rank (all ranks call; every rank gets the result)."""
    if dist is None:
        return {"min": value, "median": value, "max": value}
    world = dist.get_world_size()
    mine = torch.tensor([value], dtype=torch.float64, device="cuda")
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    vals = sorted(float(t.item()) for t in every)
    return {"min": vals[0], "median": statistics.median(vals), "max": vals[-1]}


def time_steps(dist, step_fn, steps: int, warmup: int, sampler=None) -> float:
    """Runs `warmup` untimed and exactly `steps` timed calls; returns ms for the timed region on
    this rank (CUDA events on the launching stream, barrier + synchronize on both sides)."""
    for _ in range(warmup):
        step_fn()
    barrier_sync(dist)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        start.record()
        for _ in range(steps):
            step_fn()
        stop.record()
        if sampler is not None:
            sampler.sample()
        barrier_sync(dist)
    return start.elapsed_time(stop)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def call_operator(wl):
    from grouped_mm_bf16_b200 import grouped_mm

    return grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs, out_dtype=wl.out_dtype)


# ----------------------------------------------------------------------------- CPU baseline (oracle)


def cpu_oracle_sample(a_cpu, b_cpu, sizes, budget_s: float, workload_rows=None):
    """Per-group fp32 matmul on CPU tensors over a bounded prefix of every group's rows.

    Returns (flops done, seconds, description). Rows are taken group by group in chunks until the
    time budget is used, so the sample keeps the workload's K, N and group structure.
    """
    from oracle.grouped_mm_oracle import grouped_mm_oracle  # the checker, used here as the CPU baseline

    k, n = a_cpu.size(1), b_cpu.size(2)
    # calibrate on one 256-row slab of the first non-empty group
    bounds, s = [], 0
    for sz in sizes:
        bounds.append((s, s + sz))
        s += sz
    g0 = next(g for g, (lo, hi) in enumerate(bounds) if hi > lo)
    rows0 = min(256, bounds[g0][1] - bounds[g0][0])
    t0 = time.perf_counter()
    grouped_mm_oracle(a_cpu[bounds[g0][0]:bounds[g0][0] + rows0], b_cpu[g0:g0 + 1],
                      torch.tensor([rows0], dtype=torch.int32))
    per_row = max((time.perf_counter() - t0) / rows0, 1e-9)
    live = [g for g, (lo, hi) in enumerate(bounds) if hi > lo]
    rows_budget = max(len(live), int(budget_s / per_row))
    take = {g: min(bounds[g][1] - bounds[g][0], max(1, rows_budget // len(live))) for g in live}
    # build the sample as one smaller grouped problem
    a_s = torch.cat([a_cpu[bounds[g][0]:bounds[g][0] + take[g]] for g in live])
    offs_s = torch.tensor([take[g] for g in live], dtype=torch.int64).cumsum(0).to(torch.int32)
    b_s = b_cpu[live]
    t0 = time.perf_counter()
    grouped_mm_oracle(a_s, b_s, offs_s)
    dt = time.perf_counter() - t0
    rows = int(a_s.size(0))
    of = workload_rows if workload_rows is not None else sum(sizes)
    return 2.0 * rows * k * n, dt, f"first {rows} of {of} rows ({rows // len(live)} per group, {len(live)} groups), K={k}, N={n}"


def workload_config(args, wl):
    """`config` of the JSON line: the same for both arms when they run the same workload."""
    groups = len(wl.sizes) if wl.sizes else wl.mat_a.size(0)
    return {
        "workload": f"{args.workload}: form {wl.form}, a {tuple(wl.mat_a.shape)}, b {tuple(wl.mat_b.shape)}, "
                    f"{groups} groups per GPU, seeded sizes",
        "sharding": "expert-parallel, one process per GPU, no collective in the timed region",
        "l2": "inputs larger than L2 (no flush needed)",
        "reduced": None if (args.dims_scale == 1.0 and args.rows_scale == 1.0) else
        f"NOT the benchmark size: dims x{args.dims_scale}, rows x{args.rows_scale} (profiling case)",
    }


def run_reference_arm(args):
    """`--impl reference`: the CPU restatement of the path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    from oracle.grouped_mm_oracle import grouped_mm_oracle  # the checker, timed here as the CPU reference arm

    wl = make_workload(args.workload, "cpu", seed=0, scale=args.rows_scale, dims_scale=args.dims_scale)
    if wl.form != "2d3d":
        print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm times the 2D x 3D form only"}))
        return
    # Calibrate on a small sample, then decide: whole passes over the full workload on the timed
    # steps if the run stays within a few minutes, else a bounded row sample per step.
    f0, t0, _ = cpu_oracle_sample(wl.mat_a, wl.mat_b, wl.sizes, 1.0)
    full_pass_s = wl.flops / max(f0 / t0, 1.0)
    full = full_pass_s * args.steps <= 200.0
    times, flops, desc = [], 0.0, ""
    for i in range(args.warmup + args.steps):
        if i < args.warmup:
            cpu_oracle_sample(wl.mat_a, wl.mat_b, wl.sizes, 1.0)  # warm-up: threads and allocator
            continue
        if full:
            t = time.perf_counter()
            grouped_mm_oracle(wl.mat_a, wl.mat_b, wl.offs)
            times.append(time.perf_counter() - t)
            flops, desc = wl.flops, f"the whole workload every timed step: all {sum(wl.sizes)} rows, {len(wl.sizes)} groups"
        else:
            per_step = max(1.0, min(8.0, 150.0 / max(1, args.steps)))
            f, dt, desc = cpu_oracle_sample(wl.mat_a, wl.mat_b, wl.sizes, per_step)
            times.append(dt)
            flops = f
    ms = 1e3 * sum(times) / len(times)
    value = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16 in, f32 accumulate", "data": "synthetic",
        "config": workload_config(args, wl),
        "reference_detail": f"per-group fp32 torch.matmul on {cores} host threads (CPU restatement of the path); {desc}",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- Triton reference on the GPU


def triton_reference_tflops(wl, steps: int, warmup: int):
    """Times the unmodified reference package (installed under baseline/_ref) on the same inputs."""
    import importlib.util

    pkg = ROOT / "baseline" / "_ref" / "grouped_mm_bf16"
    if not (pkg / "__init__.py").exists():
        return {"unavailable": "baseline/_ref/grouped_mm_bf16 not present"}
    if max(wl.mat_a.numel(), wl.mat_b.numel()) >= 2 ** 31:
        # Its kernels index with 32-bit products (g * stride_bg, kernels.py:340-341); on operands of
        # 2^31 elements or more (the DeepSeek-shape weights) they made an illegal memory access on a
        # B200. Known from that record; never launched at such a size.
        return {"unavailable": "reference faults at this size (32-bit index arithmetic past 2^31 elements); not run"}
    try:
        spec = importlib.util.spec_from_file_location("_reference_grouped_mm_bf16", pkg / "__init__.py",
                                                      submodule_search_locations=[str(pkg)])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["_reference_grouped_mm_bf16"] = mod
        spec.loader.exec_module(mod)
        if wl.form == "2d2d" and wl.out_dtype == torch.float32:
            # its operator rejects an fp32 result for bf16 inputs; its kernel-level function takes one
            from importlib import import_module

            kernels = import_module("_reference_grouped_mm_bf16.kernels")
            out32 = torch.empty((wl.offs.numel(), wl.mat_a.size(0), wl.mat_b.size(1)), dtype=torch.float32,
                                device=wl.mat_a.device)
            fn = lambda: kernels.grouped_mm_2d2d(wl.mat_a, wl.mat_b, wl.offs, out32)  # noqa: E731
        else:
            fn = lambda: mod.grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)  # noqa: E731
        ms = time_steps(None, fn, steps, warmup) / steps
        return {"value": wl.flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps}
    except Exception as exc:  # the baseline is informative; its failure must not hide our number
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


def training_step_tflops(op, wl, steps: int, warmup: int):
    """Forward + both gradients of the workload through autograd (3x the forward FLOPs)."""
    a = wl.mat_a.detach().clone().requires_grad_(True)
    b = wl.mat_b.detach().clone().requires_grad_(True)
    cot = torch.ones_like(op(a, b, offs=wl.offs)).detach()

    def step():
        out = op(a, b, offs=wl.offs)
        torch.autograd.grad(out, [a, b], cot)

    ms = time_steps(None, step, steps, warmup) / steps
    return {"value": 3.0 * wl.flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms, "steps": steps,
            "what": "forward + dA + dB per step, 3x the forward FLOPs"}


def moe_routing_leg(dev, peaks, tokens: int = 16384, topk: int = 2, experts: int = 8, hidden: int = 4096):
    """Times the caller-side steps around the GEMM at the Mixtral shape: expert ids -> offsets and
    permutation, token-row gather, weighted scatter back. HBM-bound byte/index work."""
    from grouped_mm_bf16_b200 import moe

    gen = torch.Generator(device=dev).manual_seed(7)
    ids = torch.randint(0, experts, (tokens, topk), device=dev, dtype=torch.int32, generator=gen)
    x = torch.randn((tokens, hidden), device=dev, generator=gen).bfloat16()
    w = torch.rand((tokens, topk), device=dev, generator=gen)
    offs, perm, inv = moe.route(ids, experts)
    y = moe.permute(x, perm, topk)
    res = {}
    legs = {
        "route": (lambda: moe.route(ids, experts), tokens * topk * 4 * 3),              # ids read twice, perm+inv written
        "permute": (lambda: moe.permute(x, perm, topk), (tokens + tokens * topk) * hidden * 2),
        "combine": (lambda: moe.combine(y, inv, w, topk), (tokens * topk + tokens) * hidden * 2),
    }
    for name, (fn, nbytes) in legs.items():
        ms = time_steps(None, fn, 50, 5) / 50
        res[name] = {"us": ms * 1e3, "GB/s": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    res["shape"] = f"{tokens} tokens, top-{topk}, {experts} experts, hidden {hidden}, bf16"
    return res


def gated_up_leg(dev, experts: int = 8, hidden: int = 4096, inter: int = 14336):
    """Times the Mixtral-shape gated up-projection (weights [8, 4096, 2 x 14336]) with the activation
    fused into the GEMM's epilogue, against grouped_mm followed by torch's silu and mul."""
    from grouped_mm_bf16_b200 import grouped_mm, moe
    from grouped_mm_bf16_b200.workloads import group_sizes

    gen = torch.Generator(device=dev).manual_seed(11)
    sizes = group_sizes("mixtral", 0)
    x = torch.randn((sum(sizes), hidden), device=dev, generator=gen).bfloat16()
    w = (torch.randn((experts, hidden, 2 * inter), device=dev, generator=gen) * 0.02).bfloat16()
    offs = torch.tensor(sizes, dtype=torch.int64).cumsum(0).to(torch.int32).to(dev)
    flops = 2.0 * sum(sizes) * hidden * 2 * inter

    def two_step():
        both = grouped_mm(x, w, offs=offs)
        return torch.nn.functional.silu(both[:, :inter]) * both[:, inter:]

    with torch.no_grad():
        fused_ms = time_steps(None, lambda: moe.gated_up_projection(x, w, offs), 20, 3) / 20
        two_ms = time_steps(None, two_step, 20, 3) / 20
    # the whole routed block at the same shape: 16384 tokens, top-2
    tokens, topk = sum(sizes) // 2, 2
    ids = torch.randint(0, experts, (tokens, topk), device=dev, dtype=torch.int32, generator=gen)
    xt = torch.randn((tokens, hidden), device=dev, generator=gen).bfloat16()
    gates = torch.rand((tokens, topk), device=dev, generator=gen)
    down = (torch.randn((experts, inter, hidden), device=dev, generator=gen) * 0.02).bfloat16()
    with torch.no_grad():
        layer_ms = time_steps(None, lambda: moe.feed_forward(xt, ids, gates, w, down), 20, 3) / 20
    layer_flops = 2.0 * tokens * topk * hidden * 3 * inter
    return {"fused_ms": fused_ms, "fused_TFLOP/s": flops / (fused_ms * 1e-3) / 1e12, "two_step_ms": two_ms,
            "feed_forward_block": {"ms": layer_ms, "tokens_per_s": tokens / (layer_ms * 1e-3),
                                   "TFLOP/s": layer_flops / (layer_ms * 1e-3) / 1e12,
                                   "what": f"moe.feed_forward: route, permute, gated up, down, combine; {tokens} tokens, top-{topk}"},
            "shape": f"{sum(sizes)} rows, {experts} experts, {hidden} -> 2 x {inter}, bf16",
            "what": "silu(x @ gate) * (x @ up): one kernel vs grouped_mm + torch silu * mul"}


def expert_parallel_leg(dist, dev, rank: int, world: int, tokens: int = 16384, topk: int = 2, experts: int = 8,
                        hidden: int = 4096, inter: int = 14336):
    """Times the expert-parallel feed-forward block: every rank holds `tokens` tokens and experts / world
    experts of the Mixtral shape; rows travel to their expert's rank and back by NCCL all-to-all."""
    from grouped_mm_bf16_b200 import expert_parallel

    if experts % world:
        return {"unavailable": f"{experts} experts do not divide over {world} ranks"}
    e_local = experts // world
    gen = torch.Generator(device=dev).manual_seed(31 + rank)
    x = torch.randn((tokens, hidden), device=dev, generator=gen).bfloat16()
    ids = torch.randint(0, experts, (tokens, topk), device=dev, dtype=torch.int32, generator=gen)
    gates = torch.rand((tokens, topk), device=dev, generator=gen)
    gate_up = (torch.randn((e_local, hidden, 2 * inter), device=dev, generator=gen) * 0.02).bfloat16()
    down = (torch.randn((e_local, inter, hidden), device=dev, generator=gen) * 0.02).bfloat16()

    def step():
        with torch.no_grad():
            expert_parallel.feed_forward(x, ids, gates, gate_up, down)

    steps = 10
    ms = max_over_ranks(dist, time_steps(dist, step, steps, 3)) / steps
    flops = 2.0 * tokens * world * topk * hidden * 3 * inter
    res = {"ms": ms, "tokens_per_s": tokens * world / (ms * 1e-3), "TFLOP/s": flops / (ms * 1e-3) / 1e12,
           "what": f"expert_parallel.feed_forward: {tokens} tokens per rank, top-{topk} of {experts} experts "
                   f"({e_local} per rank), {hidden} <-> {inter}; dispatch and combine by NCCL all-to-all"}
    try:
        buffers = expert_parallel.PeerBuffers(world * tokens * topk, hidden, torch.bfloat16, dev)

        def peer_step():
            with torch.no_grad():
                expert_parallel.feed_forward_peer(x, ids, gates, gate_up, down, buffers)

        p_ms = max_over_ranks(dist, time_steps(dist, peer_step, steps, 3)) / steps
        from grouped_mm_bf16_b200 import _op

        res["peer_memory"] = {"ms": p_ms, "tokens_per_s": tokens * world / (p_ms * 1e-3),
                              "TFLOP/s": flops / (p_ms * 1e-3) / 1e12, "device_status": _op.check_status(dev),
                              "what": "feed_forward_peer: rows stored into / loaded from the peers' buffers by this "
                                      "package's kernels, no host synchronisation"}
    except Exception as exc:
        res["peer_memory"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    return res


# ----------------------------------------------------------------------------- legs beside the headline


def roofline_of(wl, ms: float, peaks, sustained: bool = False):
    """Roofline position of one launch: bound = the slower of FLOPs / tensor peak and bytes / HBM peak."""
    tflops_peak = peaks["tflops_sustained"] if (sustained and peaks["tflops_sustained"]) else peaks["tflops"]
    t_flops = wl.flops / (tflops_peak * 1e12) * 1e3
    t_bytes = wl.algorithmic_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
    return {"bound": "tensor" if t_flops >= t_bytes else "hbm", "floor_ms": max(t_flops, t_bytes),
            "frac": max(t_flops, t_bytes) / ms, "TFLOP/s": wl.flops / (ms * 1e-3) / 1e12,
            "GB/s": wl.algorithmic_bytes / (ms * 1e-3) / 1e9}


def sampled_within_tolerance(wl, out, max_rows: int = 96):
    """Slab-sampled check of a result against the CPU oracle: rows spread over every group (one per
    32-row slab, thinned to at most `max_rows`), all columns. Returns the worst error as a fraction
    of the tolerance |out - ref| <= 8e-3 |ref| + 1e-2 sqrt(K) sigma_a sigma_b (<= 1 passes)."""
    from oracle.grouped_mm_oracle import atol_for, group_bounds, max_violation  # the checker

    def pick(rows):
        return rows[:: max(1, -(-len(rows) // max_rows))]

    worst = 0.0
    if wl.form == "2d3d":
        bounds = group_bounds(wl.offs.cpu(), wl.mat_a.size(0))
        rows = pick([(g, r) for g, (s, e) in enumerate(bounds) for r in range(s + 5 % max(1, e - s), e, 32)])
        atol = atol_for(wl.k, wl.sigma_a, wl.sigma_b)
        for g in sorted({g for g, _ in rows}):
            idx = torch.tensor([r for gg, r in rows if gg == g], device=out.device)
            ref = wl.mat_a[idx].cpu().float() @ wl.mat_b[g].cpu().float()
            worst = max(worst, max_violation(out[idx], ref, torch.ones_like(ref, dtype=torch.bool), atol))
    elif wl.form == "3d3d":
        atol = atol_for(wl.k, wl.sigma_a, wl.sigma_b)
        per = max(1, max_rows // wl.mat_a.size(0))
        for g in range(wl.mat_a.size(0)):
            idx = torch.tensor(pick(list(range(5, wl.mat_a.size(1), 32)))[:per], device=out.device)
            ref = wl.mat_a[g][idx].cpu().float() @ wl.mat_b[g].cpu().float()
            worst = max(worst, max_violation(out[g][idx], ref, torch.ones_like(ref, dtype=torch.bool), atol))
    else:  # 2d2d: every group, a few rows each; empty groups must be exactly zero
        bounds = group_bounds(wl.offs.cpu(), wl.mat_a.size(1))
        idx = torch.tensor(pick(list(range(5, wl.mat_a.size(0), 32)))[:8], device=out.device)
        a_rows, b_cpu = wl.mat_a[idx].cpu().float(), wl.mat_b.cpu().float()
        for g, (s, e) in enumerate(bounds):
            if e == s:
                worst = max(worst, 0.0 if float(out[g].abs().max()) == 0.0 else float("inf"))
                continue
            ref = a_rows[:, s:e] @ b_cpu[s:e]
            worst = max(worst, max_violation(out[g][idx], ref, torch.ones_like(ref, dtype=torch.bool),
                                             atol_for(e - s, wl.sigma_a, wl.sigma_b)))
    return float(worst)


KERNEL_NAMES = {0: "none", 1: "gmm_sm100_kernel (one CTA per 128x256 tile)", 2: "gmm_generic_kernel",
                3: "gmm_sm100_pair_kernel (cta_group::2, CTA pair per 256x256 tile)"}


def all_configs_leg(dev, peaks, steps: int = 20, with_triton: bool = True):
    """The other benchmark configurations, each timed for `steps` launches (CUDA events) and checked
    on a slab sample against the CPU oracle; the reference's Triton kernel beside each where it runs."""
    from grouped_mm_bf16_b200 import _lib, _op

    forms = {"2d3d": _lib.FORM_2D3D, "3d3d": _lib.FORM_3D3D, "2d2d": _lib.FORM_2D2D, "3d2d": _lib.FORM_3D2D}
    res = {}
    for name in ("readme", "batched", "deepseek_up", "deepseek_down", "wgrad"):
        try:
            wl = make_workload(name, dev, seed=0)
            out = call_operator(wl)
            entry = {"kernel": KERNEL_NAMES.get(_op.selected_kernel(forms[wl.form], wl.mat_a, wl.mat_b, out), "?")}
            entry["within_tolerance"] = sampled_within_tolerance(wl, out)
            del out
            sampler = ClockSampler(dev.index or 0)
            ms = time_steps(None, lambda: call_operator(wl), steps, 3, sampler) / steps
            entry.update({"ms": ms, "steps": steps, "flops": wl.flops, "algorithmic_bytes": wl.algorithmic_bytes,
                          "sm_mhz": sampler.summary()["sm_mhz"], "reasons": sampler.summary()["reasons"]})
            entry.update(roofline_of(wl, ms, peaks))
            if name == "readme":
                entry["note"] = "196608 FLOP: launch latency only, no roofline meaning"
            if with_triton:
                entry["triton_reference"] = triton_reference_tflops(wl, 5, 2)
            entry["device_status"] = _op.check_status(dev)
            res[name] = entry
            del wl
            torch.cuda.empty_cache()
        except Exception as exc:  # informative legs must not hide the headline number
            res[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    return res


def sustained_leg(step_fn, flops: float, ms_hint: float, peaks, device_index: int, min_seconds: float = 2.0):
    """The same launch repeated back to back for at least `min_seconds`: the power-capped steady
    state, against the sustained cuBLAS peak. ms x MHz separates clock effects from kernel effects."""
    steps = max(20, int(min_seconds * 1e3 / max(ms_hint, 1e-3)) + 1)
    sampler = ClockSampler(device_index, period_s=0.02)
    ms = time_steps(None, step_fn, steps, 3, sampler) / steps
    clocks = sampler.summary()
    tf = flops / (ms * 1e-3) / 1e12
    return {"value": tf, "unit": UNIT, "ms_per_step": ms, "steps": steps, "seconds": ms * steps * 1e-3,
            "sm_mhz_median": clocks["sm_mhz"], "reasons": clocks["reasons"],
            "ms_x_mhz": (ms * clocks["sm_mhz"]) if clocks["sm_mhz"] else None,
            "frac_of_sustained_peak": (tf / peaks["tflops_sustained"]) if peaks["tflops_sustained"] else None,
            "sustained_peak": peaks["tflops_sustained"]}


def cublas_yardstick(dev, peaks, m: int = 32768, k: int = 4096, n: int = 14336):
    """torch.matmul (cuBLAS) on the dense GEMM of the headline's size, in this process: a yardstick
    for what the box gives a library kernel at the same moment, as a burst and sustained."""
    gen = torch.Generator(device=dev).manual_seed(5)
    a = torch.randn((m, k), device=dev, generator=gen).bfloat16()
    b = (torch.randn((k, n), device=dev, generator=gen) * 0.02).bfloat16()
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    flops = 2.0 * m * k * n
    fn = lambda: torch.matmul(a, b, out=out)  # noqa: E731
    sampler = ClockSampler(dev.index or 0)
    burst_ms = time_steps(None, fn, 20, 5, sampler) / 20
    res = {"what": f"torch.matmul bf16 [{m},{k}] @ [{k},{n}] (one dense GEMM with the headline's FLOPs)",
           "burst": {"value": flops / (burst_ms * 1e-3) / 1e12, "unit": UNIT, "ms": burst_ms, "steps": 20,
                     "sm_mhz_median": sampler.summary()["sm_mhz"]},
           "sustained": sustained_leg(fn, flops, burst_ms, peaks, dev.index or 0)}
    return res


def copy_rates_leg(dist, dev, nbytes: int = 512 << 20):
    """Per-direction pinned-host copy rate of every rank, all ranks copying at the same time."""
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    devbuf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    res = {}
    for name, fn in (("h2d", lambda: devbuf.copy_(host, non_blocking=True)),
                     ("d2h", lambda: host.copy_(devbuf, non_blocking=True))):
        ms = time_steps(dist, fn, 4, 1) / 4
        res[name + "_GBps_per_rank"] = rank_stats(dist, nbytes / (ms * 1e-3) / 1e9)
    res["what"] = f"{nbytes >> 20} MiB pinned copies, every rank at once, each direction alone"
    return res


# ----------------------------------------------------------------------------- main arm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral",
                    choices=["mixtral", "deepseek_up", "deepseek_down", "batched", "wgrad"])
    ap.add_argument("--dims-scale", type=float, default=1.0,
                    help="shrink the fixed dimensions (K, N, M) of the workload; for small profiling cases only")
    ap.add_argument("--rows-scale", type=float, default=1.0,
                    help="shrink the ragged extent (routed rows) of the workload; for small profiling cases only")
    ap.add_argument("--no-baselines", action="store_true", help="skip the CPU and Triton baseline legs")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ep-block", action="store_true",
                    help="N > 1 only: also time the expert-parallel routed feed-forward block (NCCL all-to-all "
                         "dispatch and combine around the grouped GEMMs); adds the key expert_parallel_block")
    ap.add_argument("--tf32", action="store_true",
                    help="fp32 operands multiplied as TF32 (torch.backends.cuda.matmul.allow_tf32 = True) instead of "
                         "the benchmark's bf16; a side measurement, reported against half the bf16 tensor peak")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    dist, rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    peaks = read_peaks()

    # Every rank owns its own experts (weak scaling): same shape, its own seeded draw.
    if args.tf32:
        torch.backends.cuda.matmul.allow_tf32 = True
        args.no_baselines = True  # the CPU and Triton legs are for the bf16 benchmark
        peaks = dict(peaks, tflops=peaks["tflops"] / 2,
                     tflops_sustained=peaks["tflops_sustained"] / 2 if peaks["tflops_sustained"] else None,
                     source=peaks["source"] + "; TF32 peak taken as half the bf16 figure")
    wl = make_workload(args.workload, dev, seed=rank, scale=args.rows_scale, dims_scale=args.dims_scale,
                       dtype=torch.float32 if args.tf32 else torch.bfloat16)
    from grouped_mm_bf16_b200 import _lib, _op

    out = call_operator(wl)
    form = {"2d3d": _lib.FORM_2D3D, "3d3d": _lib.FORM_3D3D, "2d2d": _lib.FORM_2D2D, "3d2d": _lib.FORM_3D2D}[wl.form]
    kernel = _op.selected_kernel(form, wl.mat_a, wl.mat_b, out)
    del out

    sampler = ClockSampler(local)
    ms_total = time_steps(dist, lambda: call_operator(wl), args.steps, args.warmup, sampler)
    status = _op.check_status(dev)
    per_rank_ms = rank_stats(dist, ms_total / args.steps) if world > 1 else None
    ms_total = max_over_ranks(dist, ms_total)
    ms_step = ms_total / args.steps
    total_flops = sum_over_ranks(dist, wl.flops)
    value = total_flops / (ms_step * 1e-3) / 1e12

    # roofline of the one kernel a step launches (this rank's launch)
    my_ms = ms_step
    achieved = wl.flops / (my_ms * 1e-3) / 1e12
    hbm_floor_ms = wl.algorithmic_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
    tensor_floor_ms = wl.flops / (peaks["tflops"] * 1e12) * 1e3
    if tensor_floor_ms >= hbm_floor_ms:
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["tflops"]}
    else:
        gbs = wl.algorithmic_bytes / (my_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"]}
    traffic, traffic_note = (None, "not captured for TF32") if args.tf32 else ncu_traffic_bytes(args.workload)
    if args.dims_scale != 1.0 or args.rows_scale != 1.0:
        traffic, traffic_note = None, "reduced size"
    roofline.update({
        "traffic": traffic, "traffic_source": traffic_note,
        "peak_source": f"{peaks['source']} (burst cuBLAS bf16 / copy bandwidth): the timed region of the default "
                       "20 steps is a burst; see `sustained` for the power-capped figure against the sustained peak",
        "frac_of_nominal_2250": None if args.tf32 else achieved / 2250.0,
        "algorithmic_flops_per_launch": wl.flops, "algorithmic_bytes_per_launch": wl.algorithmic_bytes,
        "kernel": {1: "gmm_sm100_kernel (TMA + tcgen05.mma, one CTA per 128x256 tile)", 2: "gmm_generic_kernel",
                   3: "gmm_sm100_pair_kernel (TMA + tcgen05.mma.cta_group::2, CTA pair per 256x256 tile)"}.get(kernel, "none"),
    })

    # end to end with host buffers
    e2e = None
    if not args.no_e2e:
        a_h, b_h = wl.mat_a.cpu().pin_memory(), wl.mat_b.cpu().pin_memory()
        offs_h = wl.offs.cpu().pin_memory() if wl.offs is not None else None
        from grouped_mm_bf16_b200 import grouped_mm

        probe = call_operator(wl)
        out_h = torch.empty(probe.shape, dtype=probe.dtype).pin_memory()
        del probe

        if wl.form == "2d3d" and wl.mat_b.is_contiguous():
            # The host-buffer entry: per-chunk H2D copies, GEMMs and D2H copies overlapped on three streams.
            from grouped_mm_bf16_b200.host import grouped_mm_host

            def e2e_step():
                grouped_mm_host(a_h, b_h, offs_h, out=out_h, device=dev)
        else:
            def e2e_step():
                a_d = a_h.to(dev, non_blocking=True)
                b_d = b_h.to(dev, non_blocking=True)
                o_d = offs_h.to(dev, non_blocking=True) if offs_h is not None else None
                res = grouped_mm(a_d, b_d, offs=o_d, out_dtype=wl.out_dtype)
                out_h.copy_(res, non_blocking=True)

        e_steps = max(3, min(args.steps, 20))
        e_ms_mine = time_steps(dist, e2e_step, e_steps, 3) / e_steps
        e_ms = max_over_ranks(dist, e_ms_mine)
        h2d = a_h.numel() * a_h.element_size() + b_h.numel() * b_h.element_size() + \
            (offs_h.numel() * 4 if offs_h is not None else 0)
        d2h = out_h.numel() * out_h.element_size()
        rates = copy_rates_leg(dist, dev) if world > 1 else None
        e2e = {"value": total_flops / (e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": e_ms, "steps": e_steps,
               "api": "grouped_mm_bf16_b200.host.grouped_mm_host (pinned host in/out, copies overlapped with compute)"
               if wl.form == "2d3d" and wl.mat_b.is_contiguous() else "pinned host -> device copies, grouped_mm, copy back"}
        if rates is not None:
            e2e["host_copy_rates"] = rates
            e2e["per_rank_ms"] = rank_stats(dist, e_ms_mine)
        del a_h, b_h, out_h

    # strong split of ONE workload across the ranks (reported beside the weak number): by rows, cutting
    # a hot expert across consecutive ranks (each holds a copy of its weights), and by whole experts.
    strong = None
    if world > 1:
        sizes = group_sizes(args.workload, 0)
        if sizes is not None and wl.form == "2d3d":
            def strong_leg(local_sizes):
                if sum(local_sizes) > 0:
                    swl = make_workload(args.workload, dev, seed=0, sizes=local_sizes,
                                        dtype=torch.float32 if args.tf32 else torch.bfloat16)
                    s_ms = time_steps(dist, lambda: call_operator(swl), args.steps, args.warmup) / args.steps
                    s_flops = swl.flops
                else:
                    s_ms = time_steps(dist, lambda: None, args.steps, args.warmup) / args.steps
                    s_flops = 0.0
                return s_ms, s_flops

            pieces = partition_rows(sizes, world)
            s_ms, s_flops = strong_leg([rows for _, _, rows in pieces[rank]])
            s_total = sum_over_ranks(dist, s_flops)
            s_max = max_over_ranks(dist, s_ms)
            loads = [sum(r for _, _, r in ps) for ps in pieces]
            strong = {"value": s_total / (s_max * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": s_max,
                      "per_rank_ms": rank_stats(dist, s_ms),
                      "row_balance_mean_over_max": (sum(loads) / len(loads)) / max(loads),
                      "experts_cut": sum(1 for g in range(len(sizes)) if sum(1 for ps in pieces for p in ps if p[0] == g) > 1),
                      "note": "one 8-expert workload split by rows: rank r owns rows [r T / N, (r+1) T / N); an expert "
                              "whose rows span several ranks has its weights on each of them, placed before timing"}
            lo, hi = partition_groups(sizes, world)[rank]
            w_ms, w_flops = strong_leg(sizes[lo:hi])
            w_total = sum_over_ranks(dist, w_flops)
            w_max = max_over_ranks(dist, w_ms)
            strong["whole_experts"] = {"value": w_total / (w_max * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": w_max,
                                       "per_rank_ms": rank_stats(dist, w_ms),
                                       "row_balance_mean_over_max": imbalance(sizes, world),
                                       "note": "the same workload split by contiguous whole-expert ranges, row-balanced"}

    ep_block = None
    if world > 1 and args.ep_block:
        ep_block = expert_parallel_leg(dist, dev, rank, world)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": "fp32 in/out multiplied as TF32, f32 accumulate (NOT the benchmark dtype)" if args.tf32
            else "bf16 in/out, f32 accumulate", "data": "synthetic",
            "config": workload_config(args, wl),
            "roofline": roofline, "e2e": e2e, "gpu_launches": args.steps, "clocks": sampler.summary(),
            "device_status": status,
        }
        if per_rank_ms is not None:
            line["per_rank_ms"] = per_rank_ms
        if ep_block is not None:
            line["expert_parallel_block"] = ep_block
        if strong is not None:
            line["strong_scaling"] = strong
        if world == 1 and not args.no_baselines:
            torch.set_num_threads(os.cpu_count() or 1)
            f, dt, desc = cpu_oracle_sample(wl.mat_a.cpu(), wl.mat_b.cpu(), wl.sizes, 15.0) if wl.form == "2d3d" \
                else (0.0, 1.0, "n/a")
            line["cpu_baseline"] = {"value": f / dt / 1e12, "unit": UNIT, "cores": os.cpu_count() or 1,
                                    "kind": "port", "sample": desc}
            line["triton_reference"] = triton_reference_tflops(wl, max(3, min(args.steps, 20)), 3)
            try:
                line["sustained"] = sustained_leg(lambda: call_operator(wl), wl.flops, ms_step, peaks, local)
                line["cublas_yardstick"] = cublas_yardstick(dev, peaks)
            except Exception as exc:  # informative legs must not hide the headline number
                line["sustained_error"] = f"{type(exc).__name__}: {exc}"[:200]
            if args.workload == "mixtral" and args.dims_scale == 1.0 and args.rows_scale == 1.0 and not args.tf32:
                line["all_configs"] = all_configs_leg(dev, peaks)
            if wl.form == "2d3d":
                from grouped_mm_bf16_b200 import grouped_mm

                try:
                    # No Triton leg here: the reference's backward kernels did not finish one Mixtral-shape
                    # step within four minutes on a B200, so they are not run inside the benchmark.
                    line["training_step"] = training_step_tflops(grouped_mm, wl, max(3, min(args.steps, 20)), 3)
                except Exception as exc:  # informative legs must not hide the headline number
                    line["training_step_error"] = f"{type(exc).__name__}: {exc}"[:200]
                try:
                    line["moe_routing"] = moe_routing_leg(dev, peaks)
                except Exception as exc:
                    line["moe_routing_error"] = f"{type(exc).__name__}: {exc}"[:200]
                try:
                    line["gated_up_projection"] = gated_up_leg(dev)
                except Exception as exc:
                    line["gated_up_projection_error"] = f"{type(exc).__name__}: {exc}"[:200]
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
