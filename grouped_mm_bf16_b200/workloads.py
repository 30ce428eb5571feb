"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs,
and the expert-parallel (group-sharded) partitioning used on more than one GPU.

The five configurations stand in for MoE layers of the named shapes (README example, a uniform
batched GEMM, a Mixtral-8x7B up-projection, a DeepSeek-V3 up/down-projection with Zipf-skewed
routing, and the weight-gradient form). No dataset or checkpoint is involved: group sizes are
drawn from a seeded CPU generator (so every rank and the CPU checker agree on them), values from a
seeded generator on the target device.

The reference's own benchmark builds its inputs the same way — ``bincount`` of routed expert ids,
then ``cumsum`` to int32 end offsets (bench/bench_2d3d.py:124-138).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


@dataclass
class Workload:
    name: str
    form: str  # "2d3d", "3d3d", "2d2d", "3d2d"
    mat_a: torch.Tensor
    mat_b: torch.Tensor
    offs: Optional[torch.Tensor]
    out_dtype: Optional[torch.dtype]
    sizes: Optional[List[int]]  # group sizes along the ragged dimension
    sigma_a: float
    sigma_b: float
    k: int  # contraction length (per group: see sizes, for the 2d2d form)
    meta: Dict[str, object] = field(default_factory=dict)

    @property
    def flops(self) -> float:
        """Useful floating-point operations: padding, masked rows and empty groups count zero."""
        a, b = self.mat_a, self.mat_b
        if self.form == "3d3d":
            return 2.0 * a.size(0) * a.size(1) * a.size(2) * b.size(2)
        if self.form == "2d3d":
            return 2.0 * sum(self.sizes) * a.size(1) * b.size(2)
        if self.form == "3d2d":
            return 2.0 * sum(self.sizes) * a.size(1) * a.size(2)
        return 2.0 * a.size(0) * b.size(1) * sum(self.sizes)

    @property
    def algorithmic_bytes(self) -> float:
        """Each operand read once, the output written once; weights of empty groups not counted."""
        a, b = self.mat_a, self.mat_b
        esz = a.element_size()
        osz = torch.empty((), dtype=self.out_dtype or a.dtype).element_size()
        if self.form == "3d3d":
            g, m, k, n = a.size(0), a.size(1), a.size(2), b.size(2)
            return esz * g * (m * k + k * n) + osz * g * m * n
        if self.form == "2d3d":
            rows, k, n = sum(self.sizes), a.size(1), b.size(2)
            live = sum(1 for s in self.sizes if s > 0)
            return esz * (rows * k + live * k * n) + osz * rows * n
        if self.form == "3d2d":
            cols, m, k = sum(self.sizes), a.size(1), a.size(2)
            live = sum(1 for s in self.sizes if s > 0)
            return esz * (live * m * k + k * cols) + osz * m * cols
        m, n, kt = a.size(0), b.size(1), sum(self.sizes)
        return esz * (m * kt + kt * n) + osz * len(self.sizes) * m * n


CONFIG_NAMES = ("readme", "batched", "mixtral", "deepseek_up", "deepseek_down", "wgrad")


def _multinomial_counts(p: torch.Tensor, draws: int, gen: torch.Generator) -> List[int]:
    idx = torch.multinomial(p, draws, replacement=True, generator=gen)
    return torch.bincount(idx, minlength=p.numel()).tolist()


def group_sizes(name: str, seed: int = 0, scale: float = 1.0) -> Optional[List[int]]:
    """Group sizes of a configuration, drawn on the CPU from ``seed``. ``scale`` shrinks the
    number of routed rows (not the number of groups) for small test cases."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    if name == "readme":
        return [0, 7, 1, 13, 0, 11]
    if name == "batched":
        return None
    if name == "mixtral":
        p = _dirichlet(torch.ones(8), gen)
        return _multinomial_counts(p, max(8, int(32768 * scale)), gen)
    if name in ("deepseek_up", "deepseek_down"):
        p = torch.arange(1, 257, dtype=torch.float64).pow(-1.1)
        p = (p / p.sum()).float()
        return _multinomial_counts(p, max(256, int(65536 * scale)), gen)
    if name == "wgrad":
        p = _dirichlet(torch.full((64,), 0.5), gen)
        return [8 * c for c in _multinomial_counts(p, max(64, int(8192 * scale)), gen)]
    raise ValueError(f"unknown config {name!r}; expected one of {CONFIG_NAMES}")


def _dirichlet(alpha: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
    """Dirichlet(alpha) from normalised Gamma(alpha, 1) draws, using the given generator."""
    g = torch._standard_gamma(alpha.double(), generator=gen).clamp_min(1e-30)
    return (g / g.sum()).float()


def _randn(shape, sigma: float, dtype, device, gen: torch.Generator) -> torch.Tensor:
    """N(0, sigma^2) values; drawn in fp32 in slabs so that no huge fp32 temporary is needed."""
    out = torch.empty(shape, dtype=dtype, device=device)
    flat = out.view(-1)
    step = 1 << 26
    for s in range(0, flat.numel(), step):
        e = min(s + step, flat.numel())
        flat[s:e] = (torch.randn(e - s, generator=gen, device=device, dtype=torch.float32) * sigma).to(dtype)
    return out


def make_workload(name: str, device="cpu", seed: int = 0, scale: float = 1.0, dims_scale: float = 1.0,
                  sizes: Optional[List[int]] = None, dtype: torch.dtype = torch.bfloat16) -> Workload:
    """Builds one configuration on ``device``.

    ``scale`` shrinks the ragged extent, ``dims_scale`` the fixed dimensions (both for small
    cases); ``sizes`` overrides the drawn group sizes (used for per-rank shards).
    """
    device = torch.device(device)
    vgen = torch.Generator(device=device).manual_seed(seed + 1000003)
    if sizes is None:
        sizes = group_sizes(name, seed, scale)

    def dim(x: int, mult: int = 64) -> int:
        return max(mult, int(round(x * dims_scale / mult)) * mult)

    def offs_of(sz: List[int]) -> torch.Tensor:
        return torch.tensor(sz, dtype=torch.int64).cumsum(0).to(torch.int32).to(device)

    if name == "readme":
        a = _randn((sum(sizes), 64), 1.0, dtype, device, vgen)
        b = _randn((len(sizes), 64, 48), 1.0, dtype, device, vgen)
        return Workload(name, "2d3d", a, b, offs_of(sizes), None, sizes, 1.0, 1.0, 64)
    if name == "batched":
        g = 16 if sizes is None else len(sizes)
        m, k, n = dim(1024), dim(4096), dim(4096)
        a = _randn((g, m, k), 1.0, dtype, device, vgen)
        b = _randn((g, k, n), 0.02, dtype, device, vgen)
        return Workload(name, "3d3d", a, b, None, None, None, 1.0, 0.02, k)
    if name == "mixtral":
        k, n = dim(4096), dim(14336)
        a = _randn((sum(sizes), k), 1.0, dtype, device, vgen)
        b = _randn((len(sizes), k, n), 0.02, dtype, device, vgen)
        return Workload(name, "2d3d", a, b, offs_of(sizes), None, sizes, 1.0, 0.02, k)
    if name in ("deepseek_up", "deepseek_down"):
        k, n = (dim(7168), dim(2048)) if name == "deepseek_up" else (dim(2048), dim(7168))
        a = _randn((sum(sizes), k), 1.0, dtype, device, vgen)
        b = _randn((len(sizes), n, k), 0.02, dtype, device, vgen).transpose(-2, -1)  # column-major [G,K,N]
        return Workload(name, "2d3d", a, b, offs_of(sizes), None, sizes, 1.0, 0.02, k)
    if name == "wgrad":
        m, n = dim(4096), dim(1536)
        kt = sum(sizes)
        a = _randn((kt, m), 1.0, dtype, device, vgen).t()  # column-major [M, K_total]
        b = _randn((kt, n), 1.0, dtype, device, vgen)
        return Workload(name, "2d2d", a, b, offs_of(sizes), torch.float32, sizes, 1.0, 1.0, kt)
    raise ValueError(f"unknown config {name!r}; expected one of {CONFIG_NAMES}")


# ----------------------------------------------------------------------------- group sharding


def partition_groups(sizes: List[int], world: int) -> List[Tuple[int, int]]:
    """Splits groups into ``world`` contiguous ranges [lo, hi) minimising the largest row count.

    Contiguous, so that each rank's rows of ``mat_a`` and of the output are one slice. Solved
    exactly by bisection on the bottleneck value with a greedy feasibility check.
    """
    n = len(sizes)
    if world <= 0:
        raise ValueError("world must be positive")
    if world >= n:
        return [(i, i + 1) if i < n else (n, n) for i in range(world)]

    def cuts_for(cap: int) -> Optional[List[int]]:
        cuts, acc, used = [], 0, 1
        for i, s in enumerate(sizes):
            if s > cap:
                return None
            if acc + s > cap:
                cuts.append(i)
                acc, used = 0, used + 1
                if used > world:
                    return None
            acc += s
        return cuts

    lo, hi = max(sizes + [0]), sum(sizes)
    while lo < hi:
        mid = (lo + hi) // 2
        if cuts_for(mid) is None:
            lo = mid + 1
        else:
            hi = mid
    cuts = cuts_for(lo) or []
    # Spend unused cuts on the largest remaining ranges so every rank owns at least one group.
    bounds = [0] + cuts + [n]
    while len(bounds) - 1 < world:
        widths = [(bounds[i + 1] - bounds[i], i) for i in range(len(bounds) - 1)]
        w, i = max(widths)
        if w < 2:
            break
        bounds.insert(i + 1, bounds[i] + w // 2)
    ranges = [(bounds[i], bounds[i + 1]) for i in range(len(bounds) - 1)]
    ranges += [(n, n)] * (world - len(ranges))
    return ranges


def partition_rows(sizes: List[int], world: int) -> List[List[Tuple[int, int, int]]]:
    """Row-balanced split that may cut a group: rank r gets rows [r * T / world, (r + 1) * T / world) of the
    T routed rows, as a list of pieces ``(group, first_row_in_group, rows)``.

    Every rank's rows are still one contiguous slice of ``mat_a`` and of the output. A group cut across
    consecutive ranks has its weights replicated on each of them (placed before any timing), so the
    ranks stay independent: no collective, no peer access. Loads differ by at most one row.
    """
    if world <= 0:
        raise ValueError("world must be positive")
    total = sum(sizes)
    starts, acc = [], 0
    for sz in sizes:
        starts.append(acc)
        acc += sz
    out: List[List[Tuple[int, int, int]]] = []
    g = 0
    for r in range(world):
        lo, hi = (r * total) // world, ((r + 1) * total) // world
        pieces = []
        while g < len(sizes) and starts[g] + sizes[g] <= lo:
            g += 1
        h = g
        while h < len(sizes) and starts[h] < hi:
            first = max(lo, starts[h])
            last = min(hi, starts[h] + sizes[h])
            if last > first:
                pieces.append((h, first - starts[h], last - first))
            h += 1
        out.append(pieces)
    return out


def shard_sizes(sizes: List[int], world: int, rank: int) -> List[int]:
    lo, hi = partition_groups(sizes, world)[rank]
    return list(sizes[lo:hi])


def imbalance(sizes: List[int], world: int) -> float:
    """mean / max of the per-rank row counts of the partition (1.0 = perfectly balanced)."""
    loads = [sum(sizes[lo:hi]) for lo, hi in partition_groups(sizes, world)]
    return (sum(loads) / len(loads)) / max(loads) if max(loads) > 0 else 1.0


def rebase_offsets(offs: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Local int32 end offsets of groups [lo, hi): the global ones minus the rows before ``lo``."""
    base = offs[lo - 1] if lo > 0 else torch.zeros((), dtype=offs.dtype, device=offs.device)
    return (offs[lo:hi] - base).to(torch.int32)
