"""Workload generators and the expert-parallel partitioning, including a two-rank run over gloo.

The multi-GPU path has no data-path collective: each rank runs the operator on its own groups.
What needs checking without GPUs is the host logic — the contiguous row-balanced split, the
rebased offsets, and that the per-rank results, gathered, equal the unsharded result. The
ranks here compute with the CPU oracle; the gather uses gloo.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grouped_mm_bf16_b200.workloads import (CONFIG_NAMES, group_sizes, imbalance, make_workload, partition_groups,
                                            rebase_offsets, shard_sizes)
from oracle.grouped_mm_oracle import grouped_mm_oracle


def test_group_sizes_are_seeded_and_sum_to_the_routed_rows():
    assert group_sizes("readme") == [0, 7, 1, 13, 0, 11]
    assert group_sizes("batched") is None
    mix = group_sizes("mixtral", 0)
    assert len(mix) == 8 and sum(mix) == 32768 and mix == group_sizes("mixtral", 0)
    assert group_sizes("mixtral", 1) != mix
    ds = group_sizes("deepseek_up", 0)
    assert len(ds) == 256 and sum(ds) == 65536 and ds == group_sizes("deepseek_down", 0)
    assert max(ds) > 50 * sorted(ds)[128]  # Zipf skew: the hottest expert dwarfs the median one
    wg = group_sizes("wgrad", 0)
    assert len(wg) == 64 and sum(wg) == 65536 and all(s % 8 == 0 for s in wg) and 0 in wg


@pytest.mark.parametrize("name", [n for n in CONFIG_NAMES if n != "readme"])
def test_scaled_workloads_have_the_documented_layouts(name):
    wl = make_workload(name, "cpu", seed=0, scale=1 / 64, dims_scale=1 / 16)
    assert wl.mat_a.dtype == torch.bfloat16 and wl.mat_b.dtype == torch.bfloat16
    if name.startswith("deepseek"):
        assert wl.mat_b.stride(-2) == 1  # column-major weights (a transposed [G, N, K] view)
    if name == "wgrad":
        assert wl.mat_a.stride() == (1, wl.mat_a.size(0)) and wl.out_dtype == torch.float32
    if wl.offs is not None:
        assert wl.offs.dtype == torch.int32 and int(wl.offs[-1]) == sum(wl.sizes)
    assert wl.flops > 0 and wl.algorithmic_bytes > 0


def test_flop_and_byte_counts_match_hand_arithmetic():
    wl = make_workload("readme", "cpu")
    assert wl.flops == 2 * 32 * 64 * 48
    # 4 non-empty groups: a 32x64, b 4x64x48, out 32x48, all bf16
    assert wl.algorithmic_bytes == 2 * (32 * 64 + 4 * 64 * 48) + 2 * 32 * 48


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_partition_is_contiguous_complete_and_bottleneck_optimal(world):
    sizes = group_sizes("deepseek_up", 0)
    parts = partition_groups(sizes, world)
    assert len(parts) == world and parts[0][0] == 0 and parts[-1][1] == len(sizes)
    assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
    worst = max(sum(sizes[lo:hi]) for lo, hi in parts)
    assert worst >= max(max(sizes), -(-sum(sizes) // world))
    assert 0 < imbalance(sizes, world) <= 1.0


def test_partition_bottleneck_matches_brute_force():
    import itertools
    import random

    rng = random.Random(0)
    for _ in range(60):
        n = rng.randint(2, 9)
        sizes = [rng.choice([0, 0, 1, 3, 7, 20, 50]) for _ in range(n)]
        for world in (2, 3, 4):
            if world >= n:
                continue
            best = min(max(sum(sizes[a:b]) for a, b in zip((0,) + cuts, cuts + (n,)))
                       for cuts in itertools.combinations(range(1, n), world - 1))
            got = max(sum(sizes[lo:hi]) for lo, hi in partition_groups(sizes, world))
            assert got == best, (sizes, world)


def test_one_group_per_rank_when_world_equals_groups():
    sizes = group_sizes("mixtral", 0)
    assert partition_groups(sizes, 8) == [(i, i + 1) for i in range(8)]
    assert shard_sizes(sizes, 8, 3) == [sizes[3]]
    assert partition_groups([5, 5], 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]  # more ranks than groups


def test_rebased_offsets():
    offs = torch.tensor([3, 3, 10, 14, 20], dtype=torch.int32)
    assert rebase_offsets(offs, 0, 2).tolist() == [3, 3]
    assert rebase_offsets(offs, 2, 5).tolist() == [7, 11, 17]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_path: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = make_workload("mixtral", "cpu", seed=0, scale=1 / 128, dims_scale=1 / 64)
        lo, hi = partition_groups(wl.sizes, world)[rank]
        row_lo = sum(wl.sizes[:lo])
        row_hi = row_lo + sum(wl.sizes[lo:hi])
        # the rank's shard: its rows of A, its experts' weights, offsets rebased to its first row
        local_out, _ = grouped_mm_oracle(wl.mat_a[row_lo:row_hi], wl.mat_b[lo:hi], rebase_offsets(wl.offs, lo, hi))
        rows = torch.tensor([row_hi - row_lo], dtype=torch.int64)
        all_rows = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(all_rows, rows)
        pad = max(int(r) for r in all_rows)
        padded = torch.zeros((pad, local_out.size(1)))
        padded[: local_out.size(0)] = local_out
        gathered = [torch.zeros_like(padded) for _ in range(world)]
        dist.all_gather(gathered, padded)  # verification only: never part of a timed region
        if rank == 0:
            full = torch.cat([g[: int(r)] for g, r in zip(gathered, all_rows)])
            ref, _ = grouped_mm_oracle(wl.mat_a, wl.mat_b, wl.offs)
            torch.save(dict(max_err=float((full - ref).abs().max()), rows=int(full.size(0))), out_path)
    finally:
        dist.destroy_process_group()


def test_partition_rows_balances_to_one_row_and_cuts_hot_groups():
    from grouped_mm_bf16_b200.workloads import partition_rows

    for name in ("mixtral", "deepseek_up", "wgrad"):
        sizes = group_sizes(name, 0)
        for world in (1, 2, 3, 4, 8):
            parts = partition_rows(sizes, world)
            loads = [sum(r for _, _, r in ps) for ps in parts]
            assert len(parts) == world and sum(loads) == sum(sizes) and max(loads) - min(loads) <= 1
            # the pieces, in rank order, tile every group exactly once and in order
            seen = {}
            last_g = -1
            for ps in parts:
                for g, first, rows in ps:
                    assert rows > 0 and g >= last_g and first == seen.get(g, 0)
                    seen[g] = first + rows
                    last_g = g
            assert all(seen.get(g, 0) == sz for g, sz in enumerate(sizes))
    # the hot expert of the Mixtral-shape draw (14787 of 32768 rows) is cut over four of eight ranks
    parts = partition_rows(group_sizes("mixtral", 0), 8)
    assert sum(1 for ps in parts if any(g == 0 for g, _, _ in ps)) == 4
    assert partition_rows([0, 5, 0, 3], 3) == [[(1, 0, 2)], [(1, 2, 3)], [(3, 0, 3)]]


def _rank_main_rows(rank, world, port, out_path):
    """Row-split sharding with a group cut across the two ranks: each rank holds a copy of the weights
    of the groups it touches, computes its rows with the CPU checker standing in for the device
    kernel, and the gathered rows must equal the unsharded result."""
    import torch.distributed as dist
    from grouped_mm_bf16_b200.workloads import partition_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sizes = [100, 20, 0, 9, 3]  # the first group holds most rows and is cut
        wl = make_workload("mixtral", "cpu", seed=3, sizes=sizes, dims_scale=1 / 64)
        pieces = partition_rows(sizes, world)[rank]
        starts = [sum(sizes[:g]) for g in range(len(sizes))]
        row0 = starts[pieces[0][0]] + pieces[0][1]
        local_rows = sum(r for _, _, r in pieces)
        a_local = wl.mat_a[row0:row0 + local_rows]
        b_local = wl.mat_b[[g for g, _, _ in pieces]]          # this rank's copies of the weights
        offs_local = torch.tensor([r for _, _, r in pieces]).cumsum(0).to(torch.int32)
        part, _ = grouped_mm_oracle(a_local, b_local, offs_local)
        gathered = [torch.zeros((sum(sizes), part.size(1))) for _ in range(world)]
        padded = torch.zeros((sum(sizes), part.size(1)))
        padded[:local_rows] = part
        dist.all_gather(gathered, padded)
        counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([local_rows]))
        if rank == 0:
            full = torch.cat([g[: int(c)] for g, c in zip(gathered, counts)])
            ref, _ = grouped_mm_oracle(wl.mat_a, wl.mat_b, wl.offs)
            torch.save(dict(max_err=float((full - ref).abs().max()), rows=int(full.size(0)),
                            cut=len(pieces) >= 1 and pieces[-1][2] < sizes[pieces[-1][0]]), out_path)
    finally:
        dist.destroy_process_group()


def test_two_rank_row_split_with_a_cut_group_over_gloo(tmp_path):
    out = tmp_path / "result_rows.pt"
    mp.spawn(_rank_main_rows, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    res = torch.load(out)
    assert res["rows"] == 132 and res["max_err"] == 0.0 and res["cut"]


def test_two_rank_group_sharding_over_gloo(tmp_path):
    out = tmp_path / "result.pt"
    mp.spawn(_rank_main, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    res = torch.load(out)
    assert res["rows"] == 256 and res["max_err"] == 0.0


def test_host_entry_plan_covers_every_row_once_and_uploads_weights_once():
    """grouped_mm_host's work items: every row of every non-empty group in exactly one item, a tall
    group cut into row pieces that upload its weights only with the first piece, tall groups first."""
    from grouped_mm_bf16_b200.host import plan_items

    for sizes, chunk in ((group_sizes("mixtral", 0), 192 << 20), ([300, 0, 513, 255, 257, 0, 40, 0], 1 << 12),
                         ([5, 0, 7], 1 << 30), ([0, 0], 1 << 20)):
        starts = [sum(sizes[:i]) for i in range(len(sizes))]
        k, n, es = (4096, 14336, 2) if len(sizes) == 8 and max(sizes) > 1000 else (200, 264, 2)
        items = plan_items(sizes, starts, (k + n) * es, k * n * es, chunk)
        covered = [0] * (sum(sizes) + 1)
        uploads = [0] * len(sizes)
        for lo, hi, r0, r1, new_b in items:
            assert 0 <= lo < hi <= len(sizes) and r0 < r1
            assert r0 >= starts[lo] and r1 <= starts[hi - 1] + sizes[hi - 1]
            if not new_b:
                assert hi == lo + 1, "only a single tall group is continued"
            for r in range(r0, r1):
                covered[r] += 1
            if new_b:
                for g in range(lo, hi):
                    uploads[g] += 1
        assert covered[:-1] == [1] * sum(sizes)
        assert all(u == 1 for g, u in enumerate(uploads) if sizes[g] > 0)
    items = plan_items(group_sizes("mixtral", 0), [0, 14787, 17079, 17633, 17912, 19184, 21224, 22213],
                       (4096 + 14336) * 2, 4096 * 14336 * 2, 192 << 20)
    assert items[0][:2] == (0, 1) and items[0][4] and not items[1][4]  # the hot expert first, in pieces
