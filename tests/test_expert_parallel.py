"""Expert-parallel routed feed-forward: the exchange and its index arithmetic on two CPU ranks over
gloo (host stand-ins from ``oracle/`` for the kernels), and the real thing on two GPUs over NCCL.

Each rank holds its own tokens and half of the experts; the result for a rank's tokens has to equal
the dense per-token computation with all experts' weights.
"""

import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grouped_mm_bf16_b200 import expert_parallel as ep
from oracle.grouped_mm_oracle import grouped_mm_oracle
from oracle.moe_oracle import combine_oracle, gated_up_oracle, permute_oracle, route_oracle

EXPERTS, TOPK, HIDDEN, INTER = 8, 2, 64, 96


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def oracle_ops() -> SimpleNamespace:
    """Host stand-ins with the signatures of the CUDA steps (fp32 throughout)."""
    def permute(x, perm, topk, n_rows=None):
        return permute_oracle(x, perm, topk)[: perm.numel() if n_rows is None else n_rows].contiguous()

    def combine(y, inv, weights, topk, out_dtype=None):
        return combine_oracle(y, inv, weights, topk).to(out_dtype or y.dtype)

    return SimpleNamespace(route=route_oracle, permute=permute, combine=combine,
                           gated_up_projection=lambda x, w, offs: gated_up_oracle(x, w, offs)[0],
                           grouped_mm=lambda a, b, offs: grouped_mm_oracle(a, b, offs)[0])


def _problem(rank: int, dtype):
    """This rank's tokens and routing, and ALL experts' weights (the same on every rank)."""
    g = torch.Generator().manual_seed(100)
    gate_up = (torch.randn(EXPERTS, HIDDEN, 2 * INTER, generator=g) * 0.1).to(dtype)
    down = (torch.randn(EXPERTS, INTER, HIDDEN, generator=g) * 0.1).to(dtype)
    g = torch.Generator().manual_seed(200 + rank)
    tokens = 37 + 11 * rank
    x = torch.randn(tokens, HIDDEN, generator=g).to(dtype)
    ids = torch.randint(0, EXPERTS, (tokens, TOPK), generator=g, dtype=torch.int32)
    ids[3, 1] = EXPERTS + 2  # routed nowhere
    if rank == 1:
        ids[ids == 5] = 4    # expert 5 gets nothing from rank 1
    w = torch.rand(tokens, TOPK, generator=g)
    return x, ids, w, gate_up, down


def _dense_reference(x, ids, w, gate_up, down, round_to=None):
    valid = (ids >= 0) & (ids < EXPERTS)
    e = ids.clamp(0, EXPERTS - 1).long()
    both = torch.einsum("th,tchn->tcn", x.float(), gate_up.float()[e])
    act = torch.nn.functional.silu(both[..., :INTER]) * both[..., INTER:]
    if round_to is not None:
        act = act.to(round_to).float()
    y = torch.einsum("tci,tcih->tch", act, down.float()[e])
    if round_to is not None:
        y = y.to(round_to).float()
    return (y * (w * valid).unsqueeze(-1)).sum(1)


def test_received_rows_are_labelled_by_source_rank_then_expert():
    recv_counts = torch.tensor([[2, 0, 1], [0, 3, 1]], dtype=torch.int32)  # [source rank, local expert]
    ids = ep.received_expert_ids(recv_counts, 7)
    assert ids.tolist() == [0, 0, 2, 1, 1, 1, 2] and ids.dtype == torch.int32
    counts = torch.tensor([[1, 1, 0], [4, 0, 2]], dtype=torch.int32)
    assert ep.split_sizes(counts, recv_counts) == ([2, 6], [3, 4])


@pytest.mark.parametrize("world,e_local,topk", [(2, 4, 2), (3, 2, 3), (4, 1, 1)])
def test_exchange_plan_places_every_row_once_in_expert_order(world, e_local, topk):
    """All ranks simulated in one process: following every rank's tables, each routed row lands on
    the owner of its expert, exactly once, inside that expert's segment of the owner's buffer, the
    segments are what offs_local says, and the way back finds the same row again."""
    experts = world * e_local
    g = torch.Generator().manual_seed(world)
    ids = [torch.randint(0, experts + 1, (20 + 7 * r, topk), generator=g, dtype=torch.int32) for r in range(world)]
    routes = [route_oracle(i, experts) for i in ids]  # id == experts is routed nowhere
    counts_all = torch.stack([torch.diff(o, prepend=o.new_zeros(1)) for o, _, _ in routes])
    cap = int(counts_all.sum())
    expert_at = [torch.full((cap,), -1, dtype=torch.long) for _ in range(world)]
    origin_at = [torch.full((cap,), -1, dtype=torch.long) for _ in range(world)]
    plans = []
    for r in range(world):
        offs, perm, inv = routes[r]
        plan = ep.exchange_plan(offs, perm, inv, counts_all, r, e_local)
        plans.append(plan)
        dst_rank, dst_row = plan[0], plan[1]
        assert all(t.dtype == torch.int32 for t in plan)
        flat = ids[r].reshape(-1)
        for p in range(perm.numel()):
            if perm[p] < 0:
                assert dst_rank[p] == -1 and dst_row[p] == -1
                continue
            assert expert_at[dst_rank[p]][dst_row[p]] == -1, "two rows were sent to the same place"
            expert_at[dst_rank[p]][dst_row[p]] = int(flat[perm[p]])
            origin_at[dst_rank[p]][dst_row[p]] = r * 10000 + int(perm[p])
    for r in range(world):
        offs_local = plans[r][4]
        n = int(offs_local[-1])
        assert bool((expert_at[r][:n] >= 0).all()) and bool((expert_at[r][n:] == -1).all())
        start = 0
        for e in range(e_local):
            assert bool((expert_at[r][start:int(offs_local[e])] == r * e_local + e).all())
            start = int(offs_local[e])
        src_rank, src_row = plans[r][2], plans[r][3]
        flat = ids[r].reshape(-1)
        for a in range(flat.numel()):
            if flat[a] >= experts:
                assert src_rank[a] == -1
            else:
                assert origin_at[src_rank[a]][src_row[a]] == r * 10000 + a


def _cpu_rank(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, ids, w, gate_up, down = _problem(rank, torch.float32)
        e_local = EXPERTS // world
        mine = slice(rank * e_local, (rank + 1) * e_local)
        out = ep.feed_forward(x, ids, w, gate_up[mine], down[mine], ops=oracle_ops(), out_dtype=torch.float32)
        ref = _dense_reference(x, ids, w, gate_up, down)
        torch.save(dict(err=float((out - ref).abs().max()), scale=float(ref.abs().max()), rows=out.size(0)),
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_over_gloo_match_the_dense_computation(tmp_path):
    mp.spawn(_cpu_rank, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank, rows in ((0, 37), (1, 48)):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["rows"] == rows
        assert res["err"] <= 1e-4 * max(1.0, res["scale"]), res


def _gpu_rank(rank: int, world: int, port: int, out_dir: str, peer_memory: bool = False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from grouped_mm_bf16_b200 import _op

        x, ids, w, gate_up, down = _problem(rank, torch.bfloat16)
        e_local = EXPERTS // world
        mine = slice(rank * e_local, (rank + 1) * e_local)
        args = (x.to(dev), ids.to(dev), w.to(dev), gate_up[mine].to(dev), down[mine].to(dev))
        with torch.no_grad():
            if peer_memory:
                buffers = ep.PeerBuffers(world * 64 * TOPK, HIDDEN, torch.bfloat16, dev)
                out = ep.feed_forward_peer(*args, buffers, out_dtype=torch.float32)
                out2 = ep.feed_forward_peer(*args, buffers, out_dtype=torch.float32)  # buffers are reusable
                assert torch.equal(out, out2)
            else:
                out = ep.feed_forward(*args, out_dtype=torch.float32)
        status = _op.check_status(dev)
        ref = _dense_reference(x, ids, w, gate_up, down, round_to=torch.bfloat16)
        torch.save(dict(out=out.cpu(), ref=ref, status=status), os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpus_over_nccl_match_the_dense_computation(tmp_path, built_library):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_gpu_rank, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in (0, 1):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["status"] == 0
        torch.testing.assert_close(res["out"], res["ref"], atol=2e-2, rtol=1e-2)


@pytest.mark.gpu
def test_two_gpus_with_rows_moved_over_peer_memory(tmp_path, built_library):
    """The same block with the dispatch written into, and the combine read from, the peers' buffers."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_gpu_rank, args=(2, _free_port(), str(tmp_path), True), nprocs=2, join=True)
    for rank in (0, 1):
        res = torch.load(tmp_path / f"rank{rank}.pt")
        assert res["status"] == 0
        torch.testing.assert_close(res["out"], res["ref"], atol=2e-2, rtol=1e-2)
