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


def _gpu_rank(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from grouped_mm_bf16_b200 import _op

        x, ids, w, gate_up, down = _problem(rank, torch.bfloat16)
        e_local = EXPERTS // world
        mine = slice(rank * e_local, (rank + 1) * e_local)
        with torch.no_grad():
            out = ep.feed_forward(x.to(dev), ids.to(dev), w.to(dev), gate_up[mine].to(dev), down[mine].to(dev),
                                  out_dtype=torch.float32)
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
