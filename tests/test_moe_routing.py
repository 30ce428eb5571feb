"""MoE routing helpers: expert ids -> (offs, perm, inv_perm), row gather, weighted scatter.

CPU part: the oracle's own invariants. GPU part: the CUDA kernels against the oracle, bit for
bit for the integer results and the gathered rows, and a whole routed layer
(route -> permute -> grouped_mm -> combine) against a dense per-token computation.
"""

import pytest
import torch

from oracle.moe_oracle import combine_oracle, permute_oracle, route_oracle


def _ids(tokens, topk, experts, seed, skew=False):
    g = torch.Generator().manual_seed(seed)
    if skew:
        p = torch.arange(1, experts + 1, dtype=torch.float64).pow(-1.1)
        return torch.multinomial((p / p.sum()).float().expand(tokens, -1), topk, generator=g).to(torch.int32)
    return torch.randint(0, experts, (tokens, topk), generator=g, dtype=torch.int32)


def test_oracle_matches_bincount_cumsum_and_is_a_stable_sort():
    ids = _ids(500, 2, 8, seed=0)
    offs, perm, inv = route_oracle(ids, 8)
    flat = ids.reshape(-1).long()
    assert offs.tolist() == torch.bincount(flat, minlength=8).cumsum(0).tolist()  # the reference's producer
    sorted_ids = flat[perm.long()]
    assert bool((sorted_ids[1:] >= sorted_ids[:-1]).all())
    same = sorted_ids[1:] == sorted_ids[:-1]
    assert bool((perm[1:][same] > perm[:-1][same]).all()), "ties keep assignment order"
    assert torch.equal(inv[perm.long()].long(), torch.arange(1000))


def test_oracle_drops_out_of_range_ids():
    ids = torch.tensor([[0, 9], [-1, 1], [1, 0]], dtype=torch.int32)
    offs, perm, inv = route_oracle(ids, 2)
    assert offs.tolist() == [2, 4] and perm.tolist() == [0, 5, 3, 4, -1, -1] and inv.tolist() == [0, -1, -1, 2, 3, 1]


gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("tokens,topk,experts,skew", [
    (16384, 2, 8, False),      # Mixtral-shape routing
    (8192, 8, 256, True),      # DeepSeek-shape routing, Zipf-skewed
    (1000, 1, 1023, False),    # the group limit, mostly empty experts
    (1, 1, 4, False), (33, 3, 5, False), (4097, 2, 7, True),
])
def test_route_matches_oracle_bit_for_bit(built_library, tokens, topk, experts, skew):
    from grouped_mm_bf16_b200 import moe

    ids = _ids(tokens, topk, experts, seed=tokens + experts, skew=skew)
    offs, perm, inv = moe.route(ids.cuda(), experts)
    o_ref, p_ref, i_ref = route_oracle(ids, experts)
    assert torch.equal(offs.cpu(), o_ref) and torch.equal(perm.cpu(), p_ref) and torch.equal(inv.cpu(), i_ref)
    # run-to-run identical (no atomics race decides an order)
    offs2, perm2, inv2 = moe.route(ids.cuda(), experts)
    assert torch.equal(perm2, perm) and torch.equal(inv2, inv) and torch.equal(offs2, offs)


@gpu
def test_route_ignores_out_of_range_ids(built_library):
    from grouped_mm_bf16_b200 import moe

    ids = torch.tensor([[0, 9], [-1, 1], [1, 0]], dtype=torch.int32)
    offs, perm, inv = moe.route(ids.cuda(), 2)
    assert offs.tolist() == [2, 4] and perm.tolist() == [0, 5, 3, 4, -1, -1] and inv.tolist() == [0, -1, -1, 2, 3, 1]
    with pytest.raises(RuntimeError, match="1024 groups"):
        moe.route(ids.cuda(), 1024)
    with pytest.raises(RuntimeError, match="int32"):
        moe.route(ids.long().cuda(), 2)
    with pytest.raises(RuntimeError, match="GPU-only"):
        moe.route(ids, 2)


@gpu
@pytest.mark.parametrize("k,dtype", [(4096, torch.bfloat16), (72, torch.bfloat16), (33, torch.bfloat16), (17, torch.float32)])
def test_permute_and_combine_match_oracle(built_library, k, dtype):
    from grouped_mm_bf16_b200 import moe

    tokens, topk, experts = 777, 2, 8
    ids = _ids(tokens, topk, experts, seed=k)
    g = torch.Generator().manual_seed(k)
    x = torch.randn(tokens, k, generator=g).to(dtype)
    w = torch.rand(tokens, topk, generator=g)
    offs, perm, inv = moe.route(ids.cuda(), experts)
    a = moe.permute(x.cuda(), perm, topk)
    assert torch.equal(a.cpu(), permute_oracle(x, perm, topk))  # a gather moves bits, it does not round
    y = torch.randn(tokens * topk, k, generator=g).to(dtype)
    out = moe.combine(y.cuda(), inv, w.cuda(), topk, out_dtype=torch.float32)
    torch.testing.assert_close(out.cpu(), combine_oracle(y, inv, w, topk), atol=1e-5, rtol=1e-5)
    out_lp = moe.combine(y.cuda(), inv, None, topk)
    torch.testing.assert_close(out_lp.float().cpu(), combine_oracle(y, inv, None, topk), atol=2e-2, rtol=8e-3)


@gpu
def test_routed_layer_matches_dense_per_token_computation(built_library):
    """route -> permute -> grouped_mm -> combine equals, token by token, sum_k w * (x @ W[e_k])."""
    from grouped_mm_bf16_b200 import grouped_mm, moe

    tokens, topk, experts, k, n = 512, 2, 8, 256, 384
    ids = _ids(tokens, topk, experts, seed=5)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    wts = (torch.randn(experts, k, n, generator=g) * 0.05).bfloat16()
    gate = torch.rand(tokens, topk, generator=g)
    offs, perm, inv = moe.route(ids.cuda(), experts)
    y = grouped_mm(moe.permute(x.cuda(), perm, topk), wts.cuda(), offs=offs)
    out = moe.combine(y, inv, gate.cuda(), topk, out_dtype=torch.float32).cpu()
    per_choice = torch.einsum("tk,tckn->tcn", x.float(), wts.float()[ids.long()])  # [tokens, topk, n]
    ref = (per_choice.bfloat16().float() * gate.unsqueeze(-1)).sum(1)  # y is rounded to bf16 before the combine
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=8e-3)


@gpu
def test_feed_forward_matches_dense_per_token_computation(built_library):
    """moe.feed_forward equals, token by token, sum_k w_k * (silu(x @ gate_e) * (x @ up_e)) @ down_e."""
    from grouped_mm_bf16_b200 import moe

    tokens, topk, experts, hidden, inter = 384, 2, 8, 256, 320
    ids = _ids(tokens, topk, experts, seed=9)
    ids[7, 1] = experts + 3  # an assignment that is routed nowhere
    g = torch.Generator().manual_seed(9)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    gate_up = (torch.randn(experts, hidden, 2 * inter, generator=g) * 0.06).bfloat16()
    down = (torch.randn(experts, inter, hidden, generator=g) * 0.06).bfloat16()
    w = torch.rand(tokens, topk, generator=g)
    with torch.no_grad():
        out = moe.feed_forward(x.cuda(), ids.cuda(), w.cuda(), gate_up.cuda(), down.cuda(), out_dtype=torch.float32).cpu()
    valid = (ids >= 0) & (ids < experts)
    e = ids.clamp(0, experts - 1).long()
    both = torch.einsum("th,tchn->tcn", x.float(), gate_up.float()[e])             # [tokens, topk, 2 inter]
    act = (torch.nn.functional.silu(both[..., :inter]) * both[..., inter:]).bfloat16().float()
    y = torch.einsum("tci,tcih->tch", act, down.float()[e]).bfloat16().float()      # rounded like the kernels' outputs
    ref = (y * (w * valid).unsqueeze(-1)).sum(1)
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=1e-2)


@gpu
def test_feed_forward_replays_from_a_cuda_graph(built_library):
    """No step of the block needs the host, so the whole block can be captured once and replayed on
    new tokens and new routing written into the same buffers."""
    from grouped_mm_bf16_b200 import moe

    tokens, topk, experts, hidden, inter = 256, 2, 8, 128, 192
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(21)
    gate_up = (torch.randn((experts, hidden, 2 * inter), device=dev, generator=g) * 0.08).bfloat16()
    down = (torch.randn((experts, inter, hidden), device=dev, generator=g) * 0.08).bfloat16()
    x = torch.randn((tokens, hidden), device=dev, generator=g).bfloat16()
    ids = torch.randint(0, experts, (tokens, topk), device=dev, dtype=torch.int32, generator=g)
    w = torch.rand((tokens, topk), device=dev, generator=g)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(2):  # warm-up outside the capture: library load, workspace, allocator pools
            moe.feed_forward(x, ids, w, gate_up, down)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), torch.no_grad():
        out = moe.feed_forward(x, ids, w, gate_up, down)
    for seed in (22, 23):
        g2 = torch.Generator(device=dev).manual_seed(seed)
        x.copy_(torch.randn((tokens, hidden), device=dev, generator=g2).bfloat16())
        ids.copy_(torch.randint(0, experts, (tokens, topk), device=dev, dtype=torch.int32, generator=g2))
        w.copy_(torch.rand((tokens, topk), device=dev, generator=g2))
        graph.replay()
        with torch.no_grad():
            eager = moe.feed_forward(x, ids, w, gate_up, down)
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
