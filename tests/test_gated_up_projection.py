"""The fused gated up-projection (``silu(x @ gate) * (x @ up)`` in the GEMM's epilogue) against the
CPU oracle and against the unfused sequence ``grouped_mm`` -> activation.

Tolerance: both products accumulate in fp32 and the result is rounded once to the 16-bit output,
so |out - ref| <= 8e-3 |ref| + 1e-2 (bf16 rounding is 2^-9 relative); fp32 outputs are held to 1e-4 relative.
"""

import pytest
import torch

from grouped_mm_bf16_b200 import _op, grouped_mm
from grouped_mm_bf16_b200.moe import gated_up_projection
from oracle.moe_oracle import gated_up_oracle

DEV = torch.device("cuda")


def _offs(sizes):
    return torch.tensor(sizes, dtype=torch.int64).cumsum(0).to(torch.int32).to(DEV)


def test_gated_up_oracle_is_the_unfused_formula():
    g = torch.Generator().manual_seed(3)
    sizes = [3, 0, 5, 1]
    x = torch.randn((sum(sizes) + 2, 16), generator=g)
    w = torch.randn((4, 16, 12), generator=g)
    out, defined = gated_up_oracle(x, w, torch.tensor(sizes).cumsum(0).to(torch.int32))
    assert defined.tolist() == [True] * 9 + [False] * 2
    row = 4  # second row of group 2
    both = x[row] @ w[2]
    torch.testing.assert_close(out[row], torch.nn.functional.silu(both[:6]) * both[6:])


def test_argument_checks_need_no_gpu():
    x = torch.zeros((4, 8), dtype=torch.bfloat16)
    w = torch.zeros((2, 8, 16), dtype=torch.bfloat16)
    offs = torch.tensor([2, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="GPU-only"):
        gated_up_projection(x, w, offs)


gpu = pytest.mark.gpu


@pytest.fixture()
def _clear_status(built_library):
    yield
    assert _op.check_status(DEV) == 0, "a bounded wait inside a kernel gave up"


def _check(x, w, offs, out_dtype=None, expect_fused=True, pair=None, monkeypatch=None):
    if pair is not None:
        monkeypatch.setenv("GROUPED_MM_B200_PAIR", "1" if pair else "0")
    n = w.size(2) // 2
    # is the fused kernel taken? ask the library about the same operands
    probe = torch.empty((x.size(0), n), dtype=out_dtype or x.dtype, device=DEV)
    fused = _op.grouped_mm_2d3d_swiglu(x, w, offs, probe)
    assert fused == expect_fused
    with torch.no_grad():
        out = gated_up_projection(x, w, offs, out_dtype=out_dtype)
    assert out.shape == (x.size(0), n) and out.dtype == (out_dtype or x.dtype)
    ref, defined = gated_up_oracle(x, w, offs)
    got = out.float().cpu()
    if out.dtype == torch.float32:
        torch.testing.assert_close(got[defined], ref[defined], rtol=1e-4, atol=1e-3)
    else:
        torch.testing.assert_close(got[defined], ref[defined], rtol=8e-3, atol=1e-2)
    if fused:
        torch.testing.assert_close(probe.float().cpu()[defined], got[defined], rtol=0, atol=0)
    return out


SIZES = [
    [128, 128, 128],
    [127, 1, 128],
    [129, 0, 255, 1],
    [40, 30, 10, 7],
    [0, 0, 300, 0, 0],
    [1, 0] * 12,
    [300, 0, 513, 255, 257],
]


@gpu
@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("sizes", SIZES)
@pytest.mark.parametrize("k,n,col_major", [(64, 48, False), (200, 136, False), (72, 264, True), (8, 8, True), (64, 128, False),
                                          (72, 36, True), (64, 21, True)])  # column-major weights: any N
def test_fused_matches_oracle(sizes, k, n, col_major, pair, monkeypatch, _clear_status):
    g = torch.Generator(device=DEV).manual_seed(len(sizes) * 100 + k + n)
    x = (torch.randn((sum(sizes), k), device=DEV, generator=g) * 0.5).bfloat16()
    if col_major:
        w = (torch.randn((len(sizes), 2 * n, k), device=DEV, generator=g) * 0.3).bfloat16().transpose(-2, -1)
    else:
        w = (torch.randn((len(sizes), k, 2 * n), device=DEV, generator=g) * 0.3).bfloat16()
    _check(x, w, _offs(sizes), pair=pair, monkeypatch=monkeypatch)


@gpu
@pytest.mark.parametrize("dtype,out_dtype", [(torch.float16, None), (torch.bfloat16, torch.float32), (torch.float16, torch.float32)])
def test_fused_dtypes(dtype, out_dtype, _clear_status):
    g = torch.Generator(device=DEV).manual_seed(5)
    sizes = [129, 0, 255, 1]
    x = (torch.randn((sum(sizes), 200), device=DEV, generator=g) * 0.5).to(dtype)
    w = (torch.randn((4, 200, 2 * 136), device=DEV, generator=g) * 0.3).to(dtype)
    _check(x, w, _offs(sizes), out_dtype=out_dtype)


@gpu
def test_rows_past_the_last_offset_and_neighbouring_memory_stay_untouched(_clear_status):
    g = torch.Generator(device=DEV).manual_seed(7)
    sizes = [70, 0, 33]
    extra = 9
    x = (torch.randn((sum(sizes) + extra, 64), device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn((3, 64, 2 * 136), device=DEV, generator=g) * 0.3).bfloat16()
    big = torch.full((x.size(0) + 2, 144), 777.0, dtype=torch.bfloat16, device=DEV)
    out = big[1:-1, :136]
    assert _op.grouped_mm_2d3d_swiglu(x, w, _offs(sizes), out)
    ref, defined = gated_up_oracle(x, w, _offs(sizes))
    torch.testing.assert_close(out.float().cpu()[defined], ref[defined], rtol=8e-3, atol=1e-2)
    assert bool((out[sum(sizes):] == 777.0).all()), "rows past offs[-1] were written"
    assert bool((big[:, 136:] == 777.0).all()) and bool((big[0] == 777.0).all()) and bool((big[-1] == 777.0).all())


@gpu
def test_unfusable_operands_take_the_two_step_path_with_the_same_values(_clear_status):
    g = torch.Generator(device=DEV).manual_seed(11)
    sizes = [40, 0, 25]
    # odd N with a row-major weight: the up half does not start on a 16-byte boundary
    x = (torch.randn((sum(sizes), 64), device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn((3, 64, 2 * 36), device=DEV, generator=g) * 0.3).bfloat16()
    _check(x, w, _offs(sizes), expect_fused=False)
    # fp32 operands
    _check(x.float(), w.float(), _offs(sizes), expect_fused=False)
    # odd K: pitches are not multiples of 16 bytes
    x = (torch.randn((sum(sizes), 33), device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn((3, 33, 2 * 40), device=DEV, generator=g) * 0.3).bfloat16()
    _check(x, w, _offs(sizes), expect_fused=False)


@gpu
def test_fused_equals_grouped_mm_then_activation_on_a_mixtral_shaped_slice(_clear_status):
    """1/8 of the Mixtral dimensions: 8 experts, K = 512, N = 1792 (weights [8, 512, 3584])."""
    g = torch.Generator(device=DEV).manual_seed(13)
    sizes = [1900, 300, 75, 33, 150, 250, 120, 1268]
    x = torch.randn((sum(sizes), 512), device=DEV, generator=g).bfloat16()
    w = (torch.randn((8, 512, 2 * 1792), device=DEV, generator=g) * 0.02).bfloat16()
    offs = _offs(sizes)
    with torch.no_grad():
        fused = gated_up_projection(x, w, offs)
        both = grouped_mm(x, w, offs=offs, out_dtype=torch.float32)
    two_step = (torch.nn.functional.silu(both[:, :1792]) * both[:, 1792:]).bfloat16()
    torch.testing.assert_close(fused.float(), two_step.float(), rtol=8e-3, atol=1e-3)
    ref, defined = gated_up_oracle(x, w, offs)
    assert bool(defined.all())
    torch.testing.assert_close(fused.float().cpu(), ref, rtol=8e-3, atol=1e-3)


@gpu
@pytest.mark.parametrize("col_major", [False, True])
def test_gradients_match_an_fp32_torch_reference(col_major, _clear_status):
    g = torch.Generator(device=DEV).manual_seed(17)
    sizes = [129, 0, 255, 1, 40]
    k, n = 200, 136
    extra = 3  # rows past offs[-1] belong to no group and get zero gradient
    x = (torch.randn((sum(sizes) + extra, k), device=DEV, generator=g) * 0.5).bfloat16().requires_grad_()
    if col_major:
        w = (torch.randn((len(sizes), 2 * n, k), device=DEV, generator=g) * 0.3).bfloat16().transpose(-2, -1)
    else:
        w = (torch.randn((len(sizes), k, 2 * n), device=DEV, generator=g) * 0.3).bfloat16()
    w = w.detach().requires_grad_()
    dy = torch.randn((x.size(0), n), device=DEV, generator=g).bfloat16()
    out = gated_up_projection(x, w, _offs(sizes))
    valid = sum(sizes)
    (out[:valid].float() * dy[:valid].float()).sum().backward()

    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    start, pieces = 0, []
    for gi, sz in enumerate(sizes):
        both = xr[start:start + sz] @ wr[gi]
        pieces.append(torch.nn.functional.silu(both[:, :n]) * both[:, n:])
        start += sz
    (torch.cat(pieces) * dy[:valid].float()).sum().backward()
    assert w.grad.stride() == w.stride()
    # operands of the gradient GEMMs are rounded to bf16 once more: 8e-3 relative plus the spec's sqrt(K) term
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=0.15)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=0.3)
    assert not x.grad[valid:].any()
    assert not w.grad[1].any(), "an empty group's weights get a zero gradient"
