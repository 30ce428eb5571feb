"""GPU parity: the CUDA path against the CPU oracle, the golden fixtures and size-independent
properties. Tolerance (from the operator's specification): |out - ref| <= 8e-3 |ref| + 1e-2 sqrt(K) sigma_a sigma_b,
with ref the fp32 per-group matmul of the same bf16 inputs; fp32 inputs are held to 3e-4.
"""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from grouped_mm_bf16_b200 import _lib, _op, grouped_mm
from grouped_mm_bf16_b200.workloads import group_sizes, make_workload
from oracle.grouped_mm_oracle import atol_for, group_bounds, grouped_mm_oracle, max_violation

DEV = torch.device("cuda")
FORMS = {"3d3d": _lib.FORM_3D3D, "2d3d": _lib.FORM_2D3D, "3d2d": _lib.FORM_3D2D, "2d2d": _lib.FORM_2D2D}


@pytest.fixture(autouse=True)
def _status_word_stays_clear(built_library):
    yield
    assert _op.check_status(DEV) == 0, "a bounded wait inside a kernel gave up"


@pytest.fixture(params=["single_cta", "cta_pair"])
def tile_kernel(request, monkeypatch):
    """Runs a test once with the single-CTA (128-row tiles) and once with the CTA-pair
    (cta_group::2, 256-row tiles) variant of the tcgen05 kernel."""
    monkeypatch.setenv("GROUPED_MM_B200_PAIR", "1" if request.param == "cta_pair" else "0")
    return request.param


class force_generic:
    def __enter__(self):
        self.prev = os.environ.get("GROUPED_MM_B200_FORCE_GENERIC")
        os.environ["GROUPED_MM_B200_FORCE_GENERIC"] = "1"

    def __exit__(self, *exc):
        if self.prev is None:
            os.environ.pop("GROUPED_MM_B200_FORCE_GENERIC", None)
        else:
            os.environ["GROUPED_MM_B200_FORCE_GENERIC"] = self.prev


def _offs(sizes):
    return torch.tensor(sizes, dtype=torch.int64).cumsum(0).to(torch.int32).to(DEV)


def _form(a, b):
    return {(2, 3): "2d3d", (3, 3): "3d3d", (3, 2): "3d2d", (2, 2): "2d2d"}[(a.dim(), b.dim())]


def _assert_parity(a, b, offs, sigma_a, sigma_b, out_dtype=None, expect_kernel=None):
    """Runs the operator and checks it against the oracle with the specification's tolerance."""
    out = grouped_mm(a, b, offs=offs, out_dtype=out_dtype)
    ref, defined = grouped_mm_oracle(a, b, offs)
    form = _form(a, b)
    if expect_kernel is not None:
        kind = _op.selected_kernel(FORMS[form], a, b, out)
        # "tcgen05" stands for either tile variant; which one ran is decided by shape and environment
        assert kind == expect_kernel or (expect_kernel == _lib.GMM_KERNEL_TCGEN05 and kind in _lib.TCGEN05_KINDS)
    if form == "2d2d":
        # K is the group's own length; an empty group must be exactly zero.
        for g, (s, e) in enumerate(group_bounds(offs.cpu(), a.size(1))):
            v = max_violation(out[g], ref[g], defined[g], atol_for(e - s, sigma_a, sigma_b))
            assert v <= 1.0, f"group {g} (k range {s}:{e}) violates tolerance by {v:.3g}x"
    else:
        v = max_violation(out, ref, defined, atol_for(a.size(-1), sigma_a, sigma_b))
        assert v <= 1.0, f"violates tolerance by {v:.3g}x"
    return out


# ----------------------------------------------------------------------------- golden fixtures


def test_golden_fixtures_on_gpu(golden_cases):
    for c in golden_cases:
        a, b = c["a"].to(DEV), c["b"].to(DEV)
        assert a.stride() == c["a"].stride() and b.stride() == c["b"].stride()
        offs = None if c["offs"] is None else c["offs"].to(DEV)
        out = grouped_mm(a, b, offs=offs)
        _, defined = grouped_mm_oracle(c["a"], c["b"], c["offs"])
        got, want = out.float().cpu()[defined], c["out"].float()[defined]
        if a.dtype == torch.float32:
            torch.testing.assert_close(got, want, atol=3e-4, rtol=3e-4)
        else:
            torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2)


# ----------------------------------------------------------------------------- the five configurations


def test_readme_config_through_the_c_abi(built_library):
    """Config 1, called through the raw C entry point with pointers, sizes and strides."""
    wl = make_workload("readme", DEV, seed=0)
    lib = _lib.load()
    out = torch.full((32, 48), float("nan"), dtype=torch.bfloat16, device=DEV)
    ws = torch.zeros(64, dtype=torch.int32, device=DEV)
    a, b, c = _op._desc(wl.mat_a), _op._desc(wl.mat_b), _op._desc(out)
    launch = _lib.GmmLaunch()
    launch.stream = torch.cuda.current_stream().cuda_stream
    launch.workspace, launch.workspace_bytes, launch.flags = ws.data_ptr(), ws.numel() * 4, 0
    rc = lib.grouped_mm_2d3d(ctypes.byref(a), ctypes.byref(b), ctypes.c_void_p(wl.offs.data_ptr()), 6,
                             ctypes.byref(c), ctypes.byref(launch))
    assert rc == 0, _lib.error_message(lib, rc)
    raw = ctypes.c_int32(-1)
    assert lib.gmm_check_status(ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(launch.stream), ctypes.byref(raw)) == 0
    assert raw.value == 0
    ref, defined = grouped_mm_oracle(wl.mat_a, wl.mat_b, wl.offs)
    assert bool(defined.all())
    assert max_violation(out, ref, defined, atol_for(64, 1.0, 1.0)) <= 1.0


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("name,scale,dims_scale", [
    ("readme", 1.0, 1.0),
    ("batched", 1.0, 1 / 8),
    ("mixtral", 1 / 16, 1 / 8),
    ("deepseek_up", 1 / 16, 1 / 8),
    ("deepseek_down", 1 / 16, 1 / 8),
    ("wgrad", 1 / 16, 1 / 8),
])
def test_scaled_configs_match_oracle(name, scale, dims_scale, generic, tile_kernel):
    wl = make_workload(name, DEV, seed=0, scale=scale, dims_scale=dims_scale)
    if generic:
        with force_generic():
            _assert_parity(wl.mat_a, wl.mat_b, wl.offs, wl.sigma_a, wl.sigma_b, wl.out_dtype, _lib.GMM_KERNEL_GENERIC)
    else:
        _assert_parity(wl.mat_a, wl.mat_b, wl.offs, wl.sigma_a, wl.sigma_b, wl.out_dtype, _lib.GMM_KERNEL_TCGEN05)


def test_deepseek_variant_with_forced_empty_groups():
    sizes = group_sizes("deepseek_up", 0, 1 / 16)
    sizes = [0 if i % 3 == 1 else s for i, s in enumerate(sizes)]
    wl = make_workload("deepseek_up", DEV, seed=0, dims_scale=1 / 8, sizes=sizes)
    _assert_parity(wl.mat_a, wl.mat_b, wl.offs, wl.sigma_a, wl.sigma_b, None, _lib.GMM_KERNEL_TCGEN05)


# ----------------------------------------------------------------------------- tile-boundary cases

M_PATTERNS = [
    [128, 128, 128],            # every group a whole tile
    [127, 1, 128],              # single-row group ending on a tile boundary
    [129, 0, 255, 1],           # one row past a tile, empty group, one row short of two tiles
    [40, 30, 10, 7],            # several groups inside one tile
    [0, 0, 300, 0, 0],          # leading and trailing empties
    [1, 0] * 12,                # alternating single rows and empties
    [5, 0, 7, 0, 3, 9],
    [32, 16, 0, 0, 0],
    [700],                      # one group, several tiles with a tail
    [300, 0, 513, 255, 257],    # around the 256-row tiles of the CTA-pair kernel
]


@pytest.mark.parametrize("sizes", M_PATTERNS)
@pytest.mark.parametrize("k,n,b_col_major", [(64, 48, False), (200, 264, False), (72, 520, True), (8, 8, True)])
def test_2d3d_tile_boundaries_tcgen05(sizes, k, n, b_col_major, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(len(sizes) * 1000 + k + n)
    a = torch.randn((sum(sizes), k), device=DEV, generator=g).bfloat16()
    if b_col_major:
        b = torch.randn((len(sizes), n, k), device=DEV, generator=g).bfloat16().transpose(-2, -1)
    else:
        b = torch.randn((len(sizes), k, n), device=DEV, generator=g).bfloat16()
    _assert_parity(a, b, _offs(sizes), 1.0, 1.0, None, _lib.GMM_KERNEL_TCGEN05)


@pytest.mark.parametrize("sizes", M_PATTERNS[:6])
def test_2d3d_odd_shapes_generic(sizes):
    g = torch.Generator(device=DEV).manual_seed(7)
    k, n = 33, 29
    a = torch.randn((sum(sizes), k), device=DEV, generator=g).bfloat16()
    b = torch.randn((len(sizes), k, n), device=DEV, generator=g).bfloat16()
    _assert_parity(a, b, _offs(sizes), 1.0, 1.0, None, _lib.GMM_KERNEL_GENERIC)


K_PATTERNS = [[64, 64], [8, 0, 16, 24, 8], [7, 0, 1, 13, 11], [63, 65, 1, 127], [0, 0, 200], [300, 0, 0]]


@pytest.mark.parametrize("sizes", K_PATTERNS)
@pytest.mark.parametrize("m,n", [(16, 24), (136, 264), (128, 256)])
@pytest.mark.parametrize("out_dtype", [None, torch.float32])
def test_2d2d_k_ragged_tcgen05(sizes, m, n, out_dtype, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(sum(sizes) + m)
    kt = sum(sizes)
    a = torch.randn((kt, m), device=DEV, generator=g).bfloat16().t()  # column-major [M, K_total]
    b = torch.randn((kt, n), device=DEV, generator=g).bfloat16()
    _assert_parity(a, b, _offs(sizes), 1.0, 1.0, out_dtype, _lib.GMM_KERNEL_TCGEN05)


@pytest.mark.parametrize("sizes", K_PATTERNS)
def test_2d2d_row_major_a_generic(sizes):
    g = torch.Generator(device=DEV).manual_seed(11)
    kt = sum(sizes)
    a = torch.randn((16, kt), device=DEV, generator=g).bfloat16()
    b = torch.randn((kt, 24), device=DEV, generator=g).bfloat16()
    _assert_parity(a, b, _offs(sizes), 1.0, 1.0, None, _lib.GMM_KERNEL_GENERIC)


@pytest.mark.parametrize("sizes", [[7, 0, 1, 13, 11], [128, 130, 0, 60], [1, 0] * 10])
@pytest.mark.parametrize("b_col_major,kernel", [(True, _lib.GMM_KERNEL_TCGEN05), (False, _lib.GMM_KERNEL_GENERIC)])
def test_3d2d_n_ragged(sizes, b_col_major, kernel, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(13)
    m, k, nt = 40, 48, sum(sizes)
    a = torch.randn((len(sizes), m, k), device=DEV, generator=g).bfloat16()
    b = torch.randn((nt, k), device=DEV, generator=g).bfloat16().t() if b_col_major else \
        torch.randn((k, nt), device=DEV, generator=g).bfloat16()
    # the output's leading stride is padded to 16 bytes; nt here is not always a multiple of 8
    _assert_parity(a, b, _offs(sizes), 1.0, 1.0, None, kernel)


@pytest.mark.parametrize("a_col_major", [False, True])
@pytest.mark.parametrize("b_col_major", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_3d3d_all_layouts(a_col_major, b_col_major, dtype, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(17)
    G, m, k, n = 3, 136, 200, 264
    a = torch.randn((G, k, m), device=DEV, generator=g).to(dtype).transpose(-2, -1) if a_col_major else \
        torch.randn((G, m, k), device=DEV, generator=g).to(dtype)
    b = torch.randn((G, n, k), device=DEV, generator=g).to(dtype).transpose(-2, -1) if b_col_major else \
        torch.randn((G, k, n), device=DEV, generator=g).to(dtype)
    _assert_parity(a, b, None, 1.0, 1.0, None, _lib.GMM_KERNEL_TCGEN05)


def test_fp32_inputs_are_true_fp32():
    g = torch.Generator(device=DEV).manual_seed(19)
    sizes = [0, 7, 1, 13, 0, 11]
    a = torch.randn((32, 29), device=DEV, generator=g)
    b = torch.randn((6, 29, 31), device=DEV, generator=g)
    out = grouped_mm(a, b, offs=_offs(sizes))
    ref, _ = grouped_mm_oracle(a, b, _offs(sizes))
    torch.testing.assert_close(out.cpu(), ref, atol=3e-4, rtol=3e-4)
    # aligned fp32 operands too, as long as torch's TF32 knob is off (its default)
    assert not torch.backends.cuda.matmul.allow_tf32
    a = torch.randn((32, 64), device=DEV, generator=g)
    b = torch.randn((6, 64, 48), device=DEV, generator=g)
    out = grouped_mm(a, b, offs=_offs(sizes))
    assert _op.selected_kernel(_lib.FORM_2D3D, a, b, out) == _lib.GMM_KERNEL_GENERIC
    ref, _ = grouped_mm_oracle(a, b, _offs(sizes))
    torch.testing.assert_close(out.cpu(), ref, atol=3e-4, rtol=3e-4)


# ----------------------------------------------------------------------------- fp32 operands as TF32


class allow_tf32:
    """Sets torch.backends.cuda.matmul.allow_tf32, the knob the reference hands to its kernels as
    ALLOW_TF32 (kernels.py:185-194), for the duration of a block."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


def _as_tf32(x):
    """fp32 with the low 13 mantissa bits cleared: what the tensor cores read of an fp32 operand.
    Keeps the shape and strides of ``x``."""
    out = torch.empty_like(x)  # preserves the layout of dense, possibly transposed, tensors
    out.copy_(x)
    flat = out.as_strided((out.untyped_storage().nbytes() // 4,), (1,), 0)
    flat.copy_((flat.view(torch.int32) & ~0x1FFF).view(torch.float32))
    return out


def _assert_tf32_parity(a, b, offs):
    """With TF32 allowed the tcgen05 kernel runs; its result equals the fp32-accumulated product of
    the TF32-truncated operands (to fp32 summation-order noise), and differs from the exact product
    by at most 2^-9 sum|a||b| (two operands, each short of its fp32 value by less than 2^-10)."""
    with allow_tf32():
        out = grouped_mm(a, b, offs=offs)
        assert out.dtype == torch.float32
        assert _op.selected_kernel(FORMS[_form(a, b)], a, b, out) in _lib.TCGEN05_KINDS
    ref_t, defined = grouped_mm_oracle(_as_tf32(a), _as_tf32(b), offs)
    torch.testing.assert_close(out.cpu()[defined], ref_t[defined], atol=1e-3, rtol=1e-4)
    ref, _ = grouped_mm_oracle(a, b, offs)
    bound, _ = grouped_mm_oracle(a.abs(), b.abs(), offs)
    excess = ((out.cpu() - ref).abs() - (bound * 2.0 ** -9 + 1e-3))[defined]
    assert excess.numel() == 0 or excess.max().item() <= 0.0
    return out


@pytest.mark.parametrize("a_col_major", [False, True])
@pytest.mark.parametrize("b_col_major", [False, True])
def test_tf32_3d3d_all_layouts(a_col_major, b_col_major, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(53)
    G, m, k, n = 3, 136, 200, 264
    a = torch.randn((G, k, m), device=DEV, generator=g).transpose(-2, -1) if a_col_major else \
        torch.randn((G, m, k), device=DEV, generator=g)
    b = torch.randn((G, n, k), device=DEV, generator=g).transpose(-2, -1) if b_col_major else \
        torch.randn((G, k, n), device=DEV, generator=g)
    _assert_tf32_parity(a, b, None)


@pytest.mark.parametrize("sizes", M_PATTERNS)
@pytest.mark.parametrize("k,n,b_col_major", [(64, 48, False), (200, 264, False), (72, 520, True), (4, 4, True)])
def test_tf32_2d3d_tile_boundaries(sizes, k, n, b_col_major, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(len(sizes) * 1000 + k + n + 1)
    a = torch.randn((sum(sizes), k), device=DEV, generator=g)
    if b_col_major:
        b = torch.randn((len(sizes), n, k), device=DEV, generator=g).transpose(-2, -1)
    else:
        b = torch.randn((len(sizes), k, n), device=DEV, generator=g)
    out = _assert_tf32_parity(a, b, _offs(sizes))
    if sum(sizes) == 0:
        assert out.numel() == 0


@pytest.mark.parametrize("sizes", K_PATTERNS)
@pytest.mark.parametrize("m,n", [(16, 24), (136, 264), (128, 256)])
def test_tf32_2d2d_k_ragged(sizes, m, n, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(sum(sizes) + m + 1)
    kt = sum(sizes)
    a = torch.randn((kt, m), device=DEV, generator=g).t()  # column-major [M, K_total]
    b = torch.randn((kt, n), device=DEV, generator=g)
    out = _assert_tf32_parity(a, b, _offs(sizes))
    for gi, sz in enumerate(sizes):
        if sz == 0:
            assert not out[gi].any(), "an empty group has to give exact zeros"


@pytest.mark.parametrize("sizes", [[7, 0, 1, 13, 11], [128, 130, 0, 60], [1, 0] * 10])
def test_tf32_3d2d_n_ragged(sizes, tile_kernel):
    g = torch.Generator(device=DEV).manual_seed(59)
    m, k, nt = 40, 48, sum(sizes)
    a = torch.randn((len(sizes), m, k), device=DEV, generator=g)
    b = torch.randn((nt, k), device=DEV, generator=g).t()
    _assert_tf32_parity(a, b, _offs(sizes))


def test_tf32_unaligned_operands_small_stay_generic_large_are_relaid_out():
    g = torch.Generator(device=DEV).manual_seed(61)
    sizes = [0, 7, 1, 13, 0, 11]
    a = torch.randn((32, 29), device=DEV, generator=g)
    b = torch.randn((6, 29, 31), device=DEV, generator=g)
    with allow_tf32():
        out = grouped_mm(a, b, offs=_offs(sizes))
        assert _op.selected_kernel(_lib.FORM_2D3D, a, b, out) == _lib.GMM_KERNEL_GENERIC
    ref, _ = grouped_mm_oracle(a, b, _offs(sizes))
    torch.testing.assert_close(out.cpu(), ref, atol=3e-4, rtol=3e-4)  # true fp32 on the generic kernel
    sizes = [700, 0, 901]
    a = torch.randn((sum(sizes), 1001), device=DEV, generator=g)
    b = torch.randn((3, 1001, 1003), device=DEV, generator=g)
    with allow_tf32():
        out = grouped_mm(a, b, offs=_offs(sizes))
        assert _op._worth_relayout(_lib.FORM_2D3D, a, b, out)
        a2, b2 = _op.tensor_core_layouts(_lib.FORM_2D3D, a, b)
        assert torch.equal(a2, a) and torch.equal(b2, b)
        assert _op.selected_kernel(_lib.FORM_2D3D, a2, b2, out) in _lib.TCGEN05_KINDS
    assert not _op._worth_relayout(_lib.FORM_2D3D, a, b, out)  # knob off again: fp32 stays true fp32
    ref_t, _ = grouped_mm_oracle(_as_tf32(a), _as_tf32(b), _offs(sizes))
    torch.testing.assert_close(out.cpu(), ref_t, atol=2e-3, rtol=1e-4)


def test_tf32_backward_matches_fp32_reference():
    """Gradients of fp32 operands run through the same kernels on transposed views."""
    g = torch.Generator(device=DEV).manual_seed(67)
    sizes = [129, 0, 255, 1, 40]
    a = torch.randn((sum(sizes), 200), device=DEV, generator=g).requires_grad_()
    b = torch.randn((len(sizes), 200, 264), device=DEV, generator=g).requires_grad_()
    with allow_tf32():
        out = grouped_mm(a, b, offs=_offs(sizes))
        out.backward(torch.ones_like(out))
    a_ref, b_ref = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    start = 0
    pieces = []
    for gi, sz in enumerate(sizes):
        pieces.append(a_ref[start:start + sz] @ b_ref[gi])
        start += sz
    torch.cat(pieces).sum().backward()
    torch.testing.assert_close(a.grad, a_ref.grad, atol=0.3, rtol=2e-2)
    torch.testing.assert_close(b.grad, b_ref.grad, atol=0.3, rtol=2e-2)


@pytest.mark.parametrize("form", ["2d3d", "3d2d", "2d2d"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_1023_groups(form, dtype, tile_kernel):
    """Alternating one-element and empty groups with a trailing empty group
    (the reference's large-group-count cases, tests/test_grouped_mm.py:661-747)."""
    sizes = [1 if i % 2 == 0 else 0 for i in range(1023)]
    sizes[-1] = 0
    offs, total = _offs(sizes), sum(sizes)
    g = torch.Generator(device=DEV).manual_seed(23)
    if form == "2d3d":
        a = torch.randn((total, 8), device=DEV, generator=g).to(dtype)
        b = torch.randn((1023, 8, 8), device=DEV, generator=g).to(dtype)
    elif form == "3d2d":
        a = torch.randn((1023, 4, 8), device=DEV, generator=g).to(dtype)
        b = torch.randn((total, 8), device=DEV, generator=g).to(dtype).t()
    else:
        a = torch.randn((total, 8), device=DEV, generator=g).to(dtype).t()
        b = torch.randn((total, 8), device=DEV, generator=g).to(dtype)
    if dtype == torch.float32:
        out = grouped_mm(a, b, offs=offs)
        ref, defined = grouped_mm_oracle(a, b, offs)
        torch.testing.assert_close(out.cpu()[defined], ref[defined], atol=3e-4, rtol=3e-4)
    else:
        _assert_parity(a, b, offs, 1.0, 1.0)


def test_registered_torch_custom_op():
    """The op registered with torch.library (the traceable entry used under torch.compile) gives
    the same bits as the eager path, which calls the same launcher directly."""
    wl = make_workload("mixtral", DEV, seed=2, scale=1 / 32, dims_scale=1 / 8)
    want = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    got = torch.empty_like(want)
    assert torch.ops.grouped_mm_b200.forward(wl.mat_a, wl.mat_b, wl.offs, got, _lib.FORM_2D3D) is None
    assert torch.equal(got, want)


@pytest.mark.parametrize("chunk_bytes", [1 << 12, 1 << 20, 1 << 30])
def test_host_buffer_entry_matches_device_entry(chunk_bytes):
    """grouped_mm_host (pinned host in/out, chunked copy/compute overlap) gives the bits of grouped_mm."""
    from grouped_mm_bf16_b200.host import grouped_mm_host

    sizes = [300, 0, 513, 255, 257, 0, 40, 0]
    g = torch.Generator().manual_seed(41)
    a = torch.randn((sum(sizes) + 11, 200), generator=g).bfloat16().pin_memory()  # 11 rows belong to no group
    b = torch.randn((len(sizes), 200, 264), generator=g).bfloat16().pin_memory()
    offs = torch.tensor(sizes, dtype=torch.int64).cumsum(0).to(torch.int32)
    out = torch.full((a.size(0), 264), 7.0, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):  # the second call reuses the staging slots of the first
        got = grouped_mm_host(a, b, offs, out=out, chunk_bytes=chunk_bytes)
        torch.cuda.current_stream().synchronize()
        want = grouped_mm(a.to(DEV), b.to(DEV), offs=offs.to(DEV)).cpu()
        assert got is out and torch.equal(got[: sum(sizes)], want[: sum(sizes)])
        assert bool((got[sum(sizes):] == 7.0).all()), "rows past offs[-1] were written"
    ref, defined = grouped_mm_oracle(a, b, offs)
    assert max_violation(out, ref, defined, atol_for(200, 1.0, 1.0)) <= 1.0
    with pytest.raises(RuntimeError, match="host tensors"):
        grouped_mm_host(a.to(DEV), b, offs)


def test_torch_compile_traces_through_the_custom_op():
    """Under torch.compile the call goes through the registered custom op (with its fake-tensor
    rule); the "eager" backend runs dynamo's tracing without generating code, so this is quick."""
    wl = make_workload("mixtral", DEV, seed=5, scale=1 / 64, dims_scale=1 / 8)

    def fn(a, b, offs):
        return grouped_mm(a, b, offs=offs).float() * 2.0

    compiled = torch.compile(fn, backend="eager")
    got = compiled(wl.mat_a, wl.mat_b, wl.offs)
    assert torch.equal(got, fn(wl.mat_a, wl.mat_b, wl.offs))


def test_backward_under_torch_compile():
    """Forward and backward through torch.compile with the aot_eager backend: AOTAutograd traces the
    autograd function's backward with fake tensors, so every launch in it has to be a registered
    custom op (the GEMMs and the zero-fill past offs[-1])."""
    wl = make_workload("mixtral", DEV, seed=6, scale=1 / 64, dims_scale=1 / 8)
    offs = wl.offs.clone()
    offs[-1] -= 5  # the last five rows belong to no group: their gradient must be zero

    a1, b1 = wl.mat_a.clone().requires_grad_(True), wl.mat_b.clone().requires_grad_(True)
    a2, b2 = wl.mat_a.clone().requires_grad_(True), wl.mat_b.clone().requires_grad_(True)
    # rows past offs[-1] are left as allocated by the forward pass: keep them out of the loss
    def masked(a, b):
        return (grouped_mm(a, b, offs=offs)[: int(offs[-1])].float() ** 2).sum()

    masked(a1, b1).backward()
    torch.compile(masked, backend="aot_eager")(a2, b2).backward()
    assert torch.equal(a1.grad, a2.grad) and torch.equal(b1.grad, b2.grad)
    assert float(a1.grad[int(offs[-1]):].abs().max()) == 0.0


def test_zero_past_offsets_entry_point():
    """gmm_zero_past_offsets zero-fills exactly the part at or past offs[-1], along either dimension,
    for contiguous and strided tensors, and touches nothing when offs[-1] is the extent."""
    for dtype in (torch.bfloat16, torch.float32):
        for dim in (0, 1):
            for end in (0, 13, 40):
                base = torch.ones((40, 56), dtype=dtype, device=DEV)
                t = base[:, :40] if dim == 1 else base[:, :33]
                offs = torch.tensor([5, end], dtype=torch.int32, device=DEV)
                _op.zero_past_offsets(t, dim, offs)
                want = torch.ones_like(base)
                if dim == 0:
                    want[end:, :33] = 0
                else:
                    want[:, end:40] = 0
                assert torch.equal(base, want), (dtype, dim, end)
    tr = torch.ones((24, 16), dtype=torch.bfloat16, device=DEV).t()  # column-major [16, 24]
    _op.zero_past_offsets(tr, 1, torch.tensor([20], dtype=torch.int32, device=DEV))
    assert float(tr[:, :20].min()) == 1.0 and float(tr[:, 20:].abs().max()) == 0.0


def test_2d2d_without_group_maps_is_refused(built_library):
    """The K-ragged tensor-core path needs the caller's group_maps buffer; without it the C entry
    point returns GMM_ERR_WORKSPACE and launches nothing."""
    wl = make_workload("wgrad", DEV, seed=0, scale=1 / 16, dims_scale=1 / 8)
    lib = _lib.load()
    out = torch.zeros((wl.offs.numel(), wl.mat_a.size(0), wl.mat_b.size(1)), dtype=torch.float32, device=DEV)
    a, b, c = _op._desc(wl.mat_a), _op._desc(wl.mat_b), _op._desc(out)
    ws = _op.workspace(DEV)
    launch = _lib.GmmLaunch()
    launch.stream = torch.cuda.current_stream().cuda_stream
    launch.workspace, launch.workspace_bytes, launch.flags = ws.data_ptr(), ws.numel() * 4, 0
    rc = lib.grouped_mm_2d2d(ctypes.byref(a), ctypes.byref(b), ctypes.c_void_p(wl.offs.data_ptr()), wl.offs.numel(),
                             ctypes.byref(c), ctypes.byref(launch))
    assert rc == -4
    need = int(lib.gmm_group_maps_bytes(wl.offs.numel()))
    assert need == 256 * wl.offs.numel()
    maps = torch.empty(need, dtype=torch.uint8, device=DEV)
    launch.group_maps, launch.group_maps_bytes = maps.data_ptr(), need
    rc = lib.grouped_mm_2d2d(ctypes.byref(a), ctypes.byref(b), ctypes.c_void_p(wl.offs.data_ptr()), wl.offs.numel(),
                             ctypes.byref(c), ctypes.byref(launch))
    assert rc == 0
    assert torch.equal(out, grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs, out_dtype=torch.float32))


@pytest.mark.parametrize("b_col_major", [False, True])
def test_tail_tiles_of_at_most_64_rows_as_m64_mma(b_col_major, monkeypatch):
    """The single-CTA kernel multiplies a tile with at most 64 valid rows with M = 64 instructions
    (64 fetched rows, another TMEM layout in the epilogue). Group sizes around the 64- and 128-row
    boundaries, checked against the oracle with the feature on and off, and against each other:
    the accumulation order per output element is the same, so the bits are."""
    monkeypatch.setenv("GROUPED_MM_B200_PAIR", "0")
    sizes = [1, 63, 64, 65, 0, 130, 192, 17, 128, 129 + 64]
    g = torch.Generator(device=DEV).manual_seed(23)
    a = torch.randn((sum(sizes) + 5, 200), device=DEV, generator=g).bfloat16()
    b = torch.randn((len(sizes), 520, 200), device=DEV, generator=g).bfloat16().transpose(-2, -1) if b_col_major \
        else torch.randn((len(sizes), 200, 520), device=DEV, generator=g).bfloat16()
    offs = _offs(sizes)
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("GROUPED_MM_B200_HALF_TILES", flag)
        outs[flag] = _assert_parity(a, b, offs, 1.0, 1.0, None, _lib.GMM_KERNEL_TCGEN05)
        out32 = _assert_parity(a, b, offs, 1.0, 1.0, torch.float32, _lib.GMM_KERNEL_TCGEN05)
        assert out32.dtype == torch.float32
    assert torch.equal(outs["1"][: sum(sizes)], outs["0"][: sum(sizes)])
    # uniform (3D x 3D) blocks of 40 rows are half tiles as well
    a3 = torch.randn((3, 40, 136), device=DEV, generator=g).bfloat16()
    b3 = torch.randn((3, 136, 264), device=DEV, generator=g).bfloat16()
    monkeypatch.setenv("GROUPED_MM_B200_HALF_TILES", "1")
    _assert_parity(a3, b3, None, 1.0, 1.0, None, _lib.GMM_KERNEL_TCGEN05)


def test_2d2d_with_few_output_tiles_splits_the_contraction(monkeypatch):
    """M = N = 256 and 4 groups give 4 output tiles for 74 CTA pairs: the call is run as 4 x S groups
    whose fp32 partial products are summed in a fixed order. Checked against the oracle, against the
    unsplit kernel, and for run-to-run reproducibility; an empty group stays exactly zero."""
    sizes = [24576, 0, 8200, 16376]
    gen = torch.Generator(device=DEV).manual_seed(9)
    a = torch.randn((sum(sizes), 256), device=DEV, generator=gen).bfloat16().t()
    b = torch.randn((sum(sizes), 256), device=DEV, generator=gen).bfloat16()
    offs = _offs(sizes)
    assert _op._split_k_factor(a, b, offs) > 1
    out = _assert_parity(a, b, offs, 1.0, 1.0, torch.float32, _lib.GMM_KERNEL_TCGEN05)
    assert float(out[1].abs().max()) == 0.0
    assert torch.equal(out, grouped_mm(a, b, offs=offs, out_dtype=torch.float32))
    out_bf16 = _assert_parity(a, b, offs, 1.0, 1.0, None, _lib.GMM_KERNEL_TCGEN05)
    monkeypatch.setenv("GROUPED_MM_B200_SPLIT_K", "0")
    unsplit = grouped_mm(a, b, offs=offs, out_dtype=torch.float32)
    torch.testing.assert_close(out, unsplit, atol=atol_for(24576, 1, 1) * 0.1, rtol=1e-4)
    assert out_bf16.dtype == torch.bfloat16


def test_side_stream_and_cuda_graph_replay():
    """The call only enqueues work on the current stream (no host sync, no allocation inside the
    library), so it can run on a side stream and be captured into a CUDA graph and replayed."""
    wl = make_workload("mixtral", DEV, seed=3, scale=1 / 32, dims_scale=1 / 8)
    want = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        got = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    side.synchronize()
    assert torch.equal(got, want)

    static_a = wl.mat_a.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = grouped_mm(static_a, wl.mat_b, offs=wl.offs)
    other = make_workload("mixtral", DEV, seed=4, scale=1 / 32, dims_scale=1 / 8, sizes=wl.sizes)
    static_a.copy_(other.mat_a)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, grouped_mm(other.mat_a, wl.mat_b, offs=wl.offs))

    # The K-ragged form: its per-group tensor maps are written on the device, by a kernel that is part
    # of the captured work, from whatever `offs` holds when the graph runs; a replay after `offs`
    # has been overwritten in place computes the new split.
    wg = make_workload("wgrad", DEV, seed=0, scale=1 / 16, dims_scale=1 / 8)
    grouped_mm(wg.mat_a, wg.mat_b, offs=wg.offs, out_dtype=torch.float32)  # outside the capture: one-time set-up
    static_offs = wg.offs.clone()
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        static_out2 = grouped_mm(wg.mat_a, wg.mat_b, offs=static_offs, out_dtype=torch.float32)
    other_offs = _offs(list(reversed(wg.sizes)))
    assert not torch.equal(other_offs, wg.offs)
    static_offs.copy_(other_offs)
    graph2.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out2, grouped_mm(wg.mat_a, wg.mat_b, offs=other_offs, out_dtype=torch.float32))


def test_k_ragged_calls_on_two_streams_do_not_share_their_group_maps():
    """Every 2D x 2D call takes its own scratch for the per-group tensor maps from torch's stream-aware
    allocator, so calls in flight on different streams, with different offsets, do not disturb each
    other (a shared buffer would let one call's map-building kernel overwrite maps the other's GEMM
    is still loading through)."""
    wg = make_workload("wgrad", DEV, seed=0, scale=1 / 4, dims_scale=1 / 4)
    offs_a, offs_b = wg.offs, _offs(list(reversed(wg.sizes)))
    want_a = grouped_mm(wg.mat_a, wg.mat_b, offs=offs_a, out_dtype=torch.float32)
    want_b = grouped_mm(wg.mat_a, wg.mat_b, offs=offs_b, out_dtype=torch.float32)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    got_a, got_b = [], []
    for _ in range(6):
        with torch.cuda.stream(s1):
            got_a.append(grouped_mm(wg.mat_a, wg.mat_b, offs=offs_a, out_dtype=torch.float32))
        with torch.cuda.stream(s2):
            got_b.append(grouped_mm(wg.mat_a, wg.mat_b, offs=offs_b, out_dtype=torch.float32))
    torch.cuda.synchronize()
    assert all(torch.equal(g, want_a) for g in got_a) and all(torch.equal(g, want_b) for g in got_b)


# ----------------------------------------------------------------------------- what must not be written


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("n,n_pad", [(40, 48), (264, 272)])
def test_guard_bands_stay_untouched(generic, n, n_pad, tile_kernel):
    """Padding columns, rows past offs[-1] and memory around the output keep their sentinel."""
    sizes = [100, 0, 29, 130, 300]  # offs[-1] = 559 < 600 rows
    k, rows, last = 64, 600, 559
    g = torch.Generator(device=DEV).manual_seed(29)
    a = torch.randn((rows, k), device=DEV, generator=g).bfloat16()
    b = torch.randn((len(sizes), k, n), device=DEV, generator=g).bfloat16()
    sentinel = 12345.0
    buf = torch.full((rows + 16, n_pad), sentinel, dtype=torch.bfloat16, device=DEV)
    out = buf[8:8 + rows, :n]
    offs = _offs(sizes)
    if generic:
        with force_generic():
            _op.grouped_mm_2d3d(a, b, offs, out)
    else:
        # the CTA-pair variant needs more than 128 columns; narrower outputs stay on the single-CTA kernel
        pair = tile_kernel == "cta_pair" and n > 128
        expected = _lib.GMM_KERNEL_TCGEN05_PAIR if pair else _lib.GMM_KERNEL_TCGEN05
        assert _op.selected_kernel(_lib.FORM_2D3D, a, b, out) == expected
        _op.grouped_mm_2d3d(a, b, offs, out)
    ref, defined = grouped_mm_oracle(a, b, offs)
    assert max_violation(out, ref, defined, atol_for(k, 1.0, 1.0)) <= 1.0
    assert bool((buf[:8] == sentinel).all()) and bool((buf[8 + rows:] == sentinel).all())
    assert bool((buf[:, n:] == sentinel).all()), "padding columns were written"
    assert bool((out[last:] == sentinel).all()), "rows past offs[-1] were written"


def test_offsets_beyond_the_extent_are_clamped():
    g = torch.Generator(device=DEV).manual_seed(31)
    a = torch.randn((40, 64), device=DEV, generator=g).bfloat16()
    b = torch.randn((3, 64, 48), device=DEV, generator=g).bfloat16()
    offs = torch.tensor([10, 25, 1000], dtype=torch.int32, device=DEV)
    _assert_parity(a, b, offs, 1.0, 1.0)


def test_results_are_bitwise_reproducible(tile_kernel):
    wl = make_workload("mixtral", DEV, seed=1, scale=1 / 16, dims_scale=1 / 8)
    first = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    for _ in range(3):
        assert torch.equal(first, grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs))
    wl = make_workload("wgrad", DEV, seed=1, scale=1 / 16, dims_scale=1 / 8)
    first = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs, out_dtype=torch.float32)
    assert torch.equal(first, grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs, out_dtype=torch.float32))


def test_zero_k_and_empty_outputs():
    a = torch.zeros((5, 0), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((2, 0, 8), dtype=torch.bfloat16, device=DEV)
    out = grouped_mm(a, b, offs=_offs([2, 3]))
    assert out.shape == (5, 8) and float(out.abs().sum()) == 0.0
    a = torch.zeros((0, 16), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((2, 16, 8), dtype=torch.bfloat16, device=DEV)
    assert grouped_mm(a, b, offs=_offs([0, 0])).shape == (0, 8)


def test_output_strides_are_padded_like_the_reference():
    a = torch.randn((32, 33), device=DEV).bfloat16()
    b = torch.randn((6, 33, 29), device=DEV).bfloat16()
    out = grouped_mm(a, b, offs=_offs([0, 7, 1, 13, 0, 11]))
    assert out.shape == (32, 29) and out.stride() == (32, 1)
    a3, b3 = torch.randn((3, 17, 19), device=DEV), torch.randn((3, 19, 23), device=DEV)
    assert grouped_mm(a3, b3).stride() == (17 * 24, 24, 1)


# ----------------------------------------------------------------------------- argument rules that need CUDA tensors


def test_offs_and_bias_rules():
    a = torch.zeros((8, 16), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((2, 16, 8), dtype=torch.bfloat16, device=DEV)
    offs = _offs([4, 4])
    with pytest.raises(RuntimeError, match="Have to provide offsets"):
        grouped_mm(a, b)
    with pytest.raises(RuntimeError, match="Have to provide offsets"):
        grouped_mm(torch.zeros((2, 8, 16), dtype=torch.bfloat16, device=DEV), b, offs=offs)
    with pytest.raises(RuntimeError, match="offs must be a CUDA/HIP tensor"):
        grouped_mm(a, b, offs=offs.cpu())
    with pytest.raises(RuntimeError, match="offs has to be 1D"):
        grouped_mm(a, b, offs=offs.view(1, 2))
    with pytest.raises(RuntimeError, match="Offsets have to be int32"):
        grouped_mm(a, b, offs=offs.long())
    with pytest.raises(RuntimeError, match="Can't process more than 1024 groups"):
        grouped_mm(a, torch.zeros((1024, 16, 8), dtype=torch.bfloat16, device=DEV),
                   offs=torch.zeros(1024, dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError, match="Bias not supported yet"):
        grouped_mm(a, b, offs=offs, bias=torch.zeros(8, device=DEV))
    with pytest.raises(RuntimeError, match="output dtype must match"):
        grouped_mm(a, b, offs=offs, out_dtype=torch.float16)
    with pytest.raises(RuntimeError, match="matrix batch sizes have to match"):
        grouped_mm(a, b, offs=_offs([4, 2, 2]))
    with pytest.raises(RuntimeError, match="Invalid strides/sizes"):
        grouped_mm(torch.zeros((8, 32), dtype=torch.bfloat16, device=DEV)[:, ::2], b, offs=offs)


def test_strict_alignment_mode(monkeypatch):
    a = torch.zeros((8, 33), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((2, 33, 8), dtype=torch.bfloat16, device=DEV)
    grouped_mm(a, b, offs=_offs([4, 4]))  # accepted by default, as in the reference
    monkeypatch.setenv("GROUPED_MM_B200_STRICT_ALIGN", "1")
    with pytest.raises(RuntimeError, match="multiple of 16 bytes"):
        grouped_mm(a, b, offs=_offs([4, 4]))


# ----------------------------------------------------------------------------- full-size configurations


def _slab_rows(start, end, slab=32):
    """One row out of every ``slab`` consecutive rows of [start, end), slabs counted from ``start``.

    The epilogue of both tcgen05 kernels stores a tile in pieces of 32 rows (one warp each), and tiles
    begin at the group's first row, so this takes a row from every (m-tile, warp) piece of the group.
    The position inside the slab varies from slab to slab so that every lane is met somewhere.
    """
    rows = []
    for i, s in enumerate(range(start, end, slab)):
        rows.append(s + (7 * i + 3) % min(slab, end - s))
    return rows


def _slab_complete_check(wl, out):
    """Compares one row of every 32-row slab of every group, over all N columns, with the fp32
    per-group matmul computed on the CPU. Returns how many rows were compared."""
    bounds = group_bounds(wl.offs.cpu(), wl.mat_a.size(0))
    atol = atol_for(wl.k, wl.sigma_a, wl.sigma_b)
    checked = 0
    for g, (s, e) in enumerate(bounds):
        if e <= s:
            continue
        idx = torch.tensor(_slab_rows(s, e), device=DEV)
        ref = wl.mat_a[idx].cpu().float() @ wl.mat_b[g].cpu().float()
        v = max_violation(out[idx], ref, torch.ones_like(ref, dtype=torch.bool), atol)
        assert v <= 1.0, f"group {g} (rows {s}:{e}): tolerance exceeded {v:.3g}x"
        checked += idx.numel()
    return checked


def test_mixtral_full_size_properties():
    wl = make_workload("mixtral", DEV, seed=0)
    assert wl.mat_a.shape == (32768, 4096) and wl.mat_b.shape == (8, 4096, 14336)
    out = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    assert _op.selected_kernel(_lib.FORM_2D3D, wl.mat_a, wl.mat_b, out) == _lib.GMM_KERNEL_TCGEN05_PAIR
    assert _slab_complete_check(wl, out) >= 32768 // 32
    # homogeneity: scaling A by a power of two scales the result exactly (bf16 exponent shift)
    assert torch.equal(grouped_mm(wl.mat_a * 2, wl.mat_b, offs=wl.offs), out * 2)
    # group independence: permuting the weights of two groups only changes those groups' rows
    b2 = wl.mat_b.clone()
    b2[[2, 3]] = wl.mat_b[[3, 2]]
    out2 = grouped_mm(wl.mat_a, b2, offs=wl.offs)
    bounds = group_bounds(wl.offs.cpu(), 32768)
    assert torch.equal(out2[: bounds[2][0]], out[: bounds[2][0]]) and torch.equal(out2[bounds[3][1]:], out[bounds[3][1]:])
    assert torch.isfinite(out.float()).all()


def test_mixtral_full_size_single_cta_kernel_slab_complete(monkeypatch):
    """The same workload on the 128-row single-CTA tiles (the kernel short groups get)."""
    monkeypatch.setenv("GROUPED_MM_B200_PAIR", "0")
    wl = make_workload("mixtral", DEV, seed=0)
    out = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    assert _op.selected_kernel(_lib.FORM_2D3D, wl.mat_a, wl.mat_b, out) == _lib.GMM_KERNEL_TCGEN05
    assert _slab_complete_check(wl, out) >= 32768 // 32


@pytest.mark.parametrize("name", ["deepseek_up", "deepseek_down"])
def test_deepseek_full_size_slab_complete(name):
    wl = make_workload(name, DEV, seed=0)
    assert wl.mat_b.stride(-2) == 1  # column-major weights
    out = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    assert _op.selected_kernel(_lib.FORM_2D3D, wl.mat_a, wl.mat_b, out) == _lib.GMM_KERNEL_TCGEN05
    assert _slab_complete_check(wl, out) >= 65536 // 32


def test_batched_full_size_slab_complete():
    wl = make_workload("batched", DEV, seed=0)
    out = grouped_mm(wl.mat_a, wl.mat_b)
    atol = atol_for(wl.k, wl.sigma_a, wl.sigma_b)
    for g in range(wl.mat_a.size(0)):
        rows = torch.tensor(_slab_rows(0, wl.mat_a.size(1)), device=DEV)
        ref = wl.mat_a[g][rows].float().cpu() @ wl.mat_b[g].float().cpu()
        v = max_violation(out[g][rows], ref, torch.ones_like(ref, dtype=torch.bool), atol)
        assert v <= 1.0, f"batch {g}: tolerance exceeded {v:.3g}x"


def test_wgrad_full_size_slab_complete_and_checksum():
    wl = make_workload("wgrad", DEV, seed=0)
    assert wl.mat_a.shape == (4096, 65536) and wl.mat_a.stride() == (1, 4096)
    out = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs, out_dtype=torch.float32)
    assert out.dtype == torch.float32 and out.shape == (64, 4096, 1536)
    assert _op.selected_kernel(_lib.FORM_2D2D, wl.mat_a, wl.mat_b, out) == _lib.GMM_KERNEL_TCGEN05_PAIR
    bounds = group_bounds(wl.offs.cpu(), 65536)
    empties = [g for g, (s, e) in enumerate(bounds) if e == s]
    assert empties, "the seeded draw has empty groups"
    rows = torch.tensor(_slab_rows(0, 4096), device=DEV)
    a_rows = wl.mat_a[rows].float().cpu()  # [128, 65536]
    b_cpu = wl.mat_b.float().cpu()
    for g, (s, e) in enumerate(bounds):
        if e == s:
            assert float(out[g].abs().max()) == 0.0, f"empty group {g} is not all zeros"
            continue
        ref = a_rows[:, s:e] @ b_cpu[s:e]
        v = max_violation(out[g][rows], ref, torch.ones_like(ref, dtype=torch.bool), atol_for(e - s, 1, 1))
        assert v <= 1.0, f"group {g} (k range {s}:{e}): tolerance exceeded {v:.3g}x"
    # the sum over groups of a K-partitioned product is the plain product A @ B
    rows = torch.tensor([5, 1000, 4000], device=DEV)
    total = out[:, rows, :].sum(0).cpu()
    ref = wl.mat_a[rows].float().cpu() @ b_cpu
    torch.testing.assert_close(total, ref, atol=atol_for(65536, 1, 1), rtol=8e-3)


def test_reference_env_knobs_are_accepted_and_ignored(monkeypatch):
    """The reference picks a debug implementation and tile sizes from GROUPED_MM_2D3D_* variables
    (grouped_mm_bf16/kernels.py:590-634). They are accepted here and change nothing."""
    wl = make_workload("readme", DEV, seed=0)
    want = grouped_mm(wl.mat_a, wl.mat_b, offs=wl.offs)
    monkeypatch.setenv("GROUPED_MM_2D3D_IMPL", "rowwise")
    monkeypatch.setenv("GROUPED_MM_2D3D_BLOCK_M", "32")
    monkeypatch.setenv("GROUPED_MM_2D3D_BLOCK_N", "64")
    got = _assert_parity(wl.mat_a, wl.mat_b, wl.offs, wl.sigma_a, wl.sigma_b)
    assert torch.equal(got, want)


# ----------------------------------------------------------------------------- large unaligned problems


@pytest.mark.parametrize("form", ["2d3d", "2d3d_colmajor_a", "3d3d", "2d2d_rowmajor_a", "3d2d_rowmajor_b"])
def test_large_unaligned_problems_are_relaid_out_for_the_tensor_cores(form):
    """Odd K and N, or a contiguous ragged dimension, normally mean the generic kernel. Above a size
    threshold the operands are copied into an aligned layout first, so the tensor-core kernels run;
    the values, and so the result, are the same."""
    g = torch.Generator(device=DEV).manual_seed(47)
    sizes = [700, 0, 901]
    rnd = lambda *shape: torch.randn(shape, device=DEV, generator=g).bfloat16()  # noqa: E731
    if form == "2d3d":
        a, b, offs, code = rnd(sum(sizes), 1001), rnd(3, 1001, 1003), _offs(sizes), _lib.FORM_2D3D
    elif form == "2d3d_colmajor_a":
        a, b, offs, code = rnd(1000, sum(sizes)).t(), rnd(3, 1000, 1003), _offs(sizes), _lib.FORM_2D3D
    elif form == "3d3d":
        a, b, offs, code = rnd(3, 701, 1001), rnd(3, 1001, 1003), None, _lib.FORM_3D3D
    elif form == "2d2d_rowmajor_a":
        a, b, offs, code = rnd(1001, sum(sizes)), rnd(sum(sizes), 1003), _offs(sizes), _lib.FORM_2D2D
    else:
        a, b, offs, code = rnd(3, 1001, 1000), rnd(1000, sum(sizes)), _offs(sizes), _lib.FORM_3D2D
    out = grouped_mm(a, b, offs=offs)
    assert _op.selected_kernel(code, a, b, out) == _lib.GMM_KERNEL_GENERIC  # as given: not addressable by TMA
    assert _op._worth_relayout(code, a, b, out)
    a2, b2 = _op.tensor_core_layouts(code, a, b)
    assert torch.equal(a2, a) and torch.equal(b2, b)
    assert _op.selected_kernel(code, a2, b2, out) in _lib.TCGEN05_KINDS
    ref, defined = grouped_mm_oracle(a, b, offs)
    if form == "2d2d_rowmajor_a":
        for gi, (s0, e0) in enumerate(group_bounds(offs.cpu(), a.size(1))):
            assert max_violation(out[gi], ref[gi], defined[gi], atol_for(e0 - s0, 1.0, 1.0)) <= 1.0
    else:
        assert max_violation(out, ref, defined, atol_for(a.size(-1), 1.0, 1.0)) <= 1.0
    with force_generic():  # the generic kernel on the untouched operands agrees
        slow = grouped_mm(a, b, offs=offs)
    torch.testing.assert_close(out.float(), slow.float(), atol=2e-2 * 32, rtol=2e-2)


# ----------------------------------------------------------------------------- bounded waits


def test_a_wait_that_runs_out_reports_a_status_and_leaves_the_gpu_usable(built_library):
    """A wait on a barrier nothing completes gives up after its budget, the kernel returns, the
    status word says so, and the next call works (no trap, no hang, context intact)."""
    lib = _lib.load()
    ws = torch.zeros(64, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.gmm_selftest_wait_timeout(ws.data_ptr(), stream, 2_000_000) == 0  # ~1 ms of waiting
    raw = ctypes.c_int32(0)
    rc = lib.gmm_check_status(ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(stream), ctypes.byref(raw))
    assert rc == _lib.GMM_ERR_DEVICE_WAIT and raw.value == 0x7E57
    assert b"bounded wait" in lib.gmm_error_string(rc)
    # the word was cleared by the check, and the device still computes
    assert lib.gmm_check_status(ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(stream), ctypes.byref(raw)) == 0
    wl = make_workload("readme", DEV, seed=0)
    _assert_parity(wl.mat_a, wl.mat_b, wl.offs, 1.0, 1.0)
    assert lib.gmm_selftest_wait_timeout(ws.data_ptr(), stream, 0) == -1


# ----------------------------------------------------------------------------- randomised shapes


@pytest.mark.parametrize("seed", range(24))
def test_random_shapes_layouts_and_dtypes(seed, tile_kernel):
    """Random group patterns, aligned sizes, operand layouts, dtypes and output dtypes, all four forms."""
    import random

    rng = random.Random(seed)
    g = torch.Generator(device=DEV).manual_seed(1000 + seed)
    dtype = rng.choice([torch.bfloat16, torch.float16])
    out_dtype = rng.choice([None, torch.float32])
    n_groups = rng.randint(1, 12)
    sizes = [rng.choice([0, 1, 8, 56, 127, 128, 129, 257, 400]) for _ in range(n_groups)]
    dim = lambda: 8 * rng.randint(1, 70)  # noqa: E731  (multiples of 8: 16-byte aligned rows)

    def mat(rows, cols, col_major, batch=None):
        shape = (rows, cols) if batch is None else (batch, rows, cols)
        if col_major:
            shape = shape[:-2] + (cols, rows)
            return torch.randn(shape, device=DEV, generator=g).to(dtype).transpose(-2, -1)
        return torch.randn(shape, device=DEV, generator=g).to(dtype)

    form = ["2d3d", "3d3d", "2d2d", "3d2d"][seed % 4]
    if form == "2d3d":
        k, n = dim(), dim()
        a, b, offs = mat(sum(sizes) + rng.choice([0, 5]), k, False), mat(k, n, rng.random() < 0.5, n_groups), _offs(sizes)
    elif form == "3d3d":
        m, k, n = dim(), dim(), dim()
        a, b, offs = mat(m, k, rng.random() < 0.5, n_groups), mat(k, n, rng.random() < 0.5, n_groups), None
    elif form == "2d2d":
        m, n = dim(), dim()
        if sum(sizes) == 0:
            sizes[0] = 8
        a, b, offs = mat(m, sum(sizes), True), mat(sum(sizes), n, False), _offs(sizes)
    else:
        m, k = dim(), dim()
        if sum(sizes) == 0:
            sizes[0] = 8
        a, b, offs = mat(m, k, rng.random() < 0.5, n_groups), mat(k, sum(sizes), True), _offs(sizes)
    if a.numel() == 0:
        pytest.skip("degenerate draw")
    _assert_parity(a, b, offs, 1.0, 1.0, out_dtype, _lib.GMM_KERNEL_TCGEN05)
