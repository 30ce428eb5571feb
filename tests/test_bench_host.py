"""Host-side pieces of bench.py that need no GPU: the CPU baseline sampler, the peak table, the
clock sampler's empty summary, and the `--impl reference` arm's JSON line (on a reduced size)."""

import json
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_cpu_oracle_sample_counts_the_flops_it_did():
    sizes = [40, 0, 25, 60]
    a = torch.randn(sum(sizes), 32).bfloat16()
    b = torch.randn(4, 32, 48).bfloat16()
    flops, seconds, desc = bench.cpu_oracle_sample(a, b, sizes, budget_s=0.5, workload_rows=1000)
    rows = int(desc.split()[1])
    assert 3 <= rows <= sum(sizes) and flops == 2.0 * rows * 32 * 48 and seconds > 0
    assert "of 1000 rows" in desc and "3 groups" in desc  # the empty group is skipped


def test_peaks_have_a_fallback_and_clock_summary_is_well_formed():
    peaks = bench.read_peaks()
    assert peaks["source"] in ("measured", "fallback") and peaks["tflops"] > 1000 and peaks["hbm_gbs"] > 5000
    summary = bench.ClockSampler.__new__(bench.ClockSampler)
    summary.samples, summary.reasons, summary.max_mhz = [], set(), None
    assert summary.summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3",
                          "--dims-scale", "0.0625"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "impl", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0


def test_sampled_tolerance_check_passes_the_oracle_and_catches_a_wrong_tile():
    """bench.py's slab-sampled checker (used for the `all_configs` key) on CPU tensors: the oracle's own
    result is within tolerance, a result with one corrupted 32-row slab is not, and a non-zero entry in
    an empty K-ragged group is reported as infinitely wrong."""
    from grouped_mm_bf16_b200.workloads import make_workload
    from oracle.grouped_mm_oracle import grouped_mm_oracle

    wl = make_workload("mixtral", "cpu", seed=0, scale=1 / 64, dims_scale=1 / 32)
    ref, _ = grouped_mm_oracle(wl.mat_a, wl.mat_b, wl.offs)
    assert bench.sampled_within_tolerance(wl, ref.bfloat16(), max_rows=10 ** 6) <= 1.0
    bad = ref.clone()
    bad[64:96] += 1.0
    assert bench.sampled_within_tolerance(wl, bad.bfloat16(), max_rows=10 ** 6) > 1.0

    wg = make_workload("wgrad", "cpu", seed=0, scale=1 / 64, dims_scale=1 / 32)
    ref, _ = grouped_mm_oracle(wg.mat_a, wg.mat_b, wg.offs)
    assert bench.sampled_within_tolerance(wg, ref) <= 1.0
    empty = [g for g, s in enumerate(wg.sizes) if s == 0]
    if empty:
        ref[empty[0], 3, 3] = 1e-3
        assert bench.sampled_within_tolerance(wg, ref) == float("inf")

    bt = make_workload("batched", "cpu", seed=0, dims_scale=1 / 32)
    ref, _ = grouped_mm_oracle(bt.mat_a, bt.mat_b)
    assert bench.sampled_within_tolerance(bt, ref.bfloat16()) <= 1.0


def test_split_offsets_cut_every_group_into_consecutive_pieces():
    from grouped_mm_bf16_b200 import _op

    offs = torch.tensor([10, 10, 50, 120], dtype=torch.int32)  # the second group is empty, the last is clamped to 100
    pieces = _op._split_offsets(offs, 100, 4).tolist()
    assert pieces == [2, 5, 7, 10, 10, 10, 10, 10, 20, 30, 40, 50, 62, 75, 87, 100]
    assert pieces == sorted(pieces) and pieces[3::4] == [10, 10, 50, 100]
