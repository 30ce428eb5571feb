"""The CPU oracle against the golden fixtures and against the independent plain-C restatement."""

import math

import pytest
import torch

from oracle import c_oracle
from oracle.grouped_mm_oracle import atol_for, group_bounds, grouped_mm_oracle, kragged_atol, max_violation


def test_golden_fixture_has_both_sources(golden_cases):
    sources = {c["source"] for c in golden_cases}
    assert sources == {"reference-interpreter", "torch-cpu"}
    assert {c["form"] for c in golden_cases} == {"2d3d", "3d3d", "2d2d", "3d2d"}


def test_oracle_matches_reference_interpreter_fp32(golden_cases):
    # fp32 inputs through the reference's own kernels: only summation order differs.
    for c in (c for c in golden_cases if c["source"] == "reference-interpreter"):
        ref, defined = grouped_mm_oracle(c["a"], c["b"], c["offs"])
        torch.testing.assert_close(ref[defined], c["out"][defined], atol=3e-5, rtol=1e-5)
        assert float(c["out"][~defined].abs().sum()) == 0.0  # untouched elements stayed zero


def test_oracle_matches_torch_cpu_bf16(golden_cases):
    # bf16 output of torch's CPU grouped_mm: the oracle's fp32 result rounds to it within 1 ulp.
    for c in (c for c in golden_cases if c["source"] == "torch-cpu"):
        ref, defined = grouped_mm_oracle(c["a"], c["b"], c["offs"])
        k = c["a"].size(-1) if c["form"] != "2d2d" else c["a"].size(-1)
        assert max_violation(c["out"], ref, defined, atol_for(k, 1.0, 1.0)) <= 1.0
        torch.testing.assert_close(c["out"].float(), ref, atol=1e-3, rtol=2 ** -7)


def test_c_oracle_agrees_with_python_oracle(golden_cases):
    for c in golden_cases:
        ref, _ = grouped_mm_oracle(c["a"], c["b"], c["offs"])
        torch.testing.assert_close(c_oracle.grouped_mm_c(c["a"], c["b"], c["offs"]), ref, atol=3e-5, rtol=1e-5)


def test_group_bounds_clamps_and_handles_empty_groups():
    assert group_bounds(torch.tensor([0, 7, 8, 21, 21, 32]), 32) == [(0, 0), (0, 7), (7, 8), (8, 21), (21, 21), (21, 32)]
    assert group_bounds(torch.tensor([5, 50]), 32) == [(0, 5), (5, 32)]


def test_2d2d_empty_group_is_exact_zero():
    a, b = torch.randn(4, 16).bfloat16(), torch.randn(16, 8).bfloat16()
    offs = torch.tensor([8, 8, 16], dtype=torch.int32)
    ref, defined = grouped_mm_oracle(a, b, offs)
    assert bool(defined.all()) and float(ref[1].abs().max()) == 0.0
    assert kragged_atol(offs, 16, 1.0, 1.0).tolist() == pytest.approx([atol_for(8, 1, 1), 0.0, atol_for(8, 1, 1)])


def test_tolerance_rule():
    assert atol_for(4096, 1.0, 0.02) == pytest.approx(1e-2 * 64 * 0.02)
    ref = torch.tensor([1.0, -2.0])
    ok = torch.ones(2, dtype=torch.bool)
    assert max_violation(ref + 0.5 * (0.1 + 8e-3 * ref.abs()), ref, ok, 0.1) == pytest.approx(0.5, rel=1e-4)
    assert math.isinf(max_violation(torch.tensor([float("nan"), 0.0]), ref, ok, 0.1))
