"""The drop-in claim, executed on a B200 with the unmodified reference installed under baseline/_ref
(baseline/install_reference.py; the folder travels with the tree but is not part of the history):

  * route A: the reference's own test file (tests/test_grouped_mm.py, 30 cases, forward and backward,
    all four shape forms) run unchanged against this repository's ``grouped_mm_bf16`` package;
  * route B: the reference's own ``api.py`` with its kernel imports (api.py:8-17) rebound to
    libgrouped_mm_b200.so through the ctypes stub printed in INTEGRATION.md, taken from that file verbatim.
"""

import importlib.util
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"


def _need(path: Path):
    if not path.exists():
        pytest.skip(f"{path.relative_to(ROOT)} is not present (run baseline/install_reference.py)")


def test_reference_test_file_passes_unchanged_against_this_package(built_library):
    test_file = REF / "tests" / "test_grouped_mm.py"
    _need(test_file)
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    # which package the name resolves to in that environment
    probe = subprocess.run([sys.executable, "-c", "import grouped_mm_bf16 as m; print(m.grouped_mm.__module__)"],
                           capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert probe.returncode == 0 and "grouped_mm_bf16_b200" in probe.stdout, probe.stdout + probe.stderr
    # --noconftest: the reference's conftest.py only prepends its own checkout to sys.path
    run = subprocess.run([sys.executable, "-m", "pytest", str(test_file), "--noconftest", "-q", "-p", "no:cacheprovider",
                          "-x"], capture_output=True, text=True, env=env, cwd=ROOT, timeout=1500)
    tail = run.stdout[-1500:] + run.stderr[-500:]
    assert run.returncode == 0, tail
    m = re.search(r"(\d+) passed", run.stdout)
    assert m and int(m.group(1)) == 30 and "skipped" not in run.stdout.splitlines()[-1], tail


def _integration_stub() -> str:
    text = (ROOT / "INTEGRATION.md").read_text()
    m = re.search(r"```python\n(# grouped_mm_bf16/kernels_b200\.py.*?)```", text, re.S)
    assert m, "INTEGRATION.md no longer holds the kernels_b200.py stub"
    return m.group(1)


def test_reference_api_runs_on_the_library_through_the_documented_stub(built_library, tmp_path):
    pkg = REF / "grouped_mm_bf16"
    _need(pkg / "api.py")
    dst = tmp_path / "grouped_mm_bf16_routeb"
    shutil.copytree(pkg, dst, ignore=shutil.ignore_patterns("__pycache__"))
    stub = _integration_stub().replace("/path/to/grouped_mm_bf16_b200/lib/libgrouped_mm_b200.so", str(built_library))
    (dst / "kernels_b200.py").write_text(stub)
    api = (dst / "api.py").read_text()
    block = re.search(r"from \.kernels import \((.*?)\)\n", api, re.S)
    assert block, "the reference's api.py import block has moved"
    api = api.replace(block.group(0),
                      "from .kernels_b200 import grouped_mm_2d2d, grouped_mm_2d3d, grouped_mm_3d2d, grouped_mm_3d3d\n"
                      "from grouped_mm_bf16_b200.kernels import (grouped_mm_2d2d_backward, grouped_mm_2d3d_backward,\n"
                      "                                          grouped_mm_3d2d_backward, grouped_mm_3d3d_backward)\n")
    (dst / "api.py").write_text(api)
    spec = importlib.util.spec_from_file_location("grouped_mm_bf16_routeb", dst / "__init__.py",
                                                  submodule_search_locations=[str(dst)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["grouped_mm_bf16_routeb"] = mod
    try:
        spec.loader.exec_module(mod)
        assert mod.grouped_mm.__module__ == "grouped_mm_bf16_routeb.api"
        dev = torch.device("cuda")
        gen = torch.Generator(device=dev).manual_seed(0)
        # the README example
        sizes = [0, 7, 1, 13, 0, 11]
        offs = torch.tensor(sizes, device=dev).cumsum(0).to(torch.int32)
        a = torch.randn((32, 64), device=dev, generator=gen).bfloat16().requires_grad_(True)
        b = torch.randn((6, 64, 48), device=dev, generator=gen).bfloat16().requires_grad_(True)
        out = mod.grouped_mm(a, b, offs=offs)
        rows = torch.arange(32, device=dev)
        gid = torch.searchsorted(offs, rows.to(torch.int32), right=True)
        ref = torch.bmm(a.float().unsqueeze(1), b.float()[gid]).squeeze(1)
        torch.testing.assert_close(out.float(), ref, atol=2e-2 * 8, rtol=2e-2)
        # one backward pass through the reference's autograd function
        w = torch.randn_like(out)
        ga, gb = torch.autograd.grad(out, [a, b], w)
        ra, rb = torch.autograd.grad(ref, [a, b], w.float())
        torch.testing.assert_close(ga.float(), ra.float(), atol=0.5, rtol=6e-2)
        torch.testing.assert_close(gb.float(), rb.float(), atol=0.6, rtol=1e-1)
        # the K-ragged form (per-group tensor maps) through the same api.py
        k_sizes = [8, 0, 16, 40]
        k_offs = torch.tensor(k_sizes, device=dev).cumsum(0).to(torch.int32)
        a2 = torch.randn((64, 24), device=dev, generator=gen).bfloat16().t()   # column-major [24, 64]
        b2 = torch.randn((64, 40), device=dev, generator=gen).bfloat16()
        out2 = mod.grouped_mm(a2, b2, offs=k_offs)
        start = 0
        for g, sz in enumerate(k_sizes):
            want = a2[:, start:start + sz].float() @ b2[start:start + sz].float()
            torch.testing.assert_close(out2[g].float(), want, atol=2e-2 * 8, rtol=2e-2)
            start += sz
        torch.cuda.synchronize()
    finally:
        for name in [n for n in sys.modules if n.startswith("grouped_mm_bf16_routeb")]:
            del sys.modules[name]
