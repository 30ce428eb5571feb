"""Installs the unmodified reference package under baseline/_ref (git-ignored; it travels to the GPU
box with a snapshot of the tree) and puts the reference's own test file beside it.

    python baseline/install_reference.py /path/to/reference/checkout

The install is the offline pip command (pure Python, so --no-deps suffices); the test file is copied
verbatim to baseline/_ref/tests/ so that it can be run, unchanged, against this repository's
`grouped_mm_bf16` package (tests/test_reference_drop_in.py) and against the reference itself.
Nothing under baseline/_ref is part of the product or of the history.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    src = Path(sys.argv[1]).resolve()
    if not (src / "grouped_mm_bf16" / "api.py").exists():
        raise SystemExit(f"{src} is not a checkout of the reference")
    with tempfile.TemporaryDirectory() as tmp:
        work = Path(tmp) / "reference"
        shutil.copytree(src, work, ignore=shutil.ignore_patterns(".git", "__pycache__"))  # pip builds in the tree
        subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                        "--upgrade", "--target", str(TARGET), str(work)], check=True)
    tests = TARGET / "tests"
    tests.mkdir(exist_ok=True)
    shutil.copy2(src / "tests" / "test_grouped_mm.py", tests / "test_grouped_mm.py")
    print(f"installed {src} into {TARGET}")


if __name__ == "__main__":
    main()
