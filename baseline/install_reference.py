"""Install the UNMODIFIED reference (flash-attention-triton) under baseline/_ref, for the two things
that run it on a GPU box: baseline/reference_triton_bench.py (its Triton kernels, timed) and
tests/test_gpu_reference_own_tests.py (its own test file, run against this package).

    python baseline/install_reference.py /path/to/flash-attention-triton

baseline/_ref is git-ignored: nothing of the reference enters this repository's history.  The
package is installed offline with pip from a copy of the source tree (pip wants to write into it),
and the reference's test file is copied, byte for byte, to baseline/_ref/reference_tests/.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
TARGET = ROOT / "baseline" / "_ref"
TEST_FILE = "tests/test_flash_attention_2.py"


def install(source: Path) -> None:
    TARGET.mkdir(parents=True, exist_ok=True)
    if not (TARGET / "flash_attention_triton").is_dir():
        with tempfile.TemporaryDirectory() as tmp:
            copy = Path(tmp) / "reference"
            shutil.copytree(source, copy)
            subprocess.run(
                [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                 "--find-links", "/opt/wheelhouse", "--target", str(TARGET), str(copy)],
                check=True)
    tests = TARGET / "reference_tests"
    tests.mkdir(exist_ok=True)
    shutil.copyfile(source / TEST_FILE, tests / Path(TEST_FILE).name)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    install(Path(sys.argv[1]))
    print(f"reference installed under {TARGET}")
