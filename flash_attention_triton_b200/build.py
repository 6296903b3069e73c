"""In-tree nvcc build of the sm_100a shared library.

``python -m flash_attention_triton_b200.build`` compiles every ``csrc/*.cu`` for
``compute_100a/sm_100a`` and links ``libfa2_b200.so`` next to this file.  nvcc
cross-compiles without a GPU, so the build can run on a CPU-only machine and the
resulting ``.so`` be carried to the B200 host.  Objects are rebuilt only when a source or
header is newer than the object.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libfa2_b200.so"

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the sm_100a library cannot be built")


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(src: Path, verbose: bool) -> Path:
    obj = BUILD_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _newest_header_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (BUILD_DIR / (src.stem + ".ptxas.log")).write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stderr[-4000:]}")
    if verbose:
        print(f"[build] compiled {src.name}")
    return obj


def build(verbose: bool = True, force: bool = False) -> Path:
    """Compile and link the library; returns the path of the ``.so``."""
    BUILD_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if force:
        for o in BUILD_DIR.glob("*.o"):
            o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest_obj:
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart_static",
               "-lpthread", "-ldl", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
        if verbose:
            print(f"[build] linked {LIB_PATH.name}")
    return LIB_PATH


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the last compile of each file."""
    out = []
    for log in sorted(BUILD_DIR.glob("*.ptxas.log")):
        out.append(f"== {log.stem}\n{log.read_text()}")
    return "\n".join(out)


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
    if "--report" in sys.argv:
        print(ptxas_report())
