"""In-tree build of the CUDA library (``cumm_b200/libcumm_b200.so``) for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

_HERE = Path(__file__).resolve().parent
CSRC = _HERE / "csrc"
OUT = _HERE / "libcumm_b200.so"
SOURCES = ["api.cu"]
HEADERS = sorted(p.name for p in CSRC.glob("*.cuh"))


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found")
    return cand


def needs_build() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [_HERE.parent / "include" / "cumm_b200.h"]
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared", "-o", str(OUT)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES]
    subprocess.run(cmd, check=True, cwd=str(CSRC))
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose=bool(os.environ.get("VERBOSE"))))
