"""Builds `libjoshua_b200.so` in-tree with nvcc for sm_100a.

    python -m joshua_b200.build [--force] [--verbose] [--ptxas] [--profiling]

Every `csrc/*.cu` is compiled to an object file (in parallel) and linked into
one shared library beside this file.  The library has no dependency beyond the
CUDA runtime (linked statically); in particular it does not link PyTorch.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libjoshua_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _deps_mtime() -> float:
    files = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [HERE.parent / "include" / "joshua_b200.h"]
    return max(f.stat().st_mtime for f in files)


def _compile(src: Path, verbose: bool, ptxas_info: bool, profiling: bool = False) -> Path:
    obj = OBJ / (src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, _deps_mtime()):
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if ptxas_info:
        cmd[1:1] = ["-Xptxas", "-v"]
    if profiling:
        cmd[1:1] = ["-DJQ_PROFILING"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose or ptxas_info:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, profiling: bool = False) -> Path:
    """`profiling` adds -DJQ_PROFILING: the trace entry points of include/joshua_b200_profiling.h and the
    measurement switches read from the environment.  It always recompiles, and the next plain build does too."""
    OBJ.mkdir(exist_ok=True)
    marker = OBJ / ".profiling"
    if profiling or marker.exists():
        force = True
    if profiling:
        marker.write_text("1")
    elif marker.exists():
        marker.unlink()
    if force:
        for f in OBJ.glob("*.o"):
            f.unlink()
    sources = sorted(CSRC.glob("*.cu"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, ptxas_info, profiling), sources))
    if force or not LIB.exists() or LIB.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fPIC",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                profiling="--profiling" in sys.argv))
