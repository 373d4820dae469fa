"""In-tree nvcc build of the sm_100a kernel library.

All kernels are plain ``extern "C"`` launchers over raw pointers and a stream, compiled
ahead of time with ``nvcc -gencode arch=compute_100a,code=sm_100a`` into one shared
object next to the sources and loaded with ``ctypes`` (the reference compiles its one
native kernel at run time through hipRTC, ``engine/fast/hipmega_rtc.py:78-215``; here
nothing is compiled while serving). The build is incremental: a source is recompiled
only when it or a header is newer than its object.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CUDA_DIR = Path(__file__).resolve().parent / "cuda"
LIB_NAME = "libb200serve_kernels.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources() -> list[Path]:
    return sorted(CUDA_DIR.glob("*.cu"))


def lib_path() -> Path:
    return CUDA_DIR / LIB_NAME


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``.cu`` under ``ops/cuda`` for sm_100a and link the shared library."""
    headers = sorted(CUDA_DIR.glob("*.cuh")) + sorted(CUDA_DIR.glob("*.h"))
    objs = []
    jobs = []
    for src in sources():
        obj = src.with_suffix(".o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            cmd = [NVCC, *ARCH_FLAGS, *COMMON, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed: {cmd[-3]}")
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        logs = list(pool.map(run, jobs))
    lib = lib_path()
    if jobs or _stale(lib, objs):
        cmd = [NVCC, *ARCH_FLAGS, "-shared", "-o", str(lib), *map(str, objs), "-lcudart"]
        run(cmd)
    if ptxas_info:
        for log in logs:
            sys.stdout.write(log)
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv))
