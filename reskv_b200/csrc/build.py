"""Ahead-of-time build of libreskv_b200.so for sm_100a.

    python -m reskv_b200.csrc.build [--force] [--verbose]

One ``nvcc`` invocation per ``.cu`` file (object files under ``build/``), then a
shared link next to this file.  Nothing links against torch or Python: the
library is plain CUDA runtime code behind the C ABI of ``include/reskv_b200.h``.
nvcc cross-compiles, so no GPU is needed to build.  ``RESKV_NVCC_FLAGS`` (environment) adds compiler flags for
experiment builds, e.g. ``RESKV_NVCC_FLAGS="-DRESKV_MMA_CTAS_PER_SM=3" python -m reskv_b200.csrc.build --force``.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libreskv_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME", "") + "/bin/nvcc", "/usr/local/cuda/bin/nvcc", shutil.which("nvcc") or ""):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    headers = sorted(HERE.glob("*.cuh")) + [HERE.parent.parent / "include" / "reskv_b200.h"]
    # extra compiler flags for experiment builds (e.g. -DRESKV_MMA_CTAS_PER_SM=3); use together with --force
    extra = os.environ.get("RESKV_NVCC_FLAGS", "").split()
    jobs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *ARCH_FLAGS, *COMMON, *extra, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(run, jobs))
    objs = [objdir / (s.stem + ".o") for s in sources()]
    if force or jobs or _stale(LIB, objs):
        run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
