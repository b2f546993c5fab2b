"""In-tree build of ``libexl3b200.so`` (hand-written CUDA for sm_100a + the C ABI).

``python -m ponyexl3_b200.build`` compiles every ``csrc/*.cu`` with nvcc and links
them into ``ponyexl3_b200/lib/libexl3b200.so``.  nvcc cross-compiles, so this runs
on a machine without a GPU.  The build is incremental on source mtimes.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "build"
LIB = LIBDIR / "libexl3b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: libexl3b200.so cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _deps_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "exl3_b200.h"]
    return max(p.stat().st_mtime for p in hdrs)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False,
          profile: bool = False) -> Path:
    """Compile what changed and link; returns the library path.

    ``profile=True`` builds a second library, ``lib/libexl3b200_prof.so``, with -DEXL3_PROFILE:
    the streamed GEMV then records wall-clock stamps per CTA (``ponyexl3_b200.profiling``).  The
    product library is never built with that flag."""
    LIBDIR.mkdir(exist_ok=True)
    objdir = OBJDIR / "prof" if profile else OBJDIR
    objdir.mkdir(exist_ok=True, parents=True)
    lib = LIBDIR / "libexl3b200_prof.so" if profile else LIB
    nvcc = _nvcc()
    hdr_t = _deps_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_t):
            cmd = [nvcc, *NVCC_FLAGS, *(["-DEXL3_PROFILE"] if profile else []), "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd: list[str]) -> None:
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if ptxas_info and r.stderr:
            (objdir / (Path(cmd[-3]).stem + ".ptxas.txt")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(run, jobs))
    if jobs or not lib.exists():
        run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-lcudart"])
    return lib


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv,
              profile="--profile" in sys.argv)
    print(p)
