"""Build the CUDA library in-tree: python -m pragnosia_b200.build

One nvcc invocation per source, sm_100a only, then one link into pragnosia_b200/lib/libpragnosia_b200.so.
Sources are rebuilt only when they (or a header) are newer than their object file.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libpragnosia_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(src: Path, obj: Path, headers) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or any(h.stat().st_mtime > t for h in headers)


def build(verbose: bool = False, force: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h"))
    if not force and LIB.exists() and all(f.stat().st_mtime <= LIB.stat().st_mtime for f in sources() + headers):
        return LIB                                  # the prebuilt library is newer than every source: nothing to do
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    jobs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        if force or _stale(src, obj, headers):
            cmd = [NVCC, *FLAGS, *( ["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return src.name

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name in ex.map(run, jobs):
            print(f"  compiled {name}")
    objs = [str(objdir / (s.stem + ".o")) for s in sources()]
    if jobs or not LIB.exists():
        r = subprocess.run([NVCC, "-shared", "-o", str(LIB), *objs], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        print(f"  linked {LIB.relative_to(PKG.parent)}")
    return LIB


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
