"""Builds liblkc.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m lokinfer_b200.build [--force] [--verbose] [--prof]

--prof compiles the tensor-core conv with its role-level cycle counters (-DLKC_TC_PROF=1, lkc_conv1d_tc_profile);
the default (product) build leaves them out.

One object per .cu (compiled in parallel, rebuilt when the source or a header is newer), linked into
lokinfer_b200/liblkc.so with the CUDA runtime linked statically, so the library loads on a machine without a
GPU (the compute calls then fail with an error, they never fall back to a CPU path)."""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent
LIB = PKG / "liblkc.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
         f"-I{ROOT / 'include'}", f"-I{CSRC}"]


def _sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, obj: Path, verbose: bool, prof: bool = False):
    cmd = [NVCC, *ARCH, *FLAGS, *(["-DLKC_TC_PROF=1"] if prof else []), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return src.name, r.stderr


def build(force: bool = False, verbose: bool = False, prof: bool = False) -> Path:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    jobs = []
    for src in _sources():
        obj = objdir / (src.stem + ".o")
        if force or verbose or prof or _stale(obj, [src, *headers]):
            jobs.append((src, obj))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name, log in ex.map(lambda j: _compile(j[0], j[1], verbose, prof), jobs):
            if verbose and log:
                print(f"--- {name}\n{log}", file=sys.stderr)
    objs = [objdir / (s.stem + ".o") for s in _sources()]
    if force or jobs or _stale(LIB, objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, prof="--prof" in sys.argv))
