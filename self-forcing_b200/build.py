"""Build libsfmonarch.so (CUDA, sm_100a only) next to this file with nvcc.

    python self-forcing_b200/build.py [--force] [--verbose]

The library has no PyTorch or Python dependency: it is a plain C-ABI shared object
(see include/sfmonarch.h).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libsfmonarch.so"
SOURCES = ["layout.cu", "tmap.cu", "monarch_rstep.cu", "monarch_rstep_tc.cu", "monarch_lstep.cu", "monarch_lstep_tc.cu", "monarch_iter_tc.cu", "dense.cu",
           "monarch_bwd.cu", "monarch_bwd_tc.cu", "monarch_bwd_row_tc.cu", "probe_dsmem.cu", "selftest.cu", "api.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found")
    return cand


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "sfmonarch.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = nvcc_path()
    common = [nvcc, *ARCH, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = objdir / (src + ".o")
        objs.append(str(obj))
        procs.append((src, subprocess.Popen(common + ["-c", str(CSRC / src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = LIB.with_suffix(".so.tmp")
    subprocess.check_call([nvcc, *ARCH, "-shared", "-o", str(tmp), *objs, "-lcudart"])
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
