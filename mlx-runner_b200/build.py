"""Builds libmlxq.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python mlx-runner_b200/build.py [--force] [--verbose]

Objects go to ``mlx-runner_b200/build/`` and the library to ``mlx-runner_b200/lib/libmlxq.so``; both are
kept out of version control.  Translation units are compiled in parallel; a unit is rebuilt when it or
any header in ``csrc/`` or ``include/`` is newer than its object.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libmlxq.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
                 "--expt-relaxed-constexpr", "-I", os.path.join(ROOT, "include")]

# (source, object name, extra flags)
UNITS = [("qmv_inst.cu", f"qmv_b{b}.o", [f"-DMLXQ_BITS={b}"]) for b in (2, 3, 4, 5, 6, 8)] + [
    ("aux_kernels.cu", "aux_kernels.o", []),
    ("dense.cu", "dense.o", []),
    ("qmv_mma.cu", "qmv_mma.o", []),
    ("qmv_pipe.cu", "qmv_pipe.o", []),
    ("qmv_tok.cu", "qmv_tok.o", []),
    ("qgemm_sm100.cu", "qgemm_sm100.o", []),
    ("api.cu", "api.o", []),
    ("comm.cu", "comm.o", []),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    hs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h")) + [os.path.abspath(__file__)]
    return max(os.path.getmtime(h) for h in hs)


def _compile(nvcc: str, src: str, obj: str, extra: list[str], verbose: bool) -> str:
    cmd = [nvcc] + COMMON + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return r.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile what is out of date and link the shared library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    hdr = _newest_header()
    units = [(s, o, e) for (s, o, e) in UNITS if os.path.exists(os.path.join(CSRC, s))]
    todo = []
    for src, obj_name, extra in units:
        obj = os.path.join(OBJ, obj_name)
        stamp = max(os.path.getmtime(os.path.join(CSRC, src)), hdr)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < stamp:
            todo.append((src, obj, extra))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            futs = [ex.submit(_compile, nvcc, s, o, e, verbose) for (s, o, e) in todo]
            for f in futs:
                out = f.result()
                if out:
                    print(out)
    objs = [os.path.join(OBJ, o) for (_, o, _) in units]
    if todo or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [nvcc] + ARCH + ["-shared", "-o", LIB] + objs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
