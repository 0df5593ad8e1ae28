"""Compile the CUDA sources of this package for sm_100a into window_matmul/libwmm_b200.so (in-tree).

    python pytorch-window-matmul_b200/build.py [--force] [-v]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically and has no other
dependency (no torch, no Python): it is the C ABI declared in include/wmm_b200.h.
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "window_matmul", "libwmm_b200.so")
SOURCES = ["wmm_api.cu", "wmm_generic.cu", "wmm_tc.cu", "wmm_small.cu", "wmm_softmax.cu", "wmm_halo.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _deps():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(HERE, "..", "include", "wmm_b200.h"))
    return hdrs


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force=False, verbose=False, defines=(), out=None):
    """`defines` (e.g. ["WMM_TRACE"]) build a variant of the library: objects go to their own directory and `out` names
    the shared object, so the normal library is left alone."""
    obj_dir = OBJ + ("_" + "_".join(defines) if defines else "")
    lib = out or LIB
    if defines and out is None:
        raise ValueError("a variant build needs its own output path")
    os.makedirs(obj_dir, exist_ok=True)
    deps = _deps()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src[:-3] + ".o")
        if force or _stale(o, [s] + deps):
            cmd = [NVCC] + FLAGS + ["-D" + d for d in defines] + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed on " + cmd[-3])

    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(run, jobs))
    objs = [os.path.join(obj_dir, s[:-3] + ".o") for s in SOURCES]
    if force or jobs or _stale(lib, objs):
        cmd = [NVCC, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        run(cmd)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-D", "--define", action="append", default=[], help="preprocessor define for a variant build (with --out)")
    ap.add_argument("--out", default=None, help="path of the shared object of a variant build")
    a = ap.parse_args()
    print(build(a.force, a.verbose, tuple(a.define), a.out))
