"""Build the UNMODIFIED reference extension into oracle/_ref/ (test infrastructure, not product).

The reference's sources are compiled where they lie (csrc/window_matmul/window_matmul.cpp,
cpu/window_matmul_cpu.cpp and, with --cuda, cuda/window_matmul_cuda.cu); nothing is copied into this
repository.  Output: oracle/_ref/window_matmul_kernel.so, the reference's own pybind module
(csrc/window_matmul/window_matmul.cpp:100-106) exposing window_matmul_forward/backward and
unwindow_matmul_forward/backward.  The reference's build system (setup.py) is not run: it appends
`-arch all-major` when no GPU is visible, which takes ~25 minutes; this recipe compiles the same
sources with the same macros (-DWITH_PYTHON [-DWITH_CUDA], -O3, --expt-relaxed-constexpr) for sm_100.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may load the result.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "window_matmul_kernel"


def build(reference_root: str, with_cuda: bool = True, verbose: bool = False) -> str:
    src = os.path.join(reference_root, "csrc", "window_matmul")
    sources = [os.path.join(src, "window_matmul.cpp"), os.path.join(src, "cpu", "window_matmul_cpu.cpp")]
    cflags = ["-O3", "-Wno-sign-compare", "-DWITH_PYTHON"]
    cuda_flags = []
    if with_cuda:
        sources.append(os.path.join(src, "cuda", "window_matmul_cuda.cu"))
        cflags.append("-DWITH_CUDA")
        cuda_flags = ["-O3", "--expt-relaxed-constexpr", "-DWITH_PYTHON", "-DWITH_CUDA"]
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    target = os.path.join(OUT, NAME + ".so")
    if os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(s) for s in sources):
        marker = os.path.join(OUT, "WITH_CUDA")
        if (not with_cuda) or os.path.exists(marker):
            return target
    build_dir = os.path.join(OUT, "_build")
    os.makedirs(build_dir, exist_ok=True)
    from torch.utils.cpp_extension import load

    load(
        name=NAME,
        sources=sources,
        extra_include_paths=[src],
        extra_cflags=cflags,
        extra_cuda_cflags=cuda_flags,
        with_cuda=with_cuda,
        build_directory=build_dir,
        is_python_module=False,
        verbose=verbose,
    )
    shutil.copyfile(os.path.join(build_dir, NAME + ".so"), target)
    if with_cuda:
        open(os.path.join(OUT, "WITH_CUDA"), "w").write("sm_100\n")
    shutil.rmtree(build_dir, ignore_errors=True)
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    ap.add_argument("--reference", default=os.environ.get("WMM_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(here)), "reference")),
                    help="root of the reference's source tree (default: $WMM_REFERENCE_ROOT, else the directory `reference` beside this repository)")
    ap.add_argument("--cpu-only", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(a.reference):
        sys.exit("reference tree not found: " + a.reference)
    print(build(a.reference, with_cuda=not a.cpu_only, verbose=a.verbose))
