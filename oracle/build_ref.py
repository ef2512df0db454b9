#!/usr/bin/env python3
"""Compile the upstream CLUSTEN CUDA extension, unmodified, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY.  The three extension modules this recipe produces
(`clustenqk_cuda`, `clustenav_cuda`, `clustenwf_cuda`) are the reference's own
kernels (clusten/src/*.cu, *.cpp of apple/ml-autofocusformer) compiled for
sm_100a straight from the read-only checkout.  They are used as a checker for
the oracle and for the parity tests, and as a speed bar in the benchmark; the
product never loads them.

No source file is copied: nvcc / g++ read the sources where they lie and only
object files and the three shared objects are written (all below oracle/_ref/,
which is git-ignored).  The upstream setup.py is not run; the commands below
are what it would amount to (three CUDAExtension modules, no extra flags:
clusten/src/setup.py:15-28) plus an explicit sm_100a target.

Usage:  python oracle/build_ref.py [--src /path/to/reference/clusten/src] [-j N]
When the source directory does not exist the script exits 0 without doing
anything, so a prebuilt oracle/_ref/ is used as is.
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

# where the reference checkout keeps the extension sources (override with CLUSTEN_REFERENCE_SRC)
DEFAULT_SRC = os.environ.get("CLUSTEN_REFERENCE_SRC", "/root/reference/clusten/src")

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = ("clustenqk_cuda", "clustenav_cuda", "clustenwf_cuda")


def _run(cmd):
    print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=DEFAULT_SRC)
    ap.add_argument("-j", type=int, default=3)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    if not os.path.isdir(args.src):
        print(f"build_ref: {args.src} not present; keeping whatever is in {OUT}")
        return 0

    import torch  # noqa: F401  (only for its headers and libraries)
    from torch.utils.cpp_extension import include_paths, library_paths

    os.makedirs(OUT, exist_ok=True)
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    incs = []
    for p in include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        incs += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-std=c++17", "-O3"]

    jobs = []
    for mod in MODULES:
        so = os.path.join(OUT, mod + suffix)
        if os.path.exists(so) and not args.force:
            continue
        cu, cpp = os.path.join(args.src, mod + "_kernel.cu"), os.path.join(args.src, mod + ".cpp")
        o_cu, o_cpp = os.path.join(OUT, mod + "_kernel.o"), os.path.join(OUT, mod + ".o")
        defs = [f"-DTORCH_EXTENSION_NAME={mod}"]
        jobs.append((mod, so, [
            ["nvcc", "-c", cu, "-o", o_cu, "-gencode", "arch=compute_100a,code=sm_100a",
             "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
             "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
             "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__"] + common + defs + incs,
            ["g++", "-c", cpp, "-o", o_cpp, "-fPIC"] + common + defs + incs,
            ["g++", "-shared", o_cu, o_cpp, "-o", so]
            + [f"-L{p}" for p in library_paths("cuda")]
            + [f"-Wl,-rpath,{p}" for p in library_paths("cuda")]
            + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"],
        ]))

    def build(job):
        mod, so, cmds = job
        for c in cmds:
            _run(c)
        for f in (os.path.join(OUT, mod + "_kernel.o"), os.path.join(OUT, mod + ".o")):
            if os.path.exists(f):
                os.remove(f)
        return so

    with ThreadPoolExecutor(max_workers=max(1, args.j)) as ex:
        for so in ex.map(build, jobs):
            print("built", so, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
