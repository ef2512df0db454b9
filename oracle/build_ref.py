#!/usr/bin/env python3
"""Compile the upstream CLUSTEN CUDA extension and byte-compile the upstream caller
modules, unmodified, into oracle/_ref/.

TEST AND MEASUREMENT INFRASTRUCTURE ONLY.  Two things are produced, all from the
read-only checkout of apple/ml-autofocusformer, nothing of it is copied as source:

  * the three extension modules `clustenqk_cuda`, `clustenav_cuda`, `clustenwf_cuda`:
    the reference's own kernels (clusten/src/*.cu, *.cpp) compiled for sm_100a.  They
    check the oracle and the parity tests and serve as a speed bar in the benchmark.
  * Python bytecode of the modules that CALL the operators: models/aff_transformer.py and
    models/point_utils.py (the AutoFocusFormer model, the caller of this repository's `clusten`
    package in the model-level benchmark) and clusten/clusten.py (the reference's autograd
    wrappers, so that the same model can also run on the reference's kernels).  They land in
    oracle/_ref/aff_model/models/ and oracle/_ref/ref_clusten/clusten/ as `.bytecode` files
    (the .pyc format under a name that file filters for Python caches leave alone) and are
    loaded as sourceless modules.  The upstream models/__init__.py is left out: it imports the
    training-side builder (models/__init__.py:8), which is not on the measured path.

nvcc / g++ / py_compile read the sources where they lie and only objects, shared
objects and bytecode are written (all below oracle/_ref/, which is git-ignored).  The
upstream setup.py is not run; the commands below are what it would amount to (three
CUDAExtension modules, no extra flags: clusten/src/setup.py:15-28) plus an explicit
sm_100a target.

Usage:  python oracle/build_ref.py [--root /path/to/ml-autofocusformer] [-j N] [--force]
The checkout is looked for at --root, else $CLUSTEN_REFERENCE_ROOT, else a directory
named `reference` beside this repository.  When it does not exist the script exits 0
without doing anything, so a prebuilt oracle/_ref/ is used as is.
"""
import argparse
import os
import py_compile
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = ("clustenqk_cuda", "clustenav_cuda", "clustenwf_cuda")
# (source inside the checkout, bytecode below oracle/_ref/)
BYTECODE = (
    ("models/aff_transformer.py", "aff_model/models/aff_transformer.bytecode"),
    ("models/point_utils.py", "aff_model/models/point_utils.bytecode"),
    ("clusten/clusten.py", "ref_clusten/clusten/clusten.bytecode"),
)


def reference_root(arg=None):
    """Where the checkout of apple/ml-autofocusformer is expected."""
    if arg:
        return arg
    env = os.environ.get("CLUSTEN_REFERENCE_ROOT")
    if env:
        return env
    return os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def byte_compile(root, force=False):
    """models/*.py and clusten/clusten.py of the checkout -> sourceless bytecode below oracle/_ref/."""
    for src_rel, dst_rel in BYTECODE:
        src, dst = os.path.join(root, src_rel), os.path.join(OUT, dst_rel)
        if not os.path.exists(src):
            continue
        if force or not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src):
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            py_compile.compile(src, cfile=dst, dfile=src_rel, doraise=True)
            print("byte-compiled", src_rel, "->", dst, flush=True)


def _run(cmd):
    print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", default=None, help="checkout of apple/ml-autofocusformer")
    ap.add_argument("-j", type=int, default=3)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    root = reference_root(args.root)
    args.src = os.path.join(root, "clusten", "src")
    if not os.path.isdir(args.src):
        print(f"build_ref: {args.src} not present; keeping whatever is in {OUT}")
        return 0
    os.makedirs(OUT, exist_ok=True)
    byte_compile(root, args.force)

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
