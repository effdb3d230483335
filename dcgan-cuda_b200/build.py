"""Builds libdcgan_b200.so from csrc/*.cu with nvcc for sm_100a, in-tree.

One nvcc invocation per translation unit (run in parallel), objects cached by
modification time under csrc/build/, then one link step.  No GPU is needed:
nvcc cross-compiles.

Run: ``python dcgan-cuda_b200/build.py [--force] [--verbose]``

``DCG_BUILD_FLAGS`` (environment) adds nvcc flags, e.g. ``-DDCG_TC_TRACING`` for the build with the
convolution kernel's timeline and loads-only / MMAs-only switches (``DCG_TC_DEBUG``); use --force with it.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libdcgan_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
          "-I", os.path.join(ROOT, "include"), "-I", CSRC] + os.environ.get("DCG_BUILD_FLAGS", "").split()


def _deps():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))


def _compile(src, force, verbose):
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    newest = max(os.path.getmtime(p) for p in [src] + _deps())
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj
    cmd = [NVCC] + ARCH + CFLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed on " + src)
    return obj


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        # The CUDA runtime is linked statically and the driver API (tensor-map
        # encoding) is resolved at run time through cudaGetDriverEntryPoint, so the
        # library loads on a machine without a driver (symbol checks on CPU boxes).
        cmd = [NVCC] + ARCH + ["-shared", "-o", LIB] + objs
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
