"""Builds the reference project IN PLACE against this repository's GPU backend.

The reference's own sources under <reference>/src/{api,cpu,memory,ops,runtime,utils} and
src/datasets/{mnist,celeba}.cu are compiled where they lie (nothing is copied; its CMake build is
not used), its src/gpu/* and src/datasets/jpg.cu are left out, and three files of this directory
take their place:

    b200_backend.cu   gpu::kernels_list / gpu::run on top of libdcgan_b200.so's C ABI
    tocha/tensor.hh   stand-in for the reference's un-vendored tensor-archive submodule
    jpg_headless.cu   img::jpg_save as PPM, no libjpeg

Objects and binaries go to <this directory>/_ref_build/ (git-ignored).  The reference's programs -
tests/test_*.cu, examples/nn_mnist.cu, dcgan/main.cu - are linked UNCHANGED; RT_MODE=CPU / MCPU run
the reference's own CPU code, RT_MODE=GPU runs this repository's kernels.

    python dcgan-cuda_b200/shim/build_reference.py [--reference DIR] [--programs a b ...] [--force]
"""
import argparse
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT = os.path.join(HERE, "_ref_build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -ffp-contract=off keeps the IEEE operation order of the reference's -O0 build in its CPU kernels
# (no fused multiply-add), so RT_MODE=CPU of these binaries is the same arithmetic as the oracle;
# -mavx2 -mfma only enable the intrinsics src/cpu/simd_kernels.cu names explicitly
CFLAGS = ["-O2", "-std=c++14", "-w", "-Xcompiler", "-fPIC,-ffp-contract=off,-mavx2,-mfma,-pthread"]

SRC_DIRS = ("api", "cpu", "memory", "ops", "runtime", "utils")
DATASET_SRCS = ("mnist.cu", "celeba.cu")

# programs of the reference that the parity tests run; name -> source path inside the reference
DEFAULT_PROGRAMS = {
    "test_conv2d": "tests/test_conv2d.cu",
    "test_conv2d_padding": "tests/test_conv2d_padding.cu",
    "test_conv2d_grad": "tests/test_conv2d_grad.cu",
    "test_conv2d_padding_grad": "tests/test_conv2d_padding_grad.cu",
    "test_conv2d_transpose": "tests/test_conv2d_transpose.cu",
    "test_conv2d_transpose_grad": "tests/test_conv2d_transpose_grad.cu",
    "test_conv2d_bias_add": "tests/test_conv2d_bias_add.cu",
    "test_conv2d_bias_add_grad": "tests/test_conv2d_bias_add_grad.cu",
    "test_adam_update": "tests/test_adam_update.cu",
    "test_moment_update": "tests/test_moment_update.cu",
    "test_moment_update2": "tests/test_moment_update2.cu",
    "test_sigmoid_cross_entropy": "tests/test_sigmoid_cross_entropy.cu",
    "test_sigmoid_cross_entropy_grad": "tests/test_sigmoid_cross_entropy_grad.cu",
    "test_leaky_relu_grad": "tests/test_leaky_relu_grad.cu",
    "test_tanh_grad": "tests/test_tanh_grad.cu",
    "test_relu_grad": "tests/test_relu_grad.cu",
    "test_reshape": "tests/test_reshape.cu",
    "test_argmax": "tests/test_argmax.cu",
    "test_mat_mul_add": "tests/test_mat_mul_add.cu",
    "test_softmax_cross_entropy_grad": "tests/test_softmax_cross_entropy_grad.cu",
    "test_conv_d1": "tests/test_conv_d1.cu",
    "test_conv_dx_d1": "tests/test_conv_dx_d1.cu",
    "test_conv_dk_d1": "tests/test_conv_dk_d1.cu",
    "test_conv_g2": "tests/test_conv_g2.cu",
    "test_dcgan_generator": "tests/test_dcgan_generator.cu",
    "nn_mnist": "examples/nn_mnist.cu",
    "dcgan": "dcgan/main.cu",
    # programs of this directory; the driver is written against the reference's public API (runtime batch size, seeded)
    "dcgan_graph_driver": os.path.join(HERE, "dcgan_graph_driver.cu"),
    "archive_tool": os.path.join(HERE, "archive_tool.cu"),
}


def default_reference():
    """The reference checkout: DCGAN_REFERENCE_DIR, else a directory `reference` next to this repository."""
    repo = os.path.dirname(os.path.dirname(HERE))
    return os.environ.get("DCGAN_REFERENCE_DIR") or os.path.join(os.path.dirname(repo), "reference")


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s%s" % (" ".join(cmd), res.stdout, res.stderr))


def _compile(src, obj, includes, force):
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
        return obj
    os.makedirs(os.path.dirname(obj), exist_ok=True)
    _run([NVCC] + ARCH + CFLAGS + includes + ["-c", src, "-o", obj])
    return obj


def build(reference=None, programs=None, force=False, jobs=None):
    """Compiles the host library and the requested programs; returns {program: path}.
    Returns {} when the reference tree is not present (nothing to build against)."""
    reference = reference or default_reference()
    if not os.path.isdir(os.path.join(reference, "src", "ops")):
        return {}
    lib = os.path.join(PKG, "libdcgan_b200.so")
    if not os.path.exists(lib):
        raise RuntimeError("build libdcgan_b200.so first (dcgan-cuda_b200/build.py)")
    src_root = os.path.join(reference, "src")
    includes = ["-I", HERE, "-I", src_root, "-I", os.path.join(ROOT, "include")]
    jobs_list = []
    for d in SRC_DIRS:
        for src in sorted(glob.glob(os.path.join(src_root, d, "*.cu"))):
            jobs_list.append((src, os.path.join(OUT, "obj", d, os.path.basename(src)[:-3] + ".o")))
    for name in DATASET_SRCS:
        jobs_list.append((os.path.join(src_root, "datasets", name), os.path.join(OUT, "obj", "datasets", name[:-3] + ".o")))
    for name in ("b200_backend.cu", "jpg_headless.cu"):
        jobs_list.append((os.path.join(HERE, name), os.path.join(OUT, "obj", "shim", name[:-3] + ".o")))
    programs = dict(DEFAULT_PROGRAMS) if programs is None else {p: DEFAULT_PROGRAMS.get(p, p) for p in programs}
    prog_objs = {}
    for name, rel in programs.items():
        src = rel if os.path.isabs(rel) else os.path.join(reference, rel)
        if not os.path.exists(src):
            raise RuntimeError("no such reference program: " + src)
        prog_objs[name] = os.path.join(OUT, "obj", "programs", name + ".o")
        jobs_list.append((src, prog_objs[name]))
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or min(16, os.cpu_count() or 4)) as ex:
        list(ex.map(lambda j: _compile(j[0], j[1], includes, force), jobs_list))
    host_objs = [o for s, o in jobs_list if o not in prog_objs.values()]
    archive = os.path.join(OUT, "libdcgan_ref_host.a")
    if force or not os.path.exists(archive) or any(os.path.getmtime(o) > os.path.getmtime(archive) for o in host_objs):
        if os.path.exists(archive):
            os.unlink(archive)
        _run(["ar", "rcs", archive] + host_objs)
    bindir = os.path.join(OUT, "bin")
    os.makedirs(bindir, exist_ok=True)
    out = {}
    for name, obj in prog_objs.items():
        exe = os.path.join(bindir, name)
        if force or not os.path.exists(exe) or os.path.getmtime(exe) < max(os.path.getmtime(obj), os.path.getmtime(archive),
                                                                         os.path.getmtime(lib)):
            # --whole-archive: the backend's table is filled by a static initialiser nobody references
            _run([NVCC] + ARCH + ["-o", exe, obj, "-Xlinker", "--whole-archive", archive, "-Xlinker", "--no-whole-archive",
                                  "-L", PKG, "-ldcgan_b200", "-Xlinker", "-rpath=$ORIGIN/../../..", "-lpthread"])
        out[name] = exe
    return out


def built_programs():
    """Programs already built (no compilation): {name: path}."""
    bindir = os.path.join(OUT, "bin")
    return {n: os.path.join(bindir, n) for n in DEFAULT_PROGRAMS if os.path.exists(os.path.join(bindir, n))}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--programs", nargs="*", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    res = build(a.reference, a.programs, a.force)
    if not res:
        sys.exit("reference tree not found (set DCGAN_REFERENCE_DIR or pass --reference)")
    for k, v in sorted(res.items()):
        print(k, v)
