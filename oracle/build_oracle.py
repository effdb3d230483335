"""Build recipe for the CPU oracle libraries (test infrastructure only).

Two shared libraries come out of this script:

* ``oracle/liboracle.so``   - oracle/dcgan_oracle.c, the plain-C restatement of
  the reference's CPU arithmetic.  Always buildable (gcc only).
* ``oracle/_ref/libdcgan_ref_cpu.so`` - oracle/ref_shim.cc compiled against the
  reference's own header-only CPU math (src/cpu/ops.hh, ops.hxx) and its
  src/utils/xorshift.cu, used where they lie in the reference checkout.  Built
  only when a reference checkout is available (``DCGAN_REFERENCE_DIR`` or the
  default location); on a machine without it the previously built file is used.

Flags follow the reference's CPU semantics: -O2 -ffp-contract=off and no
-march, so no fused multiply-adds and no reassociation change the IEEE
operation order of src/cpu/ops.hxx.

Run: ``python oracle/build_oracle.py``
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: DCGAN_REFERENCE_DIR, else a directory `reference` next to this repository
REF_DIR = os.environ.get("DCGAN_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
PORT_LIB = os.path.join(HERE, "liboracle.so")
REF_OUT_DIR = os.path.join(HERE, "_ref")
REF_LIB = os.path.join(REF_OUT_DIR, "libdcgan_ref_cpu.so")

COMMON = ["-O2", "-ffp-contract=off", "-fPIC", "-shared", "-fno-fast-math"]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_port(force=False):
    src = os.path.join(HERE, "dcgan_oracle.c")
    if force or _stale(PORT_LIB, [src]):
        cmd = ["gcc", "-std=c11"] + COMMON + [src, "-o", PORT_LIB, "-lm"]
        subprocess.check_call(cmd)
    return PORT_LIB


def reference_available():
    return os.path.isfile(os.path.join(REF_DIR, "src", "cpu", "ops.hh"))


def build_ref(force=False):
    """Returns the path of the reference library, or None when it can neither
    be built (no reference checkout) nor found prebuilt."""
    if not reference_available():
        return REF_LIB if os.path.exists(REF_LIB) else None
    shim = os.path.join(HERE, "ref_shim.cc")
    xs = os.path.join(REF_DIR, "src", "utils", "xorshift.cu")
    if force or _stale(REF_LIB, [shim, xs, os.path.join(REF_DIR, "src", "cpu", "ops.hxx")]):
        os.makedirs(REF_OUT_DIR, exist_ok=True)
        cmd = (["g++", "-std=c++11", "-w"] + COMMON +
               ["-I", os.path.join(REF_DIR, "src"), shim, "-x", "c++", xs,
                "-o", REF_LIB])
        subprocess.check_call(cmd)
    return REF_LIB


def build(force=False):
    return build_port(force), build_ref(force)


if __name__ == "__main__":
    p, r = build(force="--force" in sys.argv)
    print("oracle port:", p)
    print("reference  :", r if r else "unavailable (no reference checkout, no prebuilt library)")
