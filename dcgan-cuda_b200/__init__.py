"""dcgan_b200: the B200 (sm_100a) convolution / Adam hot path of dcgan-cuda.

All compute lives in libdcgan_b200.so (hand-written CUDA behind the C ABI of
include/dcgan_b200.h).  This package is the thin host side: ctypes bindings,
runtime-instruction records mirroring the reference's rt::Node, and helpers
that pass torch CUDA tensors' device pointers through.

The directory name carries a hyphen, so the package is imported under the name
``dcgan_cuda_b200`` through ``__graft_entry__.load_package()``.
"""
from . import _lib, functional, nodes  # noqa: F401
from ._lib import (ACT_LEAKY, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH, PREC_3XTF32,  # noqa: F401
                   PREC_FP32, PREC_TF32, DcgError, lib)
from .nodes import Context  # noqa: F401


def build_info():
    return lib.dcg_build_info().decode()


def launches_total():
    """Kernels launched by the library since it was loaded."""
    return int(lib.dcg_launches_total())
from .trainer import Trainer  # noqa: E402,F401
