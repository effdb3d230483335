"""The C-ABI library loads without a GPU and exports what include/dcgan_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dcgan_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(dcg_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("dcg_conv2d_fwd", "dcg_conv2d_dx", "dcg_conv2d_dk", "dcg_adam_multi", "dcg_run_nodes",
                 "dcg_colsum", "dcg_sigmoid_xent", "dcg_bias_act", "dcg_act_grad", "dcg_matmul"):
        assert must in names
    assert len(names) >= 30


def test_library_exports_every_declared_symbol(pkg):
    for name in declared_functions():
        assert hasattr(pkg.lib, name), "libdcgan_b200.so does not export " + name


def test_python_binding_covers_every_declared_symbol(pkg):
    assert sorted(pkg._lib.SIGNATURES) == declared_functions()


def test_argument_errors_need_no_gpu(pkg):
    L = pkg.lib
    # null descriptor / null tensors are rejected before anything touches CUDA
    assert L.dcg_conv2d_fwd(None, None, None, None, None, 0, None, 0, None) == pkg._lib.ERR_INVALID
    assert b"null descriptor" in L.dcg_last_error()
    d = pkg.functional.conv_desc((1, 8, 8, 4), (5, 5, 4, 8))
    assert L.dcg_conv2d_fwd(ctypes.byref(d), None, None, None, None, 0, None, 0, None) == pkg._lib.ERR_INVALID
    assert L.dcg_conv2d_fwd(ctypes.byref(d), 16, 16, 16, None, 99, None, 0, None) == pkg._lib.ERR_INVALID
    bad = pkg.functional.conv_desc((1, 8, 8, 4), (5, 5, 4, 8))
    bad.stride_h = 0
    assert L.dcg_conv2d_dk(ctypes.byref(bad), 16, 16, 16, 0, None, 0, None) == pkg._lib.ERR_INVALID
    assert L.dcg_adam_multi(None, 3, 0.1, 0.5, 0.9, 1e-8, 1.0, None) == pkg._lib.ERR_INVALID
    assert L.dcg_colsum(None, None, 4, 4, None, 0, None) == pkg._lib.ERR_INVALID
    with pytest.raises(pkg.DcgError):
        pkg._lib.check(L.dcg_add(None, None, None, 4, None))


def test_conv_desc_same_padding(pkg):
    d = pkg.functional.conv_desc((64, 64, 64, 3), (5, 5, 3, 64))
    assert (d.ho, d.wo, d.pad_top, d.pad_left) == (32, 32, 1, 1)
    d = pkg.functional.conv_desc((2, 7, 9, 3), (5, 5, 3, 4))
    assert (d.ho, d.wo, d.pad_top, d.pad_left) == (4, 5, 2, 2)


def test_adam_lr_t_is_host_side(pkg):
    t = ctypes.c_float(0)
    lr1 = pkg.functional.adam_lr_t(t, 2e-4, 0.5, 0.999)
    assert t.value == 1.0
    import numpy as np
    expect = np.float32(2e-4) * np.sqrt(np.float32(1) - np.float32(0.999)) / (np.float32(1) - np.float32(0.5))
    assert abs(lr1 - float(expect)) < 1e-10
