"""Generates tests/golden/reference_cases.npz.

Inputs: the hand-typed tensors of the reference's own unit tests, parsed as text
from its tests/test_*.cu files (the reference stores inputs only; its expected
values were produced by TensorFlow at test time).  Expected outputs: the
reference's own CPU implementation (src/cpu/ops.hxx), compiled from its sources
into oracle/_ref/ and called through oracle.reference() - the same arithmetic
`RT_MODE=CPU` runs.  The graph each case evaluates follows the test's main().

Needs a reference checkout (environment variable DCGAN_REFERENCE_DIR, or the default
of oracle/build_oracle.py); the committed .npz is what travels.

Run: ``python tests/golden/gen_golden.py``
"""
import ctypes
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oracle import build_oracle  # noqa: E402

REF_TESTS = os.path.join(build_oracle.REF_DIR, "tests")
ARRAY_RE = re.compile(r"dbl_t\s+(\w+)\s*\[\d*\]\s*=\s*\{([^}]*)\}", re.S)
SCALAR_RE = re.compile(r"dbl_t\s+(\w+)\s*=\s*([-+0-9.eE]+)\s*;")


def parse(test_name):
    """Returns ({array name: flat float32 array}, {scalar name: float}) of a reference test."""
    text = open(os.path.join(REF_TESTS, test_name)).read()
    text = re.sub(r"//[^\n]*", "", text)
    arrays = {}
    for name, body in ARRAY_RE.findall(text):
        vals = [float("".join(v.split())) for v in body.split(",") if v.strip()]
        arrays[name] = np.asarray(vals, dtype=np.float32)
    scalars = {name: float(v) for name, v in SCALAR_RE.findall(text)}
    return arrays, scalars


def conv_grad_case(R, arrays, x_shape, k_shape, y_shape, stride=2):
    x = arrays["input"].reshape(x_shape)
    k = arrays["kernel"].reshape(k_shape)
    y = arrays["y"].reshape(y_shape)
    y_hat = R.conv2d(x, k, (stride, stride))
    n = y.shape[0]
    dy_hat = R.mse_grad(y.reshape(n, -1), y_hat.reshape(n, -1)).reshape(y_shape)
    pad = (oracle.same_pad(x_shape[1], k_shape[0], stride), oracle.same_pad(x_shape[2], k_shape[1], stride))
    return {"x": x, "k": k, "y": y, "y_hat": y_hat, "dy_hat": dy_hat,
            "dx": R.conv2d_input_grad(dy_hat, k, stride, x_shape[1:3]),
            "dk": R.conv2d_kernel_grad(dy_hat, x, stride, pad),
            "pad": np.asarray(pad, dtype=np.int32)}


def act_grad_case(R, arrays, fwd, grad):
    x = arrays["x"].reshape(4, 3)
    y = arrays["y"].reshape(4, 3)
    y_hat = fwd(x)
    dy_hat = R.mse_grad(y, y_hat)
    return {"x": x, "y": y, "y_hat": y_hat, "dy_hat": dy_hat, "dx": grad(x, y_hat, dy_hat)}


def main():
    R = oracle.reference()
    if R is None or not build_oracle.reference_available():
        raise SystemExit("no reference checkout: cannot regenerate the golden vectors")
    out = {}

    def put(case, d):
        for k, v in d.items():
            out[case + "/" + k] = np.asarray(v)

    a, _ = parse("test_conv2d.cu")
    x, k = a["input"].reshape(2, 4, 4, 2), a["kernel"].reshape(2, 2, 2, 2)
    put("conv2d", {"x": x, "k": k, "y": R.conv2d(x, k, (2, 2))})

    a, _ = parse("test_conv2d_padding.cu")
    x, k = a["input"].reshape(2, 3, 5, 3), a["kernel"].reshape(2, 3, 3, 2)
    put("conv2d_padding", {"x": x, "k": k, "y": R.conv2d(x, k, (2, 2))})

    a, _ = parse("test_conv2d_grad.cu")
    put("conv2d_grad", conv_grad_case(R, a, (2, 4, 4, 3), (2, 2, 3, 2), (2, 2, 2, 2)))

    a, _ = parse("test_conv2d_padding_grad.cu")
    put("conv2d_padding_grad", conv_grad_case(R, a, (2, 3, 5, 3), (2, 3, 3, 2), (2, 2, 3, 2)))

    a, _ = parse("test_conv2d_transpose.cu")
    x, k = a["input"].reshape(2, 2, 2, 1), a["kernel"].reshape(2, 2, 1, 1)
    put("conv2d_transpose", {"x": x, "k": k, "y": R.conv2d_transpose(x, k, (2, 4, 4, 1), 2)})

    a, _ = parse("test_conv2d_transpose_grad.cu")
    x, k, y = a["input"].reshape(2, 4, 4, 3), a["kernel"].reshape(2, 2, 2, 3), a["y"].reshape(2, 8, 8, 2)
    y_hat = R.conv2d_transpose(x, k, (2, 8, 8, 2), 2)
    dy_hat = R.mse_grad(y.reshape(2, -1), y_hat.reshape(2, -1)).reshape(y.shape)
    put("conv2d_transpose_grad", {
        "x": x, "k": k, "y": y, "y_hat": y_hat, "dy_hat": dy_hat,
        "dx": R.conv2d_transpose_input_grad(dy_hat, k, 2, (4, 4)),
        "dk": R.conv2d_transpose_kernel_grad(dy_hat, x, 2, (2, 2))})

    a, _ = parse("test_conv2d_bias_add.cu")
    x, b = a["input"].reshape(2, 2, 2, 2), a["bias"]
    put("conv2d_bias_add", {"x": x, "bias": b, "out": R.mvrow_add(x, b)})

    a, _ = parse("test_conv2d_bias_add_grad.cu")
    x, b, y = a["input"].reshape(2, 2, 2, 2), a["bias"], a["y"].reshape(2, 2, 2, 2)
    y_hat = R.mvrow_add(x, b)
    dy_hat = R.mse_grad(y.reshape(2, 8), y_hat.reshape(2, 8)).reshape(2, 2, 2, 2)
    put("conv2d_bias_add_grad", {"x": x, "bias": b, "y": y, "dy_hat": dy_hat, "dx": dy_hat,
                                 "db": R.mat_sum_cols(dy_hat)})

    a, _ = parse("test_leaky_relu_grad.cu")
    put("leaky_relu_grad", act_grad_case(R, a, lambda x: R.vect_relu_leaky(x, 0.3),
                                         lambda x, yh, d: R.leaky_relu_grad(x, d, 0.3)))
    a, _ = parse("test_relu_grad.cu")
    put("relu_grad", act_grad_case(R, a, R.vect_relu, lambda x, yh, d: R.relu_grad(x, d)))
    a, _ = parse("test_tanh_grad.cu")
    put("tanh_grad", act_grad_case(R, a, R.vect_tanh, lambda x, yh, d: R.tanh_grad(yh, d)))

    a, _ = parse("test_sigmoid_cross_entropy.cu")
    x, y = a["x"].reshape(5, 3), a["y"].reshape(5, 3)
    put("sigmoid_cross_entropy", {"x": x, "y": y, "loss": R.sigmoid_cross_entropy(y, x)})
    a, _ = parse("test_sigmoid_cross_entropy_grad.cu")
    x, y = a["x"].reshape(5, 3), a["y"].reshape(5, 3)
    put("sigmoid_cross_entropy_grad", {"x": x, "y": y, "dx": R.sigmoid_cross_entropy_grad(y, x)})

    for name, sq in (("moment_update", False), ("moment_update2", True)):
        a, s = parse("test_%s.cu" % name)
        var, dt = a["a"].reshape(2, 2), a["b"].reshape(2, 2)
        res = var.copy()
        fn = R.lib.ref_moment_update2 if sq else R.lib.ref_moment_update
        fn(dt.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
           res.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
           ctypes.c_float(s["c1"]), ctypes.c_float(s["c2"]), ctypes.c_size_t(4))
        put(name, {"var": var, "dt": dt, "c1": np.float32(s["c1"]), "c2": np.float32(s["c2"]), "out": res})

    # test_adam_update.cu: builder.adam_update(x, m, v, 0.45, 0.68, 0.27, 2), first step (t: 0 -> 1)
    a, _ = parse("test_adam_update.cu")
    p = a["x"].copy()
    t = ctypes.c_float(0)
    lrt = R.lib.ref_adam_lr_t(ctypes.byref(t), ctypes.c_float(0.45), ctypes.c_float(0.68), ctypes.c_float(0.27))
    fp = ctypes.POINTER(ctypes.c_float)
    R.lib.ref_adam_update(a["m"].ctypes.data_as(fp), a["v"].ctypes.data_as(fp), p.ctypes.data_as(fp),
                          ctypes.c_float(lrt), ctypes.c_float(2), ctypes.c_size_t(4))
    put("adam_update", {"x": a["x"], "m": a["m"], "v": a["v"], "lr": np.float32(0.45),
                        "beta1": np.float32(0.68), "beta2": np.float32(0.27), "eps": np.float32(2),
                        "out": p})

    a, _ = parse("test_argmax.cu")
    y, y_hat = a["y"].reshape(10, 3), a["y_hat"].reshape(10, 3)
    put("argmax", {"y": y, "y_hat": y_hat, "acc": R.argmax_acc(y, y_hat)})

    # seeded generator: first values after xorshift::seed(234) (tests/test_conv_s1.cu:31)
    R.xorshift_seed(234)
    put("xorshift", {"seed": np.int64(234), "f32": R.xorshift_fill((64,))})

    path = os.path.join(HERE, "reference_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, "with", len(out), "arrays,", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
