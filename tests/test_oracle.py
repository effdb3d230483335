"""Pins the CPU oracle (oracle/dcgan_oracle.c).

1. against the committed golden vectors: inputs typed in the reference's own unit
   tests, outputs from the reference's CPU code (tests/golden/gen_golden.py);
2. bit for bit against the reference's CPU code compiled from its sources
   (oracle/_ref), on seeded random shapes including ragged / odd sizes;
3. against torch's conv2d / conv_transpose2d in fp64 as an independent second
   opinion on the SAME-padding and transposed-convolution conventions;
4. through adjoint identities for the padded transposed-convolution gradients,
   which the reference's CPU code only implements for zero padding.
"""
import numpy as np
import pytest

import oracle
from conftest import seeded


# ---- 1. golden vectors ---------------------------------------------------------
def test_golden_conv2d(orc, golden):
    for case in ("conv2d", "conv2d_padding"):
        y = orc.conv2d(golden[case + "/x"], golden[case + "/k"], (2, 2))
        assert np.array_equal(y, golden[case + "/y"]), case


@pytest.mark.parametrize("case", ["conv2d_grad", "conv2d_padding_grad"])
def test_golden_conv2d_grad(orc, golden, case):
    x, k, y = golden[case + "/x"], golden[case + "/k"], golden[case + "/y"]
    y_hat = orc.conv2d(x, k, (2, 2))
    assert np.array_equal(y_hat, golden[case + "/y_hat"])
    n = y.shape[0]
    dy = orc.mse_grad(y.reshape(n, -1), y_hat.reshape(n, -1)).reshape(y.shape)
    assert np.array_equal(dy, golden[case + "/dy_hat"])
    assert np.array_equal(orc.conv2d_input_grad(dy, k, 2, x.shape[1:3]), golden[case + "/dx"])
    assert np.array_equal(orc.conv2d_kernel_grad(dy, x, 2, tuple(golden[case + "/pad"])), golden[case + "/dk"])


def test_golden_conv2d_transpose(orc, golden):
    y = orc.conv2d_transpose(golden["conv2d_transpose/x"], golden["conv2d_transpose/k"], (2, 4, 4, 1), 2)
    assert np.array_equal(y, golden["conv2d_transpose/y"])
    c = "conv2d_transpose_grad"
    x, k, dy = golden[c + "/x"], golden[c + "/k"], golden[c + "/dy_hat"]
    assert np.array_equal(orc.conv2d_transpose(x, k, (2, 8, 8, 2), 2), golden[c + "/y_hat"])
    assert np.array_equal(orc.conv2d_transpose_input_grad(dy, k, 2, (4, 4)), golden[c + "/dx"])
    assert np.array_equal(orc.conv2d_transpose_kernel_grad(dy, x, 2, (2, 2)), golden[c + "/dk"])


def test_golden_bias(orc, golden):
    assert np.array_equal(orc.mvrow_add(golden["conv2d_bias_add/x"], golden["conv2d_bias_add/bias"]),
                          golden["conv2d_bias_add/out"])
    assert np.array_equal(orc.mat_sum_cols(golden["conv2d_bias_add_grad/dy_hat"]),
                          golden["conv2d_bias_add_grad/db"])


def test_golden_activation_grads(orc, golden):
    g = golden
    assert np.array_equal(orc.vect_relu_leaky(g["leaky_relu_grad/x"], 0.3), g["leaky_relu_grad/y_hat"])
    assert np.array_equal(orc.leaky_relu_grad(g["leaky_relu_grad/x"], g["leaky_relu_grad/dy_hat"], 0.3),
                          g["leaky_relu_grad/dx"])
    assert np.array_equal(orc.relu_grad(g["relu_grad/x"], g["relu_grad/dy_hat"]), g["relu_grad/dx"])
    assert np.array_equal(orc.vect_tanh(g["tanh_grad/x"]), g["tanh_grad/y_hat"])
    assert np.array_equal(orc.tanh_grad(g["tanh_grad/y_hat"], g["tanh_grad/dy_hat"]), g["tanh_grad/dx"])


def test_golden_losses_and_updates(orc, golden):
    g = golden
    assert orc.sigmoid_cross_entropy(g["sigmoid_cross_entropy/y"], g["sigmoid_cross_entropy/x"]) == \
        g["sigmoid_cross_entropy/loss"]
    assert np.array_equal(orc.sigmoid_cross_entropy_grad(g["sigmoid_cross_entropy_grad/y"],
                                                         g["sigmoid_cross_entropy_grad/x"]),
                          g["sigmoid_cross_entropy_grad/dx"])
    assert orc.argmax_acc(g["argmax/y"], g["argmax/y_hat"]) == g["argmax/acc"]
    # adam_update node alone (test_adam_update.cu): reproduce with zero-gradient moments
    import ctypes
    fp = ctypes.POINTER(ctypes.c_float)
    p = g["adam_update/x"].copy()
    t = ctypes.c_float(0)
    lrt = orc.lib.orc_adam_lr_t(ctypes.byref(t), ctypes.c_float(g["adam_update/lr"]),
                                ctypes.c_float(g["adam_update/beta1"]), ctypes.c_float(g["adam_update/beta2"]))
    m, v = np.ascontiguousarray(g["adam_update/m"]), np.ascontiguousarray(g["adam_update/v"])
    orc.lib.orc_adam_update(m.ctypes.data_as(fp), v.ctypes.data_as(fp), p.ctypes.data_as(fp),
                            ctypes.c_float(lrt), ctypes.c_float(g["adam_update/eps"]), ctypes.c_size_t(4))
    assert t.value == 1.0
    assert np.array_equal(p, g["adam_update/out"])
    for name, fn in (("moment_update", orc.lib.orc_moment_update), ("moment_update2", orc.lib.orc_moment_update2)):
        res = g[name + "/var"].copy()
        dt = np.ascontiguousarray(g[name + "/dt"])
        fn(dt.ctypes.data_as(fp), res.ctypes.data_as(fp), ctypes.c_float(g[name + "/c1"]),
           ctypes.c_float(g[name + "/c2"]), ctypes.c_size_t(4))
        assert np.array_equal(res, g[name + "/out"]), name


def test_golden_xorshift(orc, golden):
    orc.xorshift_seed(int(golden["xorshift/seed"]))
    assert np.array_equal(orc.xorshift_fill((64,)), golden["xorshift/f32"])


# ---- 2. bit-exact against the reference's compiled CPU code ---------------------
SHAPES = [  # N, H, W, C, K, O, stride
    (2, 8, 8, 4, 5, 6, 2), (1, 7, 9, 3, 5, 4, 2), (2, 6, 6, 2, 3, 3, 1), (2, 5, 4, 3, 2, 2, 2),
    (3, 3, 5, 1, 2, 3, 1), (1, 16, 16, 8, 5, 8, 2), (2, 9, 9, 5, 5, 2, 2), (1, 1, 1, 1, 1, 1, 1),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_port_matches_reference_conv(orc, ref, shape):
    N, H, W, C, K, O, s = shape
    x = seeded((N, H, W, C), 234)
    k = seeded((K, K, C, O), 235)
    y = orc.conv2d(x, k, (s, s))
    assert np.array_equal(y, ref.conv2d(x, k, (s, s)))
    dy = seeded(y.shape, 236)
    assert np.array_equal(orc.conv2d_input_grad(dy, k, s, (H, W)), ref.conv2d_input_grad(dy, k, s, (H, W)))
    pad = (oracle.same_pad(H, K, s), oracle.same_pad(W, K, s))
    assert np.array_equal(orc.conv2d_kernel_grad(dy, x, s, pad), ref.conv2d_kernel_grad(dy, x, s, pad))
    assert np.array_equal(orc.conv2d_transpose(dy, k, (N, H, W, C), s), ref.conv2d_transpose(dy, k, (N, H, W, C), s))


def test_port_matches_reference_transpose_grads_zero_pad(orc, ref):
    x = seeded((2, 4, 4, 3), 1)
    k = seeded((2, 2, 2, 3), 2)
    dy = seeded((2, 8, 8, 2), 3)
    assert np.array_equal(orc.conv2d_transpose_input_grad(dy, k, 2, (4, 4)),
                          ref.conv2d_transpose_input_grad(dy, k, 2, (4, 4)))
    assert np.array_equal(orc.conv2d_transpose_kernel_grad(dy, x, 2, (2, 2)),
                          ref.conv2d_transpose_kernel_grad(dy, x, 2, (2, 2)))


def test_port_matches_reference_elementwise(orc, ref):
    a = seeded((64, 33), 11, -3, 3)
    b = seeded((33, 17), 12)
    c = seeded((64, 17), 13)
    d = seeded((17, 33), 14)
    bias = seeded((17,), 15)
    assert np.array_equal(orc.mm_mul(a, b), ref.mm_mul(a, b))
    assert np.array_equal(orc.tmm_mul(a, c), ref.tmm_mul(a, c))
    assert np.array_equal(orc.mtm_mul(a, d), ref.mtm_mul(a, d))
    assert np.array_equal(orc.mat_mul_add(a, b, bias), ref.mat_mul_add(a, b, bias))
    assert np.array_equal(orc.mvrow_add(c, bias), ref.mvrow_add(c, bias))
    assert np.array_equal(orc.mat_sum_cols(c), ref.mat_sum_cols(c))
    assert np.array_equal(orc.mat_sum_rows(c), ref.mat_sum_rows(c))
    v = seeded((1000,), 16, -4, 4)
    w = seeded((1000,), 17)
    for f in ("vect_sigmoid", "vect_relu", "vect_relu_leaky", "vect_tanh"):
        assert np.array_equal(getattr(orc, f)(v), getattr(ref, f)(v)), f
    for f in ("relu_grad", "leaky_relu_grad", "sigmoid_grad", "vect_add", "sigmoid_cross_entropy_grad", "mse_grad"):
        assert np.array_equal(getattr(orc, f)(v, w), getattr(ref, f)(v, w)), f
    t = orc.vect_tanh(v)
    assert np.array_equal(orc.tanh_grad(t, w), ref.tanh_grad(t, w))
    labels = (seeded((1000,), 18) > 0).astype(np.float32)
    assert orc.sigmoid_cross_entropy(labels, v) == ref.sigmoid_cross_entropy(labels, v)
    assert orc.mse(a, a * np.float32(0.5)) == ref.mse(a, a * np.float32(0.5))
    noisy = a + seeded(a.shape, 19)
    assert orc.argmax_acc(a, noisy) == ref.argmax_acc(a, noisy)


def test_port_matches_reference_adam(orc, ref):
    p0 = seeded((4097,), 21)
    sp, sm, sv, st = p0.copy(), np.zeros_like(p0), np.zeros_like(p0), 0.0
    rp, rm, rv, rt = p0.copy(), np.zeros_like(p0), np.zeros_like(p0), 0.0
    for it in range(4):
        g = seeded((4097,), 30 + it)
        sp, sm, sv, st, l1 = orc.adam_step(sp, g, sm, sv, st, 2e-4, 0.5, 0.999, 1e-8)
        rp, rm, rv, rt, l2 = ref.adam_step(rp, g, rm, rv, rt, 2e-4, 0.5, 0.999, 1e-8)
        assert l1 == l2 and st == rt == it + 1
        assert np.array_equal(sp, rp) and np.array_equal(sm, rm) and np.array_equal(sv, rv)


# ---- 3. independent second opinion: torch in fp64 ---------------------------------
def _torch_conv(x, k, s, pad_total):
    import torch
    import torch.nn.functional as F
    pt, pl = pad_total[0] // 2, pad_total[1] // 2
    xt = torch.from_numpy(x).double().permute(0, 3, 1, 2)
    xt = F.pad(xt, (pl, pad_total[1] - pl, pt, pad_total[0] - pt))
    kt = torch.from_numpy(k).double().permute(3, 2, 0, 1)
    return F.conv2d(xt, kt, stride=s).permute(0, 2, 3, 1).numpy()


@pytest.mark.parametrize("shape", [(2, 8, 8, 4, 5, 6, 2), (1, 7, 9, 3, 5, 4, 2), (2, 16, 16, 3, 5, 8, 2)])
def test_port_matches_torch(orc, shape):
    import torch
    N, H, W, C, K, O, s = shape
    x = seeded((N, H, W, C), 41)
    k = seeded((K, K, C, O), 42)
    pad = (oracle.same_pad(H, K, s), oracle.same_pad(W, K, s))
    y = orc.conv2d(x, k, (s, s))
    np.testing.assert_allclose(y, _torch_conv(x, k, s, pad), rtol=0, atol=2e-5)
    # gradients through autograd of the same padded convolution
    dy = seeded(y.shape, 43)
    xt = torch.from_numpy(x).double().requires_grad_()
    kt = torch.from_numpy(k).double().requires_grad_()
    import torch.nn.functional as F
    pt, pl = pad[0] // 2, pad[1] // 2
    yt = F.conv2d(F.pad(xt.permute(0, 3, 1, 2), (pl, pad[1] - pl, pt, pad[0] - pt)),
                  kt.permute(3, 2, 0, 1), stride=s).permute(0, 2, 3, 1)
    yt.backward(torch.from_numpy(dy).double())
    np.testing.assert_allclose(orc.conv2d_input_grad(dy, k, s, (H, W)), xt.grad.numpy(), rtol=0, atol=5e-5)
    np.testing.assert_allclose(orc.conv2d_kernel_grad(dy, x, s, pad), kt.grad.numpy(), rtol=0, atol=2e-4)


# ---- 4. padded transposed-convolution gradients: adjoint identities --------------
def test_transpose_grads_are_adjoints(orc):
    # generator-style layer: [2,4,4,6] -> [2,8,8,5], 5x5 stride 2 SAME
    x = seeded((2, 4, 4, 6), 51)
    k = seeded((5, 5, 5, 6), 52)
    dy = seeded((2, 8, 8, 5), 53)
    y = orc.conv2d_transpose(x, k, (2, 8, 8, 5), 2).astype(np.float64)
    dx = orc.conv2d_transpose_input_grad(dy, k, 2, (4, 4)).astype(np.float64)
    dk = orc.conv2d_transpose_kernel_grad(dy, x, 2, (5, 5)).astype(np.float64)
    lhs = float((y * dy).sum())
    assert abs(lhs - float((dx * x).sum())) < 1e-3 * max(1.0, abs(lhs))
    assert abs(lhs - float((dk * k).sum())) < 1e-3 * max(1.0, abs(lhs))


def test_same_pad_rule():
    # src/ops/conv2d.cu:33-41
    assert oracle.same_pad(64, 5, 2) == 3 and oracle.same_pad(7, 5, 2) == 4
    assert oracle.same_pad(8, 2, 2) == 0 and oracle.same_pad(5, 3, 1) == 2
