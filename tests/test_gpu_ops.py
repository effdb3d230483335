"""GPU parity of the memory-bound operators and the dense layers against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import seeded

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _s():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("rows,cols", [(8, 2), (64 * 16 * 16, 128), (1000, 3), (77, 36), (64, 8192), (5, 1)])
def test_bias_act_and_colsum(pkg, dev, orc, rows, cols):
    L = pkg.lib
    a = seeded((rows, cols), 500)
    b = seeded((cols,), 501)
    ad, bd = _t(a, dev), _t(b, dev)
    z, act = torch.empty_like(ad), torch.empty_like(ad)
    pkg._lib.check(L.dcg_bias_act(ad.data_ptr(), bd.data_ptr(), z.data_ptr(), act.data_ptr(), rows, cols,
                                  pkg.ACT_LEAKY, 0.2, _s()))
    torch.cuda.synchronize()
    z_ref = orc.mvrow_add(a, b)
    assert np.array_equal(z.cpu().numpy(), z_ref)
    assert np.array_equal(act.cpu().numpy(), orc.vect_relu_leaky(z_ref, 0.2))
    got = pkg.functional.colsum(ad).cpu().numpy()
    ref = orc.mat_sum_cols(a)
    # different (tree) summation order than the sequential reference loop
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-6 * rows ** 0.5 + 1e-5 * np.abs(ref).max())
    rs = torch.empty((rows,), device=dev)
    pkg._lib.check(L.dcg_rowsum(ad.data_ptr(), rs.data_ptr(), rows, cols, _s()))
    np.testing.assert_allclose(rs.cpu().numpy(), orc.mat_sum_rows(a), rtol=0, atol=1e-5 * max(1, cols) ** 0.5)


@pytest.mark.parametrize("n", [1, 12, 4099, 1 << 20])
def test_activations_and_grads(pkg, dev, orc, n):
    L = pkg.lib
    a = seeded((n,), 510, -4, 4)
    d = seeded((n,), 511)
    ad, dd = _t(a, dev), _t(d, dev)
    out = torch.empty_like(ad)
    for act, fn, exact in ((pkg.ACT_LEAKY, lambda v: orc.vect_relu_leaky(v, 0.3), True),
                           (pkg.ACT_RELU, orc.vect_relu, True), (pkg.ACT_TANH, orc.vect_tanh, False),
                           (pkg.ACT_SIGMOID, orc.vect_sigmoid, False)):
        pkg._lib.check(L.dcg_act_fwd(ad.data_ptr(), out.data_ptr(), n, act, 0.3, _s()))
        got = out.cpu().numpy()
        if exact:
            assert np.array_equal(got, fn(a))
        else:
            np.testing.assert_allclose(got, fn(a), rtol=0, atol=2e-6)
    t = orc.vect_tanh(a)
    sg = orc.vect_sigmoid(a)
    for act, gate, fn in ((pkg.ACT_LEAKY, a, lambda g, x: orc.leaky_relu_grad(g, x, 0.3)),
                          (pkg.ACT_RELU, a, orc.relu_grad), (pkg.ACT_TANH, t, orc.tanh_grad),
                          (pkg.ACT_SIGMOID, sg, orc.sigmoid_grad)):
        gd = _t(gate, dev)
        pkg._lib.check(L.dcg_act_grad(gd.data_ptr(), dd.data_ptr(), out.data_ptr(), n, act, 0.3, _s()))
        assert np.array_equal(out.cpu().numpy(), fn(gate, d)), act
    pkg._lib.check(L.dcg_add(ad.data_ptr(), dd.data_ptr(), out.data_ptr(), n, _s()))
    assert np.array_equal(out.cpu().numpy(), orc.vect_add(a, d))
    coeff = torch.tensor([-0.37], device=dev)
    var = ad.clone()
    pkg._lib.check(L.dcg_update(dd.data_ptr(), var.data_ptr(), coeff.data_ptr(), n, _s()))
    assert np.array_equal(var.cpu().numpy(), orc.vect_update(d, a, -0.37))


def test_golden_small_ops(pkg, dev, golden):
    """The reference's unit-test tensors for bias add, activation gradients, losses, argmax."""
    L, g = pkg.lib, golden
    x, b = _t(g["conv2d_bias_add/x"], dev), _t(g["conv2d_bias_add/bias"], dev)
    out = torch.empty_like(x)
    pkg._lib.check(L.dcg_bias_act(x.data_ptr(), b.data_ptr(), out.data_ptr(), None, 8, 2, 0, 0.0, _s()))
    assert np.array_equal(out.cpu().numpy(), g["conv2d_bias_add/out"])
    assert np.array_equal(pkg.functional.colsum(_t(g["conv2d_bias_add_grad/dy_hat"], dev)).cpu().numpy(),
                          g["conv2d_bias_add_grad/db"])
    for case, act, gate_key in (("leaky_relu_grad", pkg.ACT_LEAKY, "x"), ("relu_grad", pkg.ACT_RELU, "x"),
                                ("tanh_grad", pkg.ACT_TANH, "y_hat")):
        gate, d = _t(g[case + "/" + gate_key], dev), _t(g[case + "/dy_hat"], dev)
        o = torch.empty_like(d)
        pkg._lib.check(L.dcg_act_grad(gate.data_ptr(), d.data_ptr(), o.data_ptr(), d.numel(), act, 0.3, _s()))
        assert np.array_equal(o.cpu().numpy(), g[case + "/dx"]), case
    x, y = _t(g["sigmoid_cross_entropy/x"], dev), _t(g["sigmoid_cross_entropy/y"], dev)
    loss = torch.empty((1,), device=dev)
    pkg._lib.check(L.dcg_sigmoid_xent(y.data_ptr(), x.data_ptr(), loss.data_ptr(), 15, _s()))
    assert abs(loss.item() - float(g["sigmoid_cross_entropy/loss"])) < 1e-6
    dx = torch.empty_like(x)
    pkg._lib.check(L.dcg_sigmoid_xent_grad(y.data_ptr(), x.data_ptr(), dx.data_ptr(), 15, _s()))
    np.testing.assert_allclose(dx.cpu().numpy(), g["sigmoid_cross_entropy_grad/dx"], rtol=0, atol=1e-7)
    ya, yh = _t(g["argmax/y"], dev), _t(g["argmax/y_hat"], dev)
    acc = torch.empty((1,), device=dev)
    pkg._lib.check(L.dcg_argmax_acc(ya.data_ptr(), yh.data_ptr(), acc.data_ptr(), 10, 3, _s()))
    assert acc.item() == float(g["argmax/acc"])  # bit-exact integer count


def test_argmax_first_max_wins_and_is_exact(pkg, dev, orc):
    rows, cols = 5000, 10
    a = np.round(seeded((rows, cols), 520) * 3).astype(np.float32)  # many ties
    b = np.round(seeded((rows, cols), 521) * 3).astype(np.float32)
    acc = torch.empty((1,), device=dev)
    ad, bd = _t(a, dev), _t(b, dev)
    pkg._lib.check(pkg.lib.dcg_argmax_acc(ad.data_ptr(), bd.data_ptr(), acc.data_ptr(), rows, cols, _s()))
    assert acc.item() == float(orc.argmax_acc(a, b))


@pytest.mark.parametrize("m,n,p", [(64, 100, 8192), (64, 8192, 1), (3, 5, 7), (100, 64, 130), (64, 784, 100)])
def test_dense(pkg, dev, orc, m, n, p):
    L = pkg.lib
    a = seeded((m, n), 530)
    b = seeded((n, p), 531) * np.float32(0.1)
    bias = seeded((p,), 532)
    ad, bd, biasd = _t(a, dev), _t(b, dev), _t(bias, dev)
    out = torch.empty((m, p), device=dev)
    pkg._lib.check(L.dcg_matmul(ad.data_ptr(), bd.data_ptr(), biasd.data_ptr(), out.data_ptr(), m, n, p, _s()))
    ref = orc.mat_mul_add(a, b, bias)
    tol = 1e-6 * n ** 0.5 * max(1.0, np.abs(ref).max())
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=0, atol=tol)
    pkg._lib.check(L.dcg_matmul(ad.data_ptr(), bd.data_ptr(), None, out.data_ptr(), m, n, p, _s()))
    np.testing.assert_allclose(out.cpu().numpy(), orc.mm_mul(a, b), rtol=0, atol=tol)
    # dW = x^T dy  (x [m, n] stored, dy [m, p]) -> [n, p]
    dy = seeded((m, p), 533)
    dyd = _t(dy, dev)
    dw = torch.empty((n, p), device=dev)
    pkg._lib.check(L.dcg_matmul_tn(ad.data_ptr(), dyd.data_ptr(), dw.data_ptr(), n, m, p, _s()))
    assert np.array_equal(dw.cpu().numpy(), orc.tmm_mul(a, dy))
    # dx = dy W^T  (dy [m, p], W [n, p]) -> [m, n]
    dx = torch.empty((m, n), device=dev)
    pkg._lib.check(L.dcg_matmul_nt(dyd.data_ptr(), bd.data_ptr(), dx.data_ptr(), m, p, n, _s()))
    assert np.array_equal(dx.cpu().numpy(), orc.mtm_mul(dy, b))


def test_losses(pkg, dev, orc):
    L = pkg.lib
    for n in (64, 1000):
        x = seeded((n,), 540, -5, 5)
        y = (seeded((n,), 541) > 0).astype(np.float32)
        xd, yd = _t(x, dev), _t(y, dev)
        loss = torch.empty((1,), device=dev)
        pkg._lib.check(L.dcg_sigmoid_xent(yd.data_ptr(), xd.data_ptr(), loss.data_ptr(), n, _s()))
        assert abs(loss.item() - float(orc.sigmoid_cross_entropy(y, x))) < 2e-6 * max(1, abs(loss.item()))
        g = torch.empty_like(xd)
        pkg._lib.check(L.dcg_sigmoid_xent_grad(yd.data_ptr(), xd.data_ptr(), g.data_ptr(), n, _s()))
        np.testing.assert_allclose(g.cpu().numpy(), orc.sigmoid_cross_entropy_grad(y, x), rtol=0, atol=1e-7)
    a, b = seeded((32, 10), 542), seeded((32, 10), 543)
    ad, bd = _t(a, dev), _t(b, dev)
    out = torch.empty((1,), device=dev)
    pkg._lib.check(L.dcg_mse(ad.data_ptr(), bd.data_ptr(), out.data_ptr(), 32, 10, _s()))
    assert abs(out.item() - float(orc.mse(a, b))) < 1e-6
    g = torch.empty_like(ad)
    pkg._lib.check(L.dcg_mse_grad(ad.data_ptr(), bd.data_ptr(), g.data_ptr(), 320, _s()))
    assert np.array_equal(g.cpu().numpy(), orc.mse_grad(a, b))
    # softmax family against torch (MNIST example operators)
    sm = torch.empty_like(ad)
    pkg._lib.check(L.dcg_softmax(ad.data_ptr(), sm.data_ptr(), 32, 10, _s()))
    assert torch.allclose(sm, torch.softmax(ad, 1), atol=1e-6)
    pkg._lib.check(L.dcg_log_softmax(ad.data_ptr(), sm.data_ptr(), 32, 10, _s()))
    assert torch.allclose(sm, torch.log_softmax(ad, 1), atol=1e-5)
    onehot = torch.zeros_like(ad)
    onehot[torch.arange(32), torch.arange(32) % 10] = 1
    pkg._lib.check(L.dcg_softmax_xent(onehot.data_ptr(), ad.data_ptr(), out.data_ptr(), 32, 10, _s()))
    want = -(onehot * torch.log_softmax(ad, 1)).sum() / 32
    assert abs(out.item() - want.item()) < 1e-5
    pkg._lib.check(L.dcg_softmax_xent_grad(onehot.data_ptr(), ad.data_ptr(), sm.data_ptr(), 32, 10, _s()))
    assert torch.allclose(sm, (torch.softmax(ad, 1) - onehot) / 32, atol=1e-6)


@pytest.mark.parametrize("sizes", [[5000], [3, 64, 4800, 512, 204800, 1], [4096 * 3 + 5, 7]])
def test_adam_multi_bit_exact(pkg, dev, orc, sizes):
    """Fused multi-tensor Adam == the reference's moment/moment2/adam node triple, bit for bit,
    over several steps (lr 2e-4, beta1 0.5, beta2 0.999, eps 1e-8 as dcgan/main.cu:35-36)."""
    F = pkg.functional
    ps = [seeded((n,), 600 + i) for i, n in enumerate(sizes)]
    ms = [np.zeros_like(p) for p in ps]
    vs = [np.zeros_like(p) for p in ps]
    pd, md, vd = ([_t(a, dev) for a in lst] for lst in (ps, ms, vs))
    t_ref = 0.0
    t = ctypes.c_float(0)
    for step in range(3):
        gs = [seeded((n,), 700 + 10 * step + i) for i, n in enumerate(sizes)]
        gd = [_t(g, dev) for g in gs]
        lr_t = F.adam_lr_t(t, 2e-4, 0.5, 0.999)
        F.adam_multi(pd, gd, md, vd, lr_t, 0.5, 0.999, 1e-8)
        torch.cuda.synchronize()
        for i in range(len(sizes)):
            ps[i], ms[i], vs[i], t_new, lr_ref = orc.adam_step(ps[i], gs[i], ms[i], vs[i], t_ref, 2e-4, 0.5, 0.999, 1e-8)
            assert lr_t == float(lr_ref)
            assert np.array_equal(pd[i].cpu().numpy(), ps[i]), (step, i)
            assert np.array_equal(md[i].cpu().numpy(), ms[i]) and np.array_equal(vd[i].cpu().numpy(), vs[i])
        t_ref = t_new
        assert t.value == t_ref


def test_adam_grad_scale_and_second_path(pkg, dev, orc):
    """grad_scale (the 1/world of data-parallel averaging) and the optional second gradient path."""
    F = pkg.functional
    n = 10000
    p, g1, g2 = seeded((n,), 801), seeded((n,), 802), seeded((n,), 803)
    pd, g1d, g2d = _t(p, dev), _t(g1, dev), _t(g2, dev)
    md, vd = torch.zeros_like(pd), torch.zeros_like(pd)
    F.adam_multi([pd], [g1d], [md], [vd], 1e-3, 0.5, 0.999, 1e-8, grad_scale=0.25, grads2=[g2d])
    g = (g1 + g2) * np.float32(0.25)
    ref, _, _, _, _ = orc.adam_step(p, g, np.zeros_like(p), np.zeros_like(p), 0.0, 2e-4, 0.5, 0.999, 1e-8)
    # same update with lr_t = 1e-3 instead of the schedule's value: recompute by hand
    m = np.float32(0.5) * g
    v = (np.float32(1) - np.float32(0.999)) * g * g
    want = p - np.float32(1e-3) * m / (np.sqrt(v) + np.float32(1e-8))
    np.testing.assert_allclose(pd.cpu().numpy(), want, rtol=0, atol=1e-6)
