"""The node-level backend (dcg_run_node / dcg_run_nodes): the reference's gpu::kernels_list / gpu::run.

Nodes are built with the mirrors of the reference's rt::Node::op_* factories, packed as the
reference's Op::compile() methods pack them, and executed through the C ABI.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from conftest import seeded

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def test_golden_graphs_through_nodes(pkg, dev, golden):
    """tests/test_conv2d_grad.cu as a node list: conv2d -> mse_grad -> input/kernel gradients."""
    N = pkg.nodes
    ctx = pkg.Context(pkg.PREC_FP32)
    for case in ("conv2d_grad", "conv2d_padding_grad"):
        x, k, y = (_t(golden[case + "/" + n], dev) for n in ("x", "k", "y"))
        pad = [int(v) for v in golden[case + "/pad"]]
        y_hat = torch.empty(golden[case + "/y_hat"].shape, device=dev)
        dy = torch.empty_like(y_hat)
        dx, dk = torch.empty_like(x), torch.empty_like(k)
        strides = (2, 2)
        nodes = [
            N.op_conv2d(x, k, strides, pad[0], pad[1], y_hat, x.shape, k.shape),
            N.op_mse_grad(y, y_hat, dy, y.numel()),
            N.op_conv2d_input_grad(dy, k, strides, dx, dy.shape, k.shape, x.shape),
            N.op_conv2d_kernel_grad(dy, x, strides, dk, dy.shape, x.shape, pad),
        ]
        ctx.run(nodes)
        torch.cuda.synchronize()
        for got, key in ((y_hat, "y_hat"), (dy, "dy_hat"), (dx, "dx"), (dk, "dk")):
            assert np.array_equal(got.cpu().numpy(), golden[case + "/" + key]), (case, key)

    # tests/test_conv2d_transpose_grad.cu
    c = "conv2d_transpose_grad"
    x, k, y = (_t(golden[c + "/" + n], dev) for n in ("x", "k", "y"))
    y_hat, dy = torch.empty_like(y), torch.empty_like(y)
    dx, dk = torch.empty_like(x), torch.empty_like(k)
    nodes = [
        N.op_conv2d_transpose(x, k, y.shape, (2, 2), y_hat, x.shape, k.shape),
        N.op_mse_grad(y, y_hat, dy, y.numel()),
        N.op_conv2d_transpose_input_grad(dy, k, (2, 2), dx, dy.shape, k.shape, x.shape),
        N.op_conv2d_transpose_kernel_grad(dy, x, (2, 2), dk, dy.shape, x.shape, k.shape),
    ]
    ctx.run(nodes)
    torch.cuda.synchronize()
    for got, key in ((y_hat, "y_hat"), (dy, "dy_hat"), (dx, "dx"), (dk, "dk")):
        assert np.array_equal(got.cpu().numpy(), golden[c + "/" + key]), key
    ctx.close()


def _layer_nodes(N, bufs):
    """One discriminator layer forward and backward, lowered like dcgan/main.cu:123-168 + autodiff:
    conv2d -> mat_rvect_add -> relu_leaky ; leaky_relu_grad -> (mat_sum_cols, kernel grad, input grad
    -> leaky_relu_grad of the layer below)."""
    b = bufs
    n, h, w, c = b["x"].shape
    kh, kw, _, o = b["k"].shape
    ho, wo = b["conv"].shape[1:3]
    pad = (oracle.same_pad(h, kh, 2), oracle.same_pad(w, kw, 2))
    rows = n * ho * wo
    fwd = [
        N.op_conv2d(b["x"], b["k"], (2, 2), pad[0], pad[1], b["conv"], b["x"].shape, b["k"].shape),
        N.op_mat_rvect_add(b["conv"], b["bias"], b["z"], rows, o),
        N.op_relu_leaky(b["z"], b["a"], rows * o, 0.2),
    ]
    bwd = [
        N.op_leaky_relu_grad(b["z"], b["da"], b["dz"], 0.2, rows * o),
        N.op_mat_sum_cols(b["dz"], b["db"], rows, o),
        N.op_conv2d_kernel_grad(b["dz"], b["x"], (2, 2), b["dk"], b["dz"].shape, b["x"].shape, pad),
        N.op_conv2d_input_grad(b["dz"], b["k"], (2, 2), b["dx"], b["dz"].shape, b["k"].shape, b["x"].shape),
        N.op_leaky_relu_grad(b["zprev"], b["dx"], b["dzprev"], 0.2, b["x"].numel()),
    ]
    return fwd, bwd


@pytest.mark.parametrize("prec_name", ["fp32", "tf32"])
def test_fused_equals_unfused_and_oracle(pkg, dev, orc, prec_name):
    N = pkg.nodes
    prec = pkg.PREC_FP32 if prec_name == "fp32" else pkg.PREC_TF32
    x = seeded((4, 16, 16, 32), 901)
    k = seeded((5, 5, 32, 64), 902) * np.float32(0.05)
    bias = seeded((64,), 903) * np.float32(0.1)
    da = seeded((4, 8, 8, 64), 904)
    zprev = seeded((4, 16, 16, 32), 905)

    def fresh():
        b = {"x": _t(x, dev), "k": _t(k, dev), "bias": _t(bias, dev), "da": _t(da, dev), "zprev": _t(zprev, dev)}
        for name, shape in (("conv", (4, 8, 8, 64)), ("z", (4, 8, 8, 64)), ("a", (4, 8, 8, 64)), ("dz", (4, 8, 8, 64)),
                            ("db", (64,)), ("dk", (5, 5, 32, 64)), ("dx", (4, 16, 16, 32)), ("dzprev", (4, 16, 16, 32))):
            b[name] = torch.full(shape, float("nan"), device=dev)
        return b

    results = {}
    launches = {}
    for fuse in (False, True):
        ctx = pkg.Context(prec)
        b = fresh()
        fwd, bwd = _layer_nodes(N, b)
        ctx.run(fwd + bwd, fuse=fuse)
        torch.cuda.synchronize()
        launches[fuse] = ctx.launch_count()
        results[fuse] = {kk: v.cpu().numpy() for kk, v in b.items()}
        ctx.close()
    # every buffer, intermediate ones included, is identical with and without fusion
    for name in ("conv", "z", "a", "dz", "db", "dk", "dx", "dzprev"):
        assert np.array_equal(results[False][name], results[True][name]), name
    assert launches[True] < launches[False]

    # Each operator is checked against the oracle applied to the inputs the GPU gave it: on the TF32
    # path a pre-activation within rounding distance of zero may land on the other side of the
    # leaky-relu kink, which changes downstream values by a finite step and is not an error.
    got = results[True]
    exact = prec == pkg.PREC_FP32
    conv = orc.conv2d(x, k, (2, 2))
    z = orc.mvrow_add(conv if exact else got["conv"], bias)
    dz = orc.leaky_relu_grad(z if exact else got["z"], da, 0.2)
    dz_in = dz if exact else got["dz"]
    dx = orc.conv2d_input_grad(dz_in, k, 2, (16, 16))
    ref = {"conv": conv, "z": z, "a": orc.vect_relu_leaky(z if exact else got["z"], 0.2), "dz": dz,
           "dk": orc.conv2d_kernel_grad(dz_in, x, 2, (3, 3)), "dx": dx,
           "dzprev": orc.leaky_relu_grad(zprev, dx if exact else got["dx"], 0.2)}
    for name, r in ref.items():
        got = results[True][name]
        if prec == pkg.PREC_FP32:
            assert np.array_equal(got, r), name
        else:
            assert np.abs(got - r).max() <= 1e-2 * np.abs(r).max(), name
    np.testing.assert_allclose(results[True]["db"], orc.mat_sum_cols(dz), rtol=0, atol=1e-4)


def test_dead_intermediates_are_skipped_only_when_flagged(pkg, dev):
    N = pkg.nodes
    x = _t(seeded((2, 8, 8, 32), 911), dev)
    k = _t(seeded((5, 5, 32, 32), 912) * np.float32(0.05), dev)
    bias = _t(seeded((32,), 913), dev)
    conv = torch.full((2, 4, 4, 32), -7.0, device=dev)
    z, a = torch.empty_like(conv), torch.empty_like(conv)
    nodes = [N.op_conv2d(x, k, (2, 2), 3, 3, conv, x.shape, k.shape),
             N.op_mat_rvect_add(conv, bias, z, 32, 32), N.op_relu_leaky(z, a, 1024, 0.2)]
    nodes[0].flags = pkg._lib.NODE_OUT_DEAD
    ctx = pkg.Context(pkg.PREC_FP32)
    ctx.run(nodes, fuse=True)
    torch.cuda.synchronize()
    assert (conv == -7.0).all()          # flagged dead: never stored
    assert torch.isfinite(z).all() and torch.isfinite(a).all()
    assert ctx.launch_count() == 1
    ctx.close()


def test_adam_triples_fuse_into_one_launch(pkg, dev, orc):
    """AdamOptimizer::minimize lowers each variable to moment_update, moment_update(sq), adam_update
    (src/api/adam-optimizer.cu:24-59); a run of such triples becomes one multi-tensor launch."""
    N = pkg.nodes
    sizes = [4800, 64, 204800, 128]
    lr, b1, b2, eps = 2e-4, 0.5, 0.999, 1e-8
    host = {}
    for fuse in (False, True):
        ps = [_t(seeded((n,), 920 + i), dev) for i, n in enumerate(sizes)]
        ms = [torch.zeros_like(p) for p in ps]
        vs = [torch.zeros_like(p) for p in ps]
        ts = [ctypes.c_float(0) for _ in sizes]
        ctx = pkg.Context(pkg.PREC_FP32)
        for step in range(2):
            gs = [_t(seeded((n,), 930 + 10 * step + i), dev) for i, n in enumerate(sizes)]
            nodes = []
            for p, g, m, v, t in zip(ps, gs, ms, vs, ts):
                # 1 - beta is formed in fp32, as AdamOptimizer::minimize does with its dbl_t members
                nodes += [N.op_moment_update(m, g, b1, float(np.float32(1) - np.float32(b1)), p.numel()),
                          N.op_moment_update2(v, g, b2, float(np.float32(1) - np.float32(b2)), p.numel()),
                          N.op_adam_update(p, t, m, v, lr, b1, b2, eps, p.numel())]
            before = ctx.launch_count()
            ctx.run(nodes, fuse=fuse)
            torch.cuda.synchronize()
            assert ctx.launch_count() - before == (1 if fuse else 3 * len(sizes))
        assert all(t.value == 2.0 for t in ts)
        host[fuse] = [p.cpu().numpy() for p in ps]
        ctx.close()
    for a, b in zip(host[False], host[True]):
        assert np.array_equal(a, b)
    # and both equal the oracle
    for i, n in enumerate(sizes):
        p, m, v, t = seeded((n,), 920 + i), np.zeros(n, np.float32), np.zeros(n, np.float32), 0.0
        for step in range(2):
            p, m, v, t, _ = orc.adam_step(p, seeded((n,), 930 + 10 * step + i), m, v, t, lr, b1, b2, eps)
        assert np.array_equal(host[True][i], p)


@pytest.mark.parametrize("prec_name", ["fp32", "tf32"])
def test_small_neighbours_fuse_into_one_launch(pkg, dev, prec_name):
    """Pairs of neighbouring nodes that run as one launch when fusion is on: dense layer + activation (tensor path:
    one 1x1-convolution launch with the activation in its epilogue), sigmoid cross-entropy + its gradient, x W^T + the
    activation gradient that gates it.  Every output of the unfused list is still written and is bit-identical."""
    N = pkg.nodes
    prec = pkg.PREC_FP32 if prec_name == "fp32" else pkg.PREC_TF32
    B = 64
    z, w, b = _t(seeded((B, 100), 1), dev), _t(seeded((100, 8192), 2) * np.float32(0.05), dev), _t(seeded((8192,), 3), dev)
    labels, logits = torch.ones((B, 1), device=dev), _t(seeded((B, 1), 4), dev)
    wh, gate = _t(seeded((8192, 1), 5), dev), _t(seeded((B, 8192), 6), dev)
    results = {}
    for fuse in (False, True):
        pre, act = torch.empty((B, 8192), device=dev), torch.empty((B, 8192), device=dev)
        loss, dl = torch.empty((1,), device=dev), torch.empty((B, 1), device=dev)
        dda, ddz = torch.empty((B, 8192), device=dev), torch.empty((B, 8192), device=dev)
        nodes = [
            N.op_mat_mul_add(z, w, b, pre, B, 100, 8192),
            N.op_relu_leaky(pre, act, pre.numel(), 0.2),
            N.op_sigmoid_cross_entropy(labels, logits, loss, B),
            N.op_sigmoid_cross_entropy_grad(labels, logits, dl, B),
            N.op_mat_tmat_mul(dl, wh, dda, B, 1, 8192),
            N.op_leaky_relu_grad(gate, dda, ddz, 0.2, dda.numel()),
        ]
        ctx = pkg.Context(prec)
        ctx.run(nodes, fuse=fuse)      # first run may allocate scratch
        before = ctx.launch_count()
        ctx.run(nodes, fuse=fuse)
        torch.cuda.synchronize()
        launches = ctx.launch_count() - before
        results[fuse] = ([t.cpu().numpy() for t in (pre, act, loss, dl, dda, ddz)], launches)
        ctx.close()
    for a, c in zip(results[False][0], results[True][0]):
        assert np.array_equal(a, c)
    # fp32: the dense layer stays on the CUDA-core kernel (no fused form), the other two pairs fuse
    assert results[False][1] == 6
    assert results[True][1] == (4 if prec_name == "fp32" else 3)


def test_reshape_is_an_alias_and_unknown_nodes_fail(pkg, dev):
    """Reshape lowers to no instruction at all (src/ops/reshape.cu:20-44): the consumer reads the
    producer's buffer, so it is bit-exact by construction.  Unknown node types are errors."""
    N = pkg.nodes
    a = _t(seeded((64, 4, 4, 8), 940), dev)
    out = torch.empty((64, 128), device=dev)
    ctx = pkg.Context(pkg.PREC_FP32)
    ctx.run([N.op_relu(a, out, a.numel())])   # consumer sees the 4-D tensor as [64, 128]
    torch.cuda.synchronize()
    assert torch.equal(out.view(-1), torch.relu(a).view(-1))
    bad = pkg._lib.Node()
    bad.type = 99
    with pytest.raises(pkg.DcgError):
        ctx.run_node(bad)
    ctx.close()
