"""GPU parity of the three convolution entry points (through the C ABI) against the CPU oracle.

DCG_PREC_FP32 keeps the reference CPU's summation order with unfused multiply/add and must
reproduce the oracle bit for bit.  DCG_PREC_TF32 (tcgen05, fp32 accumulate) must stay within
1e-2 * max|ref| per output tensor - the tolerance stated for the TF32 tensor-core path.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import seeded

pytestmark = pytest.mark.gpu

TF32_TOL = 1e-2  # max abs error <= TF32_TOL * max|ref|
X3_TOL = 1e-5    # 3xTF32 (operand = TF32 part + residual, three MMAs per K step), same norm

# N, H, W, C, K, O, stride.  Small / ragged shapes the reference's unit tests use, odd sizes,
# channel counts below and above one 32-wide K chunk, and DCGAN layer shapes at batch 2.
SHAPES = [
    (2, 4, 4, 2, 2, 2, 2), (2, 3, 5, 3, 3, 2, 2), (1, 7, 9, 3, 5, 4, 2), (2, 6, 6, 2, 3, 3, 1),
    (3, 3, 5, 1, 2, 3, 1), (2, 9, 9, 5, 5, 2, 2), (1, 1, 1, 1, 1, 1, 1),
    (2, 8, 8, 4, 5, 8, 2), (2, 16, 16, 32, 5, 64, 2), (2, 12, 20, 36, 5, 40, 2),
    (2, 64, 64, 3, 5, 64, 2), (2, 32, 32, 64, 5, 128, 2), (2, 16, 16, 128, 5, 256, 2),
    (2, 8, 8, 256, 5, 512, 2),
    # narrow-channel paths (<= 4 input channels, O a multiple of 32): window-map forward, one-tile
    # kernel gradient over pixel partitions, GEMM + gather input gradient; stride 1, even kernel
    (3, 20, 12, 1, 3, 32, 1), (2, 16, 16, 4, 5, 96, 2), (5, 32, 32, 2, 4, 64, 2), (2, 10, 14, 3, 5, 160, 2),
]


def _check(got, ref, prec, pkg, what):
    got = got.cpu().numpy()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    if prec == pkg.PREC_FP32:
        assert np.array_equal(got, ref), "%s: fp32 path differs from the oracle, max err %g" % (
            what, np.abs(got - ref).max())
    else:
        lim = (X3_TOL if prec == pkg.PREC_3XTF32 else TF32_TOL) * max(np.abs(ref).max(), 1e-30)
        err = np.abs(got - ref).max()
        assert err <= lim, "%s: max err %g > %g" % (what, err, lim)


PRECS = {"fp32": "PREC_FP32", "tf32": "PREC_TF32", "3xtf32": "PREC_3XTF32"}


@pytest.mark.parametrize("prec_name", ["fp32", "tf32", "3xtf32"])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv_fwd_dx_dk(pkg, dev, orc, shape, prec_name):
    F = pkg.functional
    prec = getattr(pkg, PRECS[prec_name])
    N, H, W, C, K, O, s = shape
    x = seeded((N, H, W, C), 234)
    k = seeded((K, K, C, O), 235) * np.float32(0.1)
    pad = (oracle.same_pad(H, K, s), oracle.same_pad(W, K, s))
    y_ref = orc.conv2d(x, k, (s, s))
    dy = seeded(y_ref.shape, 236)
    xd, kd, dyd = (torch.from_numpy(a).to(dev) for a in (x, k, dy))
    y = F.conv2d_fwd(xd, kd, (s, s), precision=prec)
    dx = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=prec)
    dk = F.conv2d_dk(xd, dyd, (K, K), (s, s), precision=prec)
    torch.cuda.synchronize()
    _check(y, y_ref, prec, pkg, "fwd")
    _check(dx, orc.conv2d_input_grad(dy, k, s, (H, W)), prec, pkg, "dx")
    _check(dk, orc.conv2d_kernel_grad(dy, x, s, pad), prec, pkg, "dk")


# stride 2 (four parity classes): the shapes the class-fused input gradient takes - tiles narrower and wider than
# 64 columns, a ragged channel chunk (40 = 32 + 8), two channel
# tiles (256 = 2 x 128), odd extents (a class with fewer rows / columns), 3x3 and 4x4 kernels
FUSED_DX_SHAPES = [
    (2, 16, 16, 32, 5, 64, 2), (2, 12, 20, 36, 5, 40, 2), (2, 32, 32, 64, 5, 128, 2), (2, 16, 16, 128, 5, 256, 2),
    (2, 8, 8, 256, 5, 512, 2), (1, 7, 9, 8, 5, 12, 2), (2, 9, 9, 8, 3, 8, 2), (3, 32, 32, 8, 4, 64, 2),
    # channel counts that rule out 16-byte stores (element-wise epilogue)
    (2, 16, 16, 6, 5, 32, 2), (2, 10, 14, 9, 5, 160, 2),
]


@pytest.mark.parametrize("shape", FUSED_DX_SHAPES)
def test_dx_with_parity_classes_fused(pkg, dev, orc, shape):
    """The input gradient that gives one CTA all parity classes of a pixel tile (planned by default only where
    one CTA per tile fills the GPU; forced here) against the reference's CPU code: plain, gated by the previous
    layer's activation with the raw gradient kept, and as a generator layer (bias, pre-activation, activation)."""
    F, L = pkg.functional, pkg.lib
    N, H, W, C, K, O, s = shape
    k = seeded((K, K, C, O), 235) * np.float32(0.1)
    y_shape = orc.conv2d(seeded((N, H, W, C), 234), k, (s, s)).shape
    dy = seeded(y_shape, 236)
    z = seeded((N, H, W, C), 237)
    b = seeded((C,), 238)
    dx_ref = orc.conv2d_input_grad(dy, k, s, (H, W))
    kd, dyd, zd, bd = (torch.from_numpy(a).to(dev) for a in (k, dy, z, b))
    before = L.dcg_debug_fused_dx_launches()
    try:
        L.dcg_debug_set_dx_mode(2)
        dx = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=pkg.PREC_TF32)
        raw = torch.empty(dx_ref.shape, device=dev)
        gated = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=pkg.PREC_TF32,
                            epilogue=F.make_epilogue(gate=zd, gate_act=pkg.ACT_LEAKY, gate_alpha=0.2, raw_out=raw))
        pre = torch.empty(dx_ref.shape, device=dev)
        act = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=pkg.PREC_TF32,
                          epilogue=F.make_epilogue(bias=bd, act=pkg.ACT_RELU, pre_act=pre))
        torch.cuda.synchronize()
    finally:
        L.dcg_debug_set_dx_mode(-1)
    assert L.dcg_device_status() == 0, L.dcg_last_error()
    assert L.dcg_debug_fused_dx_launches() - before == 3, "the fused kernel did not take this shape"
    _check(dx, dx_ref, pkg.PREC_TF32, pkg, "dx")
    _check(raw, dx_ref, pkg.PREC_TF32, pkg, "raw dx")
    _check(gated, orc.leaky_relu_grad(z, dx_ref, 0.2), pkg.PREC_TF32, pkg, "gated dx")
    pre_ref = orc.mvrow_add(dx_ref.reshape(-1, C), b).reshape(dx_ref.shape)
    _check(pre, pre_ref, pkg.PREC_TF32, pkg, "pre-activation")
    _check(act, orc.vect_relu(pre_ref), pkg.PREC_TF32, pkg, "activation")
    # and the same call planned the other way gives the same numbers up to TF32 summation order
    L.dcg_debug_set_dx_mode(0)
    try:
        dx0 = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=pkg.PREC_TF32)
        torch.cuda.synchronize()
    finally:
        L.dcg_debug_set_dx_mode(-1)
    assert L.dcg_debug_fused_dx_launches() - before == 3
    _check(dx0, dx_ref, pkg.PREC_TF32, pkg, "dx, one tile per class")


@pytest.mark.parametrize("shape", [(40, 64, 64, 3, 5, 64, 2), (40, 60, 52, 3, 5, 64, 2), (37, 64, 64, 4, 5, 32, 2)])
def test_three_channel_layers_with_persistent_ctas(pkg, dev, orc, shape):
    """More tiles than SMs: the forward of a <= 4-channel layer and the GEMM of its input gradient run as
    persistent CTAs that walk several tiles each (weights resident, accumulator double-buffered).  Forward with
    the whole fused chain, input gradient with bias + tanh (a generator's last layer), against the CPU code;
    tile counts that do and do not divide by the grid, output extents that do not fill the pixel tiles."""
    F = pkg.functional
    N, H, W, C, K, O, s = shape
    x = seeded((N, H, W, C), 234)
    k = seeded((K, K, C, O), 235) * np.float32(0.1)
    b = seeded((O,), 303)
    raw_ref = orc.conv2d(x, k, (s, s))
    z_ref = orc.mvrow_add(raw_ref, b)
    xd, kd, bd = (torch.from_numpy(a).to(dev) for a in (x, k, b))
    raw = torch.empty(raw_ref.shape, device=dev)
    z = torch.empty(raw_ref.shape, device=dev)
    y = F.conv2d_fwd(xd, kd, (s, s), precision=pkg.PREC_TF32,
                     epilogue=F.make_epilogue(bias=bd, act=pkg.ACT_LEAKY, alpha=0.2, pre_act=z, raw_out=raw))
    torch.cuda.synchronize()
    assert pkg.lib.dcg_device_status() == 0, pkg.lib.dcg_last_error()
    _check(raw, raw_ref, pkg.PREC_TF32, pkg, "raw")
    _check(z, z_ref, pkg.PREC_TF32, pkg, "pre-activation")
    _check(y, orc.vect_relu_leaky(z_ref, 0.2), pkg.PREC_TF32, pkg, "activation")
    dy = seeded(raw_ref.shape, 236)
    bc = seeded((C,), 304)
    dyd, bcd = torch.from_numpy(dy).to(dev), torch.from_numpy(bc).to(dev)
    dx_ref = orc.conv2d_input_grad(dy, k, s, (H, W))
    dx = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=pkg.PREC_TF32)
    t = F.conv2d_dx(dyd, kd, (H, W), (s, s), precision=pkg.PREC_TF32, epilogue=F.make_epilogue(bias=bcd, act=pkg.ACT_TANH))
    torch.cuda.synchronize()
    assert pkg.lib.dcg_device_status() == 0, pkg.lib.dcg_last_error()
    _check(dx, dx_ref, pkg.PREC_TF32, pkg, "dx")
    np.testing.assert_allclose(t.cpu().numpy(), orc.vect_tanh(orc.mvrow_add(dx_ref, bc)), rtol=0,
                               atol=TF32_TOL * max(np.abs(dx_ref).max(), 1.0))


@pytest.mark.parametrize("prec_name", ["fp32", "tf32"])
def test_golden_reference_cases(pkg, dev, golden, prec_name):
    """The reference's own unit-test tensors (tests/test_conv2d*.cu) through the C ABI."""
    F = pkg.functional
    prec = pkg.PREC_FP32 if prec_name == "fp32" else pkg.PREC_TF32
    for case in ("conv2d", "conv2d_padding"):
        x, k = (torch.from_numpy(golden[case + "/" + n]).to(dev) for n in ("x", "k"))
        _check(F.conv2d_fwd(x, k, precision=prec), golden[case + "/y"], prec, pkg, case)
    for case in ("conv2d_grad", "conv2d_padding_grad"):
        x, k, dy = (torch.from_numpy(golden[case + "/" + n]).to(dev) for n in ("x", "k", "dy_hat"))
        _check(F.conv2d_dx(dy, k, x.shape[1:3], precision=prec), golden[case + "/dx"], prec, pkg, case + " dx")
        _check(F.conv2d_dk(x, dy, k.shape[:2], precision=prec), golden[case + "/dk"], prec, pkg, case + " dk")
    # conv2d_transpose = dx of the mirrored conv; its gradients = fwd / dk with roles swapped
    c = "conv2d_transpose_grad"
    x, k, dy = (torch.from_numpy(golden[c + "/" + n]).to(dev) for n in ("x", "k", "dy_hat"))
    _check(F.conv2d_dx(x, k, (8, 8), pad=(0, 0), precision=prec), golden[c + "/y_hat"], prec, pkg, "convT fwd")
    _check(F.conv2d_fwd(dy, k, pad=(0, 0), precision=prec), golden[c + "/dx"], prec, pkg, "convT dx")
    _check(F.conv2d_dk(dy, x, (2, 2), pad=(0, 0), precision=prec), golden[c + "/dk"], prec, pkg, "convT dk")


@pytest.mark.parametrize("prec_name", ["fp32", "tf32"])
@pytest.mark.parametrize("shape", [(2, 9, 9, 5, 5, 6, 2), (2, 16, 16, 32, 5, 64, 2), (2, 16, 16, 3, 5, 64, 2)])
def test_fused_epilogues(pkg, dev, orc, shape, prec_name):
    F = pkg.functional
    prec = pkg.PREC_FP32 if prec_name == "fp32" else pkg.PREC_TF32
    N, H, W, C, K, O, s = shape
    x = seeded((N, H, W, C), 301)
    k = seeded((K, K, C, O), 302) * np.float32(0.1)
    b = seeded((O,), 303)
    raw_ref = orc.conv2d(x, k, (s, s))
    z_ref = orc.mvrow_add(raw_ref, b)
    xd, kd, bd = (torch.from_numpy(a).to(dev) for a in (x, k, b))
    for act, fn in ((pkg.ACT_LEAKY, lambda a: orc.vect_relu_leaky(a, 0.2)), (pkg.ACT_RELU, orc.vect_relu),
                    (pkg.ACT_TANH, orc.vect_tanh), (pkg.ACT_SIGMOID, orc.vect_sigmoid), (pkg.ACT_NONE, lambda a: a)):
        raw = torch.empty(raw_ref.shape, device=dev)
        z = torch.empty(raw_ref.shape, device=dev)
        ep = F.make_epilogue(bias=bd, act=act, alpha=0.2, pre_act=z, raw_out=raw)
        y = F.conv2d_fwd(xd, kd, (s, s), epilogue=ep, precision=prec)
        torch.cuda.synchronize()
        _check(raw, raw_ref, prec, pkg, "raw")
        _check(z, z_ref, prec, pkg, "pre_act")
        a_ref = fn(z_ref)
        if prec == pkg.PREC_FP32 and act in (pkg.ACT_TANH, pkg.ACT_SIGMOID):
            # device expf is not glibc's: a few ulp on the exponential
            np.testing.assert_allclose(y.cpu().numpy(), a_ref, rtol=0, atol=2e-6)
        else:
            _check(y, a_ref, prec, pkg, "act %d" % act)

    # input gradient gated by the derivative of the previous layer's activation
    dy = seeded(raw_ref.shape, 304)
    zprev = seeded((N, H, W, C), 305)
    dyd, zd = torch.from_numpy(dy).to(dev), torch.from_numpy(zprev).to(dev)
    dx_ref = orc.conv2d_input_grad(dy, k, s, (H, W))
    for gact, fn in ((pkg.ACT_LEAKY, lambda g, d: orc.leaky_relu_grad(g, d, 0.2)), (pkg.ACT_RELU, orc.relu_grad),
                     (pkg.ACT_TANH, orc.tanh_grad)):
        raw = torch.empty(dx_ref.shape, device=dev)
        ep = F.make_epilogue(gate=zd, gate_act=gact, gate_alpha=0.2, raw_out=raw)
        dx = F.conv2d_dx(dyd, kd, (H, W), (s, s), epilogue=ep, precision=prec)
        torch.cuda.synchronize()
        _check(raw, dx_ref, prec, pkg, "dx raw")
        ref_g = fn(zprev, dx_ref)
        if prec == pkg.PREC_FP32:
            assert np.array_equal(dx.cpu().numpy(), ref_g)
        else:
            _check(dx, ref_g, prec, pkg, "gated dx")


def test_transposed_conv_roles(pkg, dev, orc):
    """Generator layer [2,4,4,64] -> [2,8,8,32] (5x5, stride 2, SAME): forward is the dx entry
    point, its input gradient the fwd entry point, its kernel gradient dk with roles swapped."""
    F = pkg.functional
    x = seeded((2, 4, 4, 64), 401)
    k = seeded((5, 5, 32, 64), 402) * np.float32(0.05)   # [kh, kw, Cout, Cin]
    dy = seeded((2, 8, 8, 32), 403)
    xd, kd, dyd = (torch.from_numpy(a).to(dev) for a in (x, k, dy))
    for prec in (pkg.PREC_FP32, pkg.PREC_TF32):
        y = F.conv2d_dx(xd, kd, (8, 8), precision=prec)
        dx = F.conv2d_fwd(dyd, kd, precision=prec)
        dk = F.conv2d_dk(dyd, xd, (5, 5), precision=prec)
        torch.cuda.synchronize()
        _check(y, orc.conv2d_transpose(x, k, (2, 8, 8, 32), 2), prec, pkg, "convT")
        _check(dx, orc.conv2d_transpose_input_grad(dy, k, 2, (4, 4)), prec, pkg, "convT dx")
        _check(dk, orc.conv2d_transpose_kernel_grad(dy, x, 2, (5, 5)), prec, pkg, "convT dk")


@pytest.mark.parametrize("layer", [(64, 32, 32, 64, 128), (64, 16, 16, 128, 256), (64, 8, 8, 256, 512),
                                   (64, 64, 64, 3, 64)])
def test_full_batch_layers_tf32_vs_fp32_path(pkg, dev, layer):
    """Batch-64 DCGAN layers: too slow for the scalar oracle, so the tensor path is compared with
    the fp32 CUDA-core path (itself bit-exact with the oracle at small sizes), and the three
    operators are tied together by the adjoint identity <conv(x,k),dy> = <x,dx> = <k,dk>."""
    F = pkg.functional
    N, H, W, C, O = layer
    g = torch.Generator(device="cpu").manual_seed(5)
    x = (torch.rand((N, H, W, C), generator=g) * 2 - 1).to(dev)
    k = (torch.randn((5, 5, C, O), generator=g) * 0.02).to(dev)
    dy = (torch.rand((N, H // 2, W // 2, O), generator=g) * 2 - 1).to(dev)
    outs = {}
    for prec in (pkg.PREC_FP32, pkg.PREC_TF32):
        outs[prec] = (F.conv2d_fwd(x, k, precision=prec), F.conv2d_dx(dy, k, (H, W), precision=prec),
                      F.conv2d_dk(x, dy, (5, 5), precision=prec))
    torch.cuda.synchronize()
    for name, a, b in zip(("fwd", "dx", "dk"), outs[pkg.PREC_FP32], outs[pkg.PREC_TF32]):
        lim = TF32_TOL * a.abs().max().item()
        assert (a - b).abs().max().item() <= lim, name
    # 3xTF32 is held to 1e-5 * max|ref| against a float64 evaluation (torch, same SAME padding: 1 before,
    # 2 after): at these sizes the fp32 paths themselves carry ~sqrt(K) * 2^-24 = 1.5e-5 of summation
    # noise in the longest reductions (65 536 pixels per kernel-gradient element), which the yardstick
    # must not
    x3 = (F.conv2d_fwd(x, k, precision=pkg.PREC_3XTF32), F.conv2d_dx(dy, k, (H, W), precision=pkg.PREC_3XTF32),
          F.conv2d_dk(x, dy, (5, 5), precision=pkg.PREC_3XTF32))
    torch.cuda.synchronize()
    assert pkg.lib.dcg_device_status() == 0
    x64 = x.double().permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    k64 = k.double().permute(3, 2, 0, 1).contiguous().requires_grad_(True)
    y64 = torch.nn.functional.conv2d(torch.nn.functional.pad(x64, (1, 2, 1, 2)), k64, stride=2)
    dx64, dk64 = torch.autograd.grad(y64, (x64, k64), dy.double().permute(0, 3, 1, 2).contiguous())
    ref64 = (y64.detach().permute(0, 2, 3, 1), dx64.permute(0, 2, 3, 1), dk64.permute(2, 3, 1, 0))
    for name, a, b in zip(("fwd", "dx", "dk"), ref64, x3):
        assert (a - b.double()).abs().max().item() <= X3_TOL * a.abs().max().item(), "3xTF32 " + name
    for name, a, b in zip(("fwd", "dx", "dk"), ref64, outs[pkg.PREC_FP32]):   # the yardstick agrees with the fp32 path
        assert (a - b.double()).abs().max().item() <= 1e-4 * a.abs().max().item(), "fp32 vs float64 " + name
    y, dx, dk = (t.double() for t in outs[pkg.PREC_TF32])
    terms = y * dy.double()
    lhs = terms.sum().item()
    # the inner product is a sum of ~1e6 signed terms that largely cancel; TF32 rounding (~5e-4 per
    # term, random sign) perturbs it by about 5e-4 * sqrt(sum of squared terms)
    tol = 5e-3 * terms.pow(2).sum().sqrt().item() + 1e-3
    assert abs(lhs - (dx * x.double()).sum().item()) <= tol
    assert abs(lhs - (dk * k.double()).sum().item()) <= tol


@pytest.mark.parametrize("batch", [20, 28, 40, 56, 100])
def test_k_partition_counts(pkg, dev, batch):
    """The number of K partitions of a tile (= thread-block cluster size) follows the tile count:
    these batches give clusters of 8, 8/7, 7/5, 5/4 and 2/3 CTAs on a 148-SM part for the
    128 -> 256 channel layer, odd sizes included.  Each must agree with the fp32 path and with itself."""
    F = pkg.functional
    g = torch.Generator(device="cpu").manual_seed(11)
    x = (torch.rand((batch, 16, 16, 128), generator=g) * 2 - 1).to(dev)
    k = (torch.randn((5, 5, 128, 256), generator=g) * 0.02).to(dev)
    dy = (torch.rand((batch, 8, 8, 256), generator=g) * 2 - 1).to(dev)
    bias = torch.randn((256,), generator=g).to(dev)
    ref = (F.conv2d_fwd(x, k, precision=pkg.PREC_FP32) + bias, F.conv2d_dx(dy, k, (16, 16), precision=pkg.PREC_FP32),
           F.conv2d_dk(x, dy, (5, 5), precision=pkg.PREC_FP32))
    run = lambda: (F.conv2d_fwd(x, k, epilogue=F.make_epilogue(bias=bias)), F.conv2d_dx(dy, k, (16, 16)),
                   F.conv2d_dk(x, dy, (5, 5)))
    a, b = run(), run()
    torch.cuda.synchronize()
    assert pkg.lib.dcg_device_status() == 0
    for name, r, u, v in zip(("fwd+bias", "dx", "dk"), ref, a, b):
        assert (r - u).abs().max().item() <= TF32_TOL * r.abs().max().item(), name
        assert torch.equal(u, v), name


def test_deterministic(pkg, dev):
    """Two runs of every operator give identical bits (fixed-order split-K reduction)."""
    F = pkg.functional
    g = torch.Generator(device="cpu").manual_seed(9)
    x = (torch.rand((8, 16, 16, 128), generator=g) * 2 - 1).to(dev)
    k = (torch.randn((5, 5, 128, 256), generator=g) * 0.02).to(dev)
    dy = (torch.rand((8, 8, 8, 256), generator=g) * 2 - 1).to(dev)
    a = (F.conv2d_fwd(x, k), F.conv2d_dx(dy, k, (16, 16)), F.conv2d_dk(x, dy, (5, 5)))
    b = (F.conv2d_fwd(x, k), F.conv2d_dx(dy, k, (16, 16)), F.conv2d_dk(x, dy, (5, 5)))
    torch.cuda.synchronize()
    for u, v in zip(a, b):
        assert torch.equal(u, v)


def test_workspace_and_alignment_contract(pkg, dev, orc):
    """What the entry points promise about their operands: a tensor-path call that needs scratch
    refuses a buffer that is too small (nothing is launched, the output stays untouched) and says how
    much it wants; operands that are not 16-byte aligned (which TMA cannot address) silently take the
    CUDA-core path, whose result is the oracle's bit for bit."""
    import ctypes
    F, L = pkg.functional, pkg.lib
    # 128 -> 256 channels at batch 8: few tiles, so the K partitions need scratch
    g = torch.Generator(device="cpu").manual_seed(41)
    x = (torch.rand((8, 16, 16, 128), generator=g) * 2 - 1).to(dev)
    k = (torch.randn((5, 5, 128, 256), generator=g) * 0.02).to(dev)
    d = F.conv_desc(x.shape, k.shape, (2, 2), None, None)
    need = L.dcg_conv_workspace_bytes(ctypes.byref(d), pkg._lib.KIND_FWD, pkg.PREC_TF32)
    assert need > 0
    y = torch.full((8, 8, 8, 256), 7.0, device=dev)
    small = torch.empty(need // 2, dtype=torch.uint8, device=dev)
    st = L.dcg_conv2d_fwd(ctypes.byref(d), x.data_ptr(), k.data_ptr(), y.data_ptr(), None, pkg.PREC_TF32,
                          small.data_ptr(), small.numel(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == pkg._lib.ERR_WORKSPACE and b"workspace" in L.dcg_last_error()
    assert bool((y == 7.0).all())
    assert L.dcg_conv_workspace_bytes(ctypes.byref(d), pkg._lib.KIND_FWD, pkg.PREC_FP32) == 0

    # the same small layer from a buffer that starts 4 bytes off a 16-byte boundary
    xs = seeded((2, 8, 8, 32), 42)
    ks = seeded((5, 5, 32, 64), 43) * np.float32(0.1)
    raw = torch.empty(xs.size + 1, device=dev)
    xo = raw[1:].view(2, 8, 8, 32)
    xo.copy_(torch.from_numpy(xs))
    assert xo.data_ptr() % 16 == 4
    y_off = F.conv2d_fwd(xo, torch.from_numpy(ks).to(dev), precision=pkg.PREC_TF32)
    torch.cuda.synchronize()
    assert np.array_equal(y_off.cpu().numpy(), orc.conv2d(xs, ks, (2, 2)))



# (batch, H, Cin, Cout): the four DCGAN layers at the batch the benchmark runs (64) and at the 128
# images of the discriminator's single pass over [fake | real]
BENCH_LAYERS = [(b, h, c, o) for b in (64, 128) for (h, c, o) in ((64, 3, 64), (32, 64, 128), (16, 128, 256), (8, 256, 512))]


@pytest.mark.parametrize("layer", BENCH_LAYERS)
def test_benchmark_shapes_vs_reference_cpu_code(pkg, dev, ref, layer):
    """The shapes bench.py times - with their K partitions, cluster shapes and two-wave grids -
    against the reference's own CPU code (oracle/_ref = src/cpu/ops.hxx compiled from its sources) on
    xorshift inputs (seed 234 as tests/test_conv_s1.cu:31).  The scalar CPU code needs minutes for a
    whole batch-64 layer, so it is run on what is independent: forward and input gradient on the
    first and last image (images do not interact), the kernel gradient over the WHOLE batch on
    two 4-channel slices of x and dy (dk[:, :, c, o] only reads x[..., c] and dy[..., o]; the slice
    keeps the reference's (n, i, j) summation order, src/cpu/ops.hxx:754-772).
    Bounds: fp32 path bit-equal, TF32 path 1e-2 * max|ref|."""
    F = pkg.functional
    B, H, C, O = layer
    Ho = H // 2
    x = seeded((B, H, H, C), 234)
    k = (seeded((5, 5, C, O), 235) * np.float32(0.05)).astype(np.float32)
    dy = seeded((B, Ho, Ho, O), 236)
    xd, kd, dyd = (torch.from_numpy(a).to(dev) for a in (x, k, dy))
    ends = [0, B - 1]
    y_ref = ref.conv2d(x[ends], k, (2, 2))
    dx_ref = ref.conv2d_input_grad(dy[ends], k, 2, (H, H))
    slices = [(0, 0), (max(C - 4, 0), O - 4)]
    pad = (oracle.same_pad(H, 5, 2), oracle.same_pad(H, 5, 2))
    dk_refs = [ref.conv2d_kernel_grad(np.ascontiguousarray(dy[..., o0:o0 + 4]), np.ascontiguousarray(x[..., c0:c0 + 4]), 2, pad)
               for c0, o0 in slices]
    for prec in (pkg.PREC_FP32, pkg.PREC_TF32):
        y = F.conv2d_fwd(xd, kd, precision=prec)
        dx = F.conv2d_dx(dyd, kd, (H, H), precision=prec)
        dk = F.conv2d_dk(xd, dyd, (5, 5), precision=prec)
        torch.cuda.synchronize()
        assert pkg.lib.dcg_device_status() == 0
        _check(y[ends], y_ref, prec, pkg, "fwd images 0 and %d" % (B - 1))
        _check(dx[ends], dx_ref, prec, pkg, "dx images 0 and %d" % (B - 1))
        for (c0, o0), dk_ref in zip(slices, dk_refs):
            got = dk[:, :, c0:c0 + 4, o0:o0 + 4].contiguous()
            if prec == pkg.PREC_FP32:
                _check(got, dk_ref, prec, pkg, "dk slice c%d o%d" % (c0, o0))
            else:   # the bound is on the operator's output tensor: scale by the whole dk
                lim = TF32_TOL * float(dk.abs().max())
                assert float(np.abs(got.cpu().numpy() - dk_ref).max()) <= lim, "dk slice c%d o%d" % (c0, o0)


def test_bounded_wait_runs_out_and_the_context_survives(pkg, dev):
    """Failure detection without a fault: the producer is told to leave one pipeline stage out, so
    the MMA warp's wait on that stage can never complete; with the wait limit lowered to about a
    millisecond the kernel gives up, records (block, role, stage) in the device status word, still
    reaches its final barrier and frees TMEM.  dcg_device_status() then reports DCG_ERR_DEVICE, and a
    normal call right after passes - the context stays usable."""
    F, L = pkg.functional, pkg.lib
    x = seeded((80, 32, 32, 32), 501)         # 160 tiles of 128 pixels: more tiles than SMs, so no K partitions, no cluster
    k = seeded((5, 5, 32, 64), 502) * np.float32(0.1)
    xd, kd = torch.from_numpy(x).to(dev), torch.from_numpy(k).to(dev)
    assert L.dcg_device_status() == 0
    try:
        L.dcg_debug_set_wait_limit(2_000_000)   # ~1 ms of SM clocks
        L.dcg_debug_skip_stage(3)
        F.conv2d_fwd(xd, kd, precision=pkg.PREC_TF32)
        torch.cuda.synchronize()                # returns: every wait in the kernel is bounded
    finally:
        L.dcg_debug_skip_stage(-1)
        L.dcg_debug_set_wait_limit(0)
    assert L.dcg_device_status() == pkg._lib.ERR_DEVICE
    assert b"gave up waiting" in L.dcg_last_error()
    assert L.dcg_device_status() == 0           # reading clears the word
    y = F.conv2d_fwd(xd, kd, precision=pkg.PREC_TF32)
    torch.cuda.synchronize()
    assert L.dcg_device_status() == 0
    y32 = F.conv2d_fwd(xd, kd, precision=pkg.PREC_FP32)   # bit-equal to the oracle (test_conv_fwd_dx_dk)
    torch.cuda.synchronize()
    assert (y - y32).abs().max().item() <= TF32_TOL * y32.abs().max().item()
