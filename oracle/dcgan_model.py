"""CPU restatement of one DCGAN training iteration, built from the oracle's operators.

TEST INFRASTRUCTURE ONLY (parity checks of the trainer, and the timed CPU baseline).

The model and the order of operations follow dcgan/main.cu: generator :44-120 (dense 100 -> 8192,
four 5x5 stride-2 conv2d_transpose layers 512 -> 256 -> 128 -> 64 -> 3, tanh), discriminator
:123-249 (four 5x5 stride-2 conv2d layers 3 -> 64 -> 128 -> 256 -> 512 with leaky-relu 0.2,
dense 8192 -> 1), sigmoid cross-entropy losses :304-307, Adam :329-332, and one iteration =
one discriminator update + two generator updates, each recomputing its forward passes :378-391.

`be` is an oracle back-end: oracle.port() or oracle.reference().  The transposed-convolution
gradients go through conv2d / conv2d_kernel_grad with the roles swapped, which is what the
reference's GPU path does (src/gpu/conv2d.cu:214-307) and is valid for SAME padding with both
back-ends.

Every function that runs convolutions is written as a Python generator: it yields
(operator name, algorithmic FLOPs) after each convolution and returns its result.  `run(gen)`
drives one to completion; the benchmark's CPU baseline instead advances it for a bounded time and
extrapolates from the FLOPs done (see bench.py).
"""
import numpy as np

G_CH = [512, 256, 128, 64, 3]
D_CH = [3, 64, 128, 256, 512]


def run(gen):
    """Drives a model generator to completion and returns its value."""
    try:
        while True:
            next(gen)
    except StopIteration as stop:
        return stop.value


def conv_flops(batch, out_hw, cin, cout):
    """Algorithmic FLOPs of a 5x5 convolution, its input gradient or its kernel gradient."""
    return 2.0 * batch * out_hw * out_hw * 25 * cin * cout


def iteration_flops(batch):
    """Convolution FLOPs of one whole training iteration (1 D update + 2 G updates)."""
    mid = sum(conv_flops(batch, 32 >> i, D_CH[i], D_CH[i + 1]) for i in range(4))  # one op per layer
    first = conv_flops(batch, 32, 3, 64)
    d_run = (mid                      # G forward
             + 2 * mid                # D forward on fake and real
             + 2 * mid                # kernel gradients, both passes
             + 2 * (mid - first))     # input gradients of layers 3..1, both passes
    g_run = 5 * mid   # G forward, D forward, D input gradients (4), G kernel gradients, G input gradients
    return d_run + 2 * g_run


def init_state(rng, batch):
    """Parameters ~ N(0, 0.02), zero biases, zero Adam moments.  Variable order of each network:
    (kernel, bias) of conv layers 0..3, dense weight, dense bias."""
    def w(*shape):
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)
    g = []
    for i in range(4):
        g += [w(5, 5, G_CH[i + 1], G_CH[i]), np.zeros(G_CH[i + 1], np.float32)]
    g += [w(100, 8192), np.zeros(8192, np.float32)]
    d = []
    for i in range(4):
        d += [w(5, 5, D_CH[i], D_CH[i + 1]), np.zeros(D_CH[i + 1], np.float32)]
    d += [w(8192, 1), np.zeros(1, np.float32)]
    zeros = lambda lst: [np.zeros_like(a) for a in lst]  # noqa: E731
    return {"g": g, "d": d, "g_m": zeros(g), "g_v": zeros(g), "d_m": zeros(d), "d_v": zeros(d),
            "g_t": 0.0, "d_t": 0.0, "batch": batch}


def generator_forward(be, g, z, g_leaky=False):
    act = (lambda a: be.vect_relu_leaky(a, 0.2)) if g_leaky else be.vect_relu
    B = z.shape[0]
    cache = {"z": z}
    cache["g0z"] = be.mat_mul_add(z, g[8], g[9])
    a = act(cache["g0z"]).reshape(B, 4, 4, 512)
    cache["in"], cache["gz"] = [], []
    for i in range(4):
        hw = 8 << i
        cache["in"].append(a)
        y = be.conv2d_transpose(a, g[2 * i], (B, hw, hw, G_CH[i + 1]), 2)
        yield "conv2d_transpose", conv_flops(B, hw // 2, G_CH[i + 1], G_CH[i])
        zi = be.mvrow_add(y, g[2 * i + 1])
        cache["gz"].append(zi)
        a = act(zi) if i < 3 else be.vect_tanh(zi)
    cache["g_out"] = a
    return a, cache


def discriminator_forward(be, d, img):
    B = img.shape[0]
    cache = {"in": [], "dz": []}
    a = img
    for i in range(4):
        cache["in"].append(a)
        y = be.conv2d(a, d[2 * i], (2, 2))
        yield "conv2d", conv_flops(B, 32 >> i, D_CH[i], D_CH[i + 1])
        zi = be.mvrow_add(y, d[2 * i + 1])
        cache["dz"].append(zi)
        a = be.vect_relu_leaky(zi, 0.2)
    cache["flat"] = a.reshape(B, 8192)
    logits = be.mat_mul_add(cache["flat"], d[8], d[9])
    return logits, cache


def discriminator_backward(be, d, cache, dlogits, want_weights, want_image):
    """Returns (weight gradients or None, image gradient or None)."""
    B = dlogits.shape[0]
    grads = [None] * 10
    if want_weights:
        grads[8] = be.tmm_mul(cache["flat"], dlogits)
        grads[9] = be.mat_sum_cols(dlogits)
    da = be.mtm_mul(dlogits, d[8]).reshape(B, 4, 4, 512)
    dimg = None
    for i in range(3, -1, -1):
        h = 64 >> i
        fl = conv_flops(B, h // 2, D_CH[i], D_CH[i + 1])
        dz = be.leaky_relu_grad(cache["dz"][i], da, 0.2)
        if want_weights:
            grads[2 * i + 1] = be.mat_sum_cols(dz)
            grads[2 * i] = be.conv2d_kernel_grad(dz, cache["in"][i], 2, (3, 3))
            yield "conv2d_kernel_grad", fl
        if i > 0:
            da = be.conv2d_input_grad(dz, d[2 * i], 2, (h, h))
            yield "conv2d_input_grad", fl
        elif want_image:
            dimg = be.conv2d_input_grad(dz, d[2 * i], 2, (h, h))
            yield "conv2d_input_grad", fl
    return (grads if want_weights else None), dimg


def d_gradients(be, st, x, z, g_leaky=False):
    """graph.run({d_opti, d_loss}) up to the update: returns (d_loss, gradients of the two paths)."""
    B = x.shape[0]
    ones, zeros = np.ones((B, 1), np.float32), np.zeros((B, 1), np.float32)
    g_out, _ = yield from generator_forward(be, st["g"], z, g_leaky)
    lf, cf = yield from discriminator_forward(be, st["d"], g_out)
    lr, cr = yield from discriminator_forward(be, st["d"], x)
    d1 = be.sigmoid_cross_entropy(zeros, lf)
    d2 = be.sigmoid_cross_entropy(ones, lr)
    gf, _ = yield from discriminator_backward(be, st["d"], cf, be.sigmoid_cross_entropy_grad(zeros, lf), True, False)
    gr, _ = yield from discriminator_backward(be, st["d"], cr, be.sigmoid_cross_entropy_grad(ones, lr), True, False)
    return np.float32(d1 + d2), gf, gr


def g_gradients(be, st, z, g_leaky=False):
    """graph.run({g_opti, g_loss}) up to the update: returns (g_loss, generator gradients)."""
    B = z.shape[0]
    ones = np.ones((B, 1), np.float32)
    g = st["g"]
    g_out, gc = yield from generator_forward(be, g, z, g_leaky)
    lf, cf = yield from discriminator_forward(be, st["d"], g_out)
    loss = be.sigmoid_cross_entropy(ones, lf)
    _, dimg = yield from discriminator_backward(be, st["d"], cf, be.sigmoid_cross_entropy_grad(ones, lf),
                                                False, True)
    dz = be.tanh_grad(g_out, dimg)
    act_grad = (lambda zz, dd: be.leaky_relu_grad(zz, dd, 0.2)) if g_leaky else be.relu_grad
    grads = [None] * 10
    for i in range(3, -1, -1):
        h = 4 << i
        fl = conv_flops(B, h, G_CH[i + 1], G_CH[i])
        grads[2 * i + 1] = be.mat_sum_cols(dz)
        # conv2d_transpose kernel gradient = conv2d kernel gradient with (dy, x) swapped
        grads[2 * i] = be.conv2d_kernel_grad(gc["in"][i], dz, 2, (3, 3))
        yield "conv2d_transpose_kernel_grad", fl
        # conv2d_transpose input gradient = strided conv2d of dz with the same kernel
        da = be.conv2d(dz, g[2 * i], (2, 2), pad=(3, 3), valid=True)
        yield "conv2d_transpose_input_grad", fl
        zprev = gc["g0z"].reshape(B, 4, 4, 512) if i == 0 else gc["gz"][i - 1]
        dz = act_grad(zprev, da)
    dz = dz.reshape(B, 8192)
    grads[8] = be.tmm_mul(gc["z"], dz)
    grads[9] = be.mat_sum_cols(dz)
    return np.float32(loss), grads


def apply_adam(be, params, grads, ms, vs, t, lr=2e-4, beta1=0.5, beta2=0.999, eps=1e-8):
    t_new = t
    for i in range(len(params)):
        p, m, v, t_new, _ = be.adam_step(params[i].reshape(-1), grads[i].reshape(-1), ms[i].reshape(-1),
                                         vs[i].reshape(-1), t, lr, beta1, beta2, eps)
        params[i], ms[i], vs[i] = p.reshape(params[i].shape), m.reshape(ms[i].shape), v.reshape(vs[i].shape)
    return t_new


def train_iteration(be, st, x, z, g_leaky=False):
    """One iteration in place on `st`; returns (d_loss, g_loss of the second generator update)."""
    d_loss, gf, gr = yield from d_gradients(be, st, x, z, g_leaky)
    grads = [be.vect_add(a.reshape(-1), b.reshape(-1)).reshape(a.shape) for a, b in zip(gf, gr)]
    st["d_t"] = apply_adam(be, st["d"], grads, st["d_m"], st["d_v"], st["d_t"])
    g_loss = None
    for _ in range(2):
        g_loss, gg = yield from g_gradients(be, st, z, g_leaky)
        st["g_t"] = apply_adam(be, st["g"], gg, st["g_m"], st["g_v"], st["g_t"])
    return d_loss, g_loss
