"""CPU-side checks of the DCGAN step restatement (oracle/dcgan_model.py) that anchors the trainer
parity tests: shapes, the gradient of the loss by finite differences, a loss that goes down, and the
FLOP bookkeeping the CPU baseline extrapolates with."""
import numpy as np

from oracle import dcgan_model as M


def test_shapes_and_finite_difference(orc):
    rng = np.random.default_rng(0)
    st = M.init_state(rng, 1)
    x = rng.uniform(-1, 1, (1, 64, 64, 3)).astype(np.float32)
    z = rng.uniform(-1, 1, (1, 100)).astype(np.float32)
    g_out, _ = M.run(M.generator_forward(orc, st["g"], z))
    assert g_out.shape == (1, 64, 64, 3) and np.abs(g_out).max() <= 1.0
    d_loss, gf, gr = M.run(M.d_gradients(orc, st, x, z))
    assert [g.shape for g in gf] == [p.shape for p in st["d"]]
    g_loss, gg = M.run(M.g_gradients(orc, st, z))
    assert [g.shape for g in gg] == [p.shape for p in st["g"]]
    # directional derivative of g_loss along the generator's last-layer kernel gradient
    k = st["g"][6]
    direction = gg[6] / np.linalg.norm(gg[6])
    eps = 1e-2
    st["g"][6] = k + eps * direction
    up, _ = M.run(M.g_gradients(orc, st, z))
    st["g"][6] = k - eps * direction
    down, _ = M.run(M.g_gradients(orc, st, z))
    st["g"][6] = k
    numeric = (float(up) - float(down)) / (2 * eps)
    analytic = float((gg[6] * direction).sum())
    assert abs(numeric - analytic) <= 0.05 * abs(analytic) + 1e-4


def test_training_and_flop_count(orc):
    rng = np.random.default_rng(1)
    st = M.init_state(rng, 1)
    x = rng.uniform(-1, 1, (1, 64, 64, 3)).astype(np.float32)
    z = rng.uniform(-1, 1, (1, 100)).astype(np.float32)
    # the generator yields the algorithmic FLOPs of each convolution it ran
    gen = M.train_iteration(orc, st, x, z)
    flops, ops = 0.0, 0
    try:
        while True:
            _, f = next(gen)
            flops += f
            ops += 1
    except StopIteration as stop:
        first, _ = stop.value
    assert ops == 4 + 8 + 8 + 6 + 2 * 20
    assert abs(flops - M.iteration_flops(1)) < 1e-6 * flops
    # 17 * (0.629 + 3 * 6.711) - 2 * 0.629 GFLOP per 64 images
    assert abs(M.iteration_flops(64) / 1e9 - 351.7) < 0.2
    for _ in range(2):
        last, _ = M.run(M.train_iteration(orc, st, x, z))
    assert float(last) < float(first)
    assert st["d_t"] == 3.0 and st["g_t"] == 6.0
