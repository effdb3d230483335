"""The reference's own programs, linked UNCHANGED against this repository's backend.

dcgan-cuda_b200/shim/build_reference.py compiles the reference's src/{api,cpu,memory,ops,runtime,
utils} where they lie, leaves out its src/gpu, and links its tests/test_*.cu, examples/nn_mnist.cu
and dcgan/main.cu with shim/b200_backend.cu (gpu::kernels_list / gpu::run over the C ABI,
src/gpu/kernels.cu:20-64, src/gpu/runner.cu:10-18).

CPU tests (need the reference checkout): everything links, and RT_MODE=CPU of the built programs
reproduces the committed golden vectors bit for bit (those came from the same CPU code through the
oracle's shim), which also checks the stand-in tensor archive both ways.

GPU tests (use the prebuilt binaries that travel with the repository): every program is run under
RT_MODE=CPU - the reference's own CPU implementation, the strongest oracle there is - and under
RT_MODE=GPU - this repository's kernels behind the reference's ops graph, autodiff, topological
sort and optimiser - and the saved tensors are compared.
"""
import importlib.util
import json
import os
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "dcgan-cuda_b200", "shim")


def _builder():
    spec = importlib.util.spec_from_file_location("dcgan_b200_build_reference", os.path.join(SHIM, "build_reference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_archive(path):
    """Reads the raw archive tocha/tensor.hh (the stand-in) writes."""
    b = open(path, "rb").read()
    assert b[:4] == b"DCGT"
    version, count = struct.unpack("<II", b[4:12])
    assert version == 1
    off, out = 12, []
    for _ in range(count):
        (rank,) = struct.unpack("<I", b[off:off + 4])
        off += 4
        dims = struct.unpack("<%dI" % rank, b[off:off + 4 * rank])
        off += 4 * rank
        n = int(np.prod(dims)) if rank else 1
        out.append(np.frombuffer(b, np.float32, n, off).reshape(dims).copy())
        off += 4 * n
    assert off == len(b)
    return out


def run_program(exe, mode, args, tmp, precision="tf32", fuse=1, timeout=900):
    env = dict(os.environ, RT_MODE=mode, DCG_SHIM_PRECISION=precision, DCG_SHIM_FUSE=str(fuse))
    res = subprocess.run([exe] + args, cwd=str(tmp), env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, "%s (RT_MODE=%s) failed:\n%s\n%s" % (exe, mode, res.stdout[-2000:], res.stderr[-2000:])
    return res.stdout


# ---- CPU: build + RT_MODE=CPU against the golden vectors ------------------------------------------------
@pytest.fixture(scope="module")
def built(pkg):
    b = _builder()
    if not os.path.isdir(os.path.join(b.default_reference(), "src", "ops")):
        pytest.skip("no reference checkout on this machine")
    return b.build()


def test_every_program_links_unchanged(built):
    b = _builder()
    assert set(built) == set(b.DEFAULT_PROGRAMS)
    for name in ("dcgan", "nn_mnist", "test_conv2d", "test_conv2d_transpose_grad", "test_adam_update"):
        assert os.access(built[name], os.X_OK), name


# program -> golden keys of its outputs, in the order its graph.run lists them
GOLDEN_OUTPUTS = {
    "test_conv2d": ["conv2d/y"],
    "test_conv2d_padding": ["conv2d_padding/y"],
    "test_conv2d_grad": ["conv2d_grad/dx", "conv2d_grad/dk", "conv2d_grad/dy_hat"],
    "test_conv2d_padding_grad": ["conv2d_padding_grad/dx", "conv2d_padding_grad/dk", "conv2d_padding_grad/dy_hat"],
    "test_conv2d_transpose": ["conv2d_transpose/y"],
    "test_conv2d_bias_add": ["conv2d_bias_add/out"],
    "test_conv2d_bias_add_grad": ["conv2d_bias_add_grad/dx", "conv2d_bias_add_grad/db", "conv2d_bias_add_grad/dy_hat"],
    "test_adam_update": ["adam_update/out"],
    "test_moment_update": ["moment_update/out"],
    "test_moment_update2": ["moment_update2/out"],
    "test_sigmoid_cross_entropy": ["sigmoid_cross_entropy/loss"],
    "test_argmax": ["argmax/acc"],
}


@pytest.mark.parametrize("prog", sorted(GOLDEN_OUTPUTS))
def test_cpu_mode_reproduces_golden(built, golden, tmp_path, prog):
    out = tmp_path / "out.bin"
    run_program(built[prog], "CPU", [str(out)], tmp_path)
    got = load_archive(str(out))
    for i, key in enumerate(GOLDEN_OUTPUTS[prog]):
        want = np.asarray(golden[key], dtype=np.float32)
        assert got[i].size == want.size, (prog, key)
        assert np.array_equal(got[i].reshape(-1), want.reshape(-1)), (prog, key)


def test_archive_reads_numpy_savez(built, tmp_path):
    """The stand-in archive reads what numpy.savez writes (how the reference's Python scripts hand
    inputs to its programs, tests/pyts/tensors_saver.py): fp32 and fp64 members, 0-d to 4-d."""
    rng = np.random.default_rng(3)
    arrs = [rng.standard_normal((2, 3, 4, 5)).astype(np.float32), rng.standard_normal((7,)),
            np.float32(2.5), rng.standard_normal((6, 1)).astype(np.float32)]
    npz, out = tmp_path / "in.npz", tmp_path / "out.bin"
    np.savez(str(npz), **{"obj_%06d" % i: a for i, a in enumerate(arrs)})
    run_program(built["archive_tool"], "CPU", [str(npz), str(out)], tmp_path)
    got = load_archive(str(out))
    assert len(got) == len(arrs)
    for g, a in zip(got, arrs):
        assert g.size == np.asarray(a).size
        assert np.array_equal(g.reshape(-1), np.asarray(a, dtype=np.float32).reshape(-1))
    out2 = tmp_path / "out2.bin"   # raw archive -> raw archive
    run_program(built["archive_tool"], "CPU", [str(out), str(out2)], tmp_path)
    assert open(str(out), "rb").read() == open(str(out2), "rb").read()


# ---- GPU: RT_MODE=CPU against RT_MODE=GPU ------------------------------------------------------------------
def _prebuilt():
    return _builder().built_programs()


BASIC_PROGRAMS = [
    "test_conv2d", "test_conv2d_padding", "test_conv2d_grad", "test_conv2d_padding_grad", "test_conv2d_transpose",
    "test_conv2d_transpose_grad", "test_conv2d_bias_add", "test_conv2d_bias_add_grad", "test_adam_update",
    "test_moment_update", "test_moment_update2", "test_sigmoid_cross_entropy", "test_sigmoid_cross_entropy_grad",
    "test_leaky_relu_grad", "test_tanh_grad", "test_relu_grad", "test_reshape", "test_argmax", "test_mat_mul_add",
    "test_softmax_cross_entropy_grad",
]


@pytest.mark.gpu
@pytest.mark.parametrize("prog", BASIC_PROGRAMS)
def test_reference_unit_program_cpu_vs_gpu(dev, tmp_path, prog):
    """The reference's unit-test programs (hand-typed inputs): the fp32 path is held to 5e-6 of the
    output's scale (conv / element-wise operators are bit-equal; reductions and transcendental
    functions differ in the last bits), the TF32 path to the 1e-2 of max|ref| bound."""
    progs = _prebuilt()
    if prog not in progs:
        pytest.skip("reference programs were not built (no reference checkout at build time)")
    cpu_out, gpu32, gputf = tmp_path / "cpu.bin", tmp_path / "gpu32.bin", tmp_path / "gputf.bin"
    run_program(progs[prog], "CPU", [str(cpu_out)], tmp_path)
    run_program(progs[prog], "GPU", [str(gpu32)], tmp_path, precision="fp32")
    run_program(progs[prog], "GPU", [str(gputf)], tmp_path, precision="tf32")
    ref = load_archive(str(cpu_out))
    for got, tol in ((load_archive(str(gpu32)), 5e-6), (load_archive(str(gputf)), 1e-2)):
        assert len(got) == len(ref)
        for r, g in zip(ref, got):
            scale = max(float(np.abs(r).max()), 1e-30)
            assert float(np.abs(g - r).max()) <= tol * scale, (prog, tol, float(np.abs(g - r).max()), scale)


@pytest.mark.gpu
def test_reference_conv_d1_batch64_cpu_vs_gpu(dev, tmp_path):
    """tests/test_conv_d1.cu: the 64 -> 128 discriminator layer at batch 64, inputs handed over as an
    .npz (numpy.savez) exactly as the reference's harness does; xorshift seed 234 inputs."""
    from conftest import seeded
    progs = _prebuilt()
    if "test_conv_d1" not in progs:
        pytest.skip("reference programs were not built")
    x = seeded((64, 32, 32, 64), 234)
    w = (seeded((5, 5, 64, 128), 235) * np.float32(0.05)).astype(np.float32)
    npz = tmp_path / "w.npz"
    np.savez(str(npz), obj_000000=x, obj_000001=w)
    outs = {}
    for tag, mode, prec in (("cpu", "CPU", "tf32"), ("fp32", "GPU", "fp32"), ("tf32", "GPU", "tf32")):
        out = tmp_path / (tag + ".bin")
        run_program(progs["test_conv_d1"], mode, ["-", str(npz), str(out)], tmp_path, precision=prec)
        (outs[tag],) = load_archive(str(out))
    assert np.array_equal(outs["fp32"], outs["cpu"])
    assert float(np.abs(outs["tf32"] - outs["cpu"]).max()) <= 1e-2 * float(np.abs(outs["cpu"]).max())


@pytest.mark.gpu
def test_generator_forward_through_reference_graph(dev, tmp_path):
    """BASELINE configs[0] through the reference's ops graph (batch 2 so that RT_MODE=CPU finishes in
    seconds): leaky generator, dense + 4 conv2d_transpose + tanh."""
    progs = _prebuilt()
    if "dcgan_graph_driver" not in progs:
        pytest.skip("reference programs were not built")
    outs = {}
    for tag, mode, prec in (("cpu", "CPU", "tf32"), ("mcpu", "MCPU", "tf32"), ("fp32", "GPU", "fp32"), ("tf32", "GPU", "tf32")):
        out = tmp_path / (tag + ".bin")
        run_program(progs["dcgan_graph_driver"], mode, ["gen", "2", "1", str(out), "leaky"], tmp_path, precision=prec)
        (outs[tag],) = load_archive(str(out))
    assert np.array_equal(outs["mcpu"], outs["cpu"])          # MCPU forward = CPU forward
    assert float(np.abs(outs["fp32"] - outs["cpu"]).max()) <= 2e-6   # tanh output, |.| <= 1
    assert float(np.abs(outs["tf32"] - outs["cpu"]).max()) <= 1e-2 * float(np.abs(outs["cpu"]).max())


@pytest.mark.gpu
def test_training_iteration_through_reference_graph(dev, tmp_path):
    """One full iteration of dcgan/main.cu:378-391 (D update, two G updates, Adam) at batch 1 driven by
    the reference's Graph::run, autodiff and AdamOptimizer: RT_MODE=CPU against RT_MODE=GPU.

    What is comparable: everything up to and including the first G run's loss - d_loss, the
    discriminator's Adam update, the generator / discriminator forward passes after it.  The
    generator's own gradients are not: the reference's CPU code evaluates conv2d_transpose_input_grad /
    conv2d_transpose_kernel_grad with zero padding (src/cpu/ops.hxx:808-902), which is the adjoint of
    its conv2d_transpose only without padding, while its GPU handlers - and this library - derive the
    padding from the sizes (src/gpu/conv2d.cu:229-236,281-288).  For the 5x5 SAME generator layers the
    reference's two modes therefore disagree with each other after the first generator update, and
    the second G run's loss and the generator's variables are only reported.

    fp32 path: losses to 1e-5; after one Adam step every discriminator weight has moved by about lr in
    the direction of its gradient's sign, so a sign flip of a near-zero gradient moves a weight by
    2 lr = 4e-4: the bound is 5e-4 absolute and 99.9 % of the entries within 1e-6.  TF32: losses 1e-2."""
    progs = _prebuilt()
    if "dcgan_graph_driver" not in progs:
        pytest.skip("reference programs were not built")
    outs = {}
    for tag, mode, prec in (("cpu", "CPU", "tf32"), ("fp32", "GPU", "fp32"), ("tf32", "GPU", "tf32")):
        out = tmp_path / (tag + ".bin")
        line = run_program(progs["dcgan_graph_driver"], mode, ["train", "1", "1", str(out), "relu"], tmp_path,
                           precision=prec, timeout=1500)
        json.loads(line.strip().splitlines()[-1])
        outs[tag] = load_archive(str(out))
    ref = outs["cpu"]
    assert len(ref) == 23
    report = {tag: {"d_loss": float(outs[tag][0][0]), "g_loss_first": float(outs[tag][22][0]), "g_loss_second": float(outs[tag][1][0]),
                    "param_maxdiff": [float(np.abs(g - r).max()) for r, g in zip(ref[2:22], outs[tag][2:22])]}
              for tag in outs}
    print("training iteration through the reference graph:", json.dumps(report))
    for tag, loss_tol in (("fp32", 1e-5), ("tf32", 1e-2)):
        got = outs[tag]
        for i in (0, 22):
            assert abs(float(got[i][0]) - float(ref[i][0])) <= loss_tol * max(1.0, abs(float(ref[i][0]))), (tag, i, report)
    for r, g in zip(ref[12:22], outs["fp32"][12:22]):   # the discriminator's 10 variables
        diff = np.abs(g - r)
        assert float(diff.max()) <= 5e-4, report
        assert float((diff <= 1e-6).mean()) >= 0.999, report
