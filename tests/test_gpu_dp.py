"""Data-parallel training on 2 GPUs (NCCL): skipped below 2 devices.

The test launches this file as 2 ranks with torch.distributed.run.  Each rank checks, and fails its
process on a mismatch:
  * fp32 path: the rank gradients of the D run, summed over ranks through the communicator behind
    the C ABI (dcg_dp_allreduce) and divided by 2, equal a single-GPU D run on the concatenated
    batch (2e-5 * max) - the average of per-shard mean gradients is the global-batch gradient;
  * fp32 path, one whole iteration with the fused update (gradient sum + Adam + parameter broadcast as
    one kernel over peer memory, plain peer loads / stores, no multimem): the parameters agree with a
    single-GPU iteration on the concatenated batch up to Adam sign flips of rounding-level gradients;
  * TF32 path, 4 whole iterations (dcg_trainer_step, replayed as one CUDA graph from the third on):
    parameters are bit-identical on both ranks and differ from the initial ones - with the fused
    update, with NCCL all-reduce + replicated Adam behind the C ABI, and with the collectives issued
    by torch.distributed between the library's phases.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker():
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    pkg = entry.load_package()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda:%d" % int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    B = 4
    g = torch.Generator().manual_seed(99)
    x_all = torch.rand((world * B, 64, 64, 3), generator=g) * 2 - 1
    z_all = torch.rand((world * B, 100), generator=g) * 2 - 1
    xs, zs = x_all[rank * B:(rank + 1) * B], z_all[rank * B:(rank + 1) * B]

    # ---- averaged rank gradients = global-batch gradients (fp32 path) ----
    tr = pkg.Trainer(batch=B, precision=pkg.PREC_FP32, seed=234, world=world)
    assert tr.dp_info() is not None and tr.dp_info()[:2] == (rank, world)
    tr.x.copy_(xs)
    tr.z.copy_(zs)
    tr.d_backward()                      # world > 1: both gradient paths are summed into d_grads
    tr.allreduce(tr.d_grads)
    torch.cuda.synchronize()
    avg = (tr.d_grads / world).cpu()
    tr.close()
    if rank == 0:
        one = pkg.Trainer(batch=world * B, precision=pkg.PREC_FP32, seed=234, world=1)
        one.x.copy_(x_all)
        one.z.copy_(z_all)
        one.d_backward()
        torch.cuda.synchronize()
        ref = torch.cat([one.tensor("d_grad%d" % i) + one.tensor("d_gradb%d" % i) for i in range(10)]).cpu()
        one.close()
        got = torch.cat([avg[o:o + n] for o, n in _segments(pkg, B)])
        err = (got - ref).abs().max().item()
        assert err <= 2e-5 * ref.abs().max().item(), ("averaged gradients", err, ref.abs().max().item())

    # ---- one whole iteration, fused update (sum + Adam + broadcast as one kernel over peer memory), fp32 path,
    # against a single GPU on the concatenated batch: Adam's first steps move every weight by about lr in the
    # direction of its gradient's sign, so the two agree except where a gradient at rounding level changes sign ----
    tr = pkg.Trainer(batch=B, precision=pkg.PREC_FP32, seed=234, world=world)
    assert tr.dp_mode() == "fused", tr.dp_mode()
    tr.x.copy_(xs)
    tr.z.copy_(zs)
    tr.step()
    torch.cuda.synchronize()
    assert pkg.lib.dcg_device_status() == 0, pkg.lib.dcg_last_error()
    got = torch.cat([tr.tensor("d_params"), tr.tensor("g_params")]).cpu()
    tr.close()
    if rank == 0:
        one = pkg.Trainer(batch=world * B, precision=pkg.PREC_FP32, seed=234, world=1)
        one.x.copy_(x_all)
        one.z.copy_(z_all)
        one.step()
        torch.cuda.synchronize()
        ref = torch.cat([one.tensor("d_params"), one.tensor("g_params")]).cpu()
        one.close()
        diff = (got - ref).abs()
        assert diff.max().item() <= 1.3e-3, diff.max().item()          # at most a few flipped steps of lr = 2e-4
        assert (diff <= 1e-6).float().mean().item() >= 0.99, (diff <= 1e-6).float().mean().item()

    # ---- replicas stay bit-identical over whole iterations ----
    for comm, fused in (("abi", "1"), ("abi", "0"), ("torch", "1")):
        os.environ["DCG_DP_FUSED"] = fused
        tr = pkg.Trainer(batch=B, precision=pkg.PREC_TF32, seed=234, world=world, comm=comm)
        assert tr.dp_mode() == {("abi", "1"): "fused", ("abi", "0"): "nccl", ("torch", "1"): "none"}[(comm, fused)]
        start = torch.cat([tr.tensor("d_params"), tr.tensor("g_params")]).clone()
        tr.x.copy_(xs)
        tr.z.copy_(zs)
        for _ in range(4):
            tr.step()
        torch.cuda.synchronize()
        assert pkg.lib.dcg_device_status() == 0
        mine = torch.cat([tr.tensor("d_params"), tr.tensor("g_params")]).clone()
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        for other in both[1:]:
            assert torch.equal(both[0], other), "replicas differ (%s, fused %s)" % (comm, fused)
        assert not torch.equal(mine, start)
        assert torch.isfinite(mine).all()
        tr.close()
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


def _segments(pkg, B):
    """(offset, count) of the 10 discriminator variables inside the 256-byte-aligned gradient arena."""
    sizes = [25 * 3 * 64, 64, 25 * 64 * 128, 128, 25 * 128 * 256, 256, 25 * 256 * 512, 512, 8192, 1]
    out, off = [], 0
    for n in sizes:
        off = (off + 63) // 64 * 64
        out.append((off, n))
        off += n
    return out


@pytest.mark.gpu
def test_two_ranks_average_gradients_and_stay_identical(pkg, dev):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", os.path.abspath(__file__)],
                         env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "rank 0 ok" in res.stdout and "rank 1 ok" in res.stdout


if __name__ == "__main__":
    _worker()
