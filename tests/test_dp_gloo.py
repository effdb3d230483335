"""Data-parallel bookkeeping at world size 2 on CPU (gloo), with the oracle model standing in for
the GPU kernels: each rank computes the discriminator gradients of its own shard, the contiguous
gradient arena is summed with one all_reduce, Adam scales by 1/world - exactly the sequence
Trainer.step runs on GPUs (d_backward, all_reduce(d_grads), d_apply(1/N)).

Checked: the averaged gradients equal the gradients of the global batch computed in one process
(the losses are batch means, src/cpu/ops.hxx:451,458), and after the update every rank holds the
same parameters."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _shard(rank):
    rng = np.random.default_rng(234 + rank)   # data seed per rank, as bench.py does
    x = rng.uniform(-1, 1, (1, 64, 64, 3)).astype(np.float32)
    z = rng.uniform(-1, 1, (1, 100)).astype(np.float32)
    return x, z


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import oracle
    from oracle import dcgan_model as M
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    be = oracle.port()
    st = M.init_state(np.random.default_rng(7), 1)          # identical weights on every rank
    x, z = _shard(rank)
    _, gf, gr = M.run(M.d_gradients(be, st, x, z))
    # the two gradient paths are summed before the exchange (trainer.cu: world > 1)
    local = [be.vect_add(a.reshape(-1), b.reshape(-1)) for a, b in zip(gf, gr)]
    arena = torch.from_numpy(np.concatenate(local))          # one contiguous buffer per network
    dist.all_reduce(arena, op=dist.ReduceOp.SUM)             # ONE collective per update
    scale = np.float32(1.0 / world)
    sizes = [g.size for g in local]
    grads, off = [], 0
    for n, ref in zip(sizes, local):
        grads.append((arena[off:off + n].numpy() * scale).astype(np.float32))
        off += n
    shaped = [g.reshape(p.shape) for g, p in zip(grads, st["d"])]
    st["d_t"] = M.apply_adam(be, st["d"], shaped, st["d_m"], st["d_v"], st["d_t"])
    params = np.concatenate([p.reshape(-1) for p in st["d"]])
    # every rank must hold bit-identical parameters after the replicated update
    mine = torch.from_numpy(params.copy())
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    same = all(torch.equal(gathered[0], g) for g in gathered)
    if rank == 0:
        np.savez(os.path.join(out_dir, "rank0.npz"), grads=np.concatenate(grads), same=np.array(same))
    dist.destroy_process_group()


def test_two_rank_average_equals_global_batch(tmp_path, orc):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.load(os.path.join(str(tmp_path), "rank0.npz"))
    assert bool(got["same"]), "replicas diverged after the replicated Adam update"
    # the same update computed in one process on the global batch of 2
    from oracle import dcgan_model as M
    st = M.init_state(np.random.default_rng(7), 2)
    xs, zs = zip(*[_shard(r) for r in range(world)])
    _, gf, gr = M.run(M.d_gradients(orc, st, np.concatenate(xs), np.concatenate(zs)))
    ref = np.concatenate([(a + b).reshape(-1) for a, b in zip(gf, gr)])
    scale = np.abs(ref).max()
    assert np.abs(got["grads"] - ref).max() <= 2e-5 * scale
