"""DCGAN training step driver: thin Python over dcg_trainer (csrc/trainer.cu).

The C++ trainer owns the model (one device arena) and executes the node lists of
one training iteration.  This wrapper adds what lives above the C ABI:

* zero-copy torch views of the trainer's device tensors (inputs, losses,
  parameter and gradient arenas);
* the end-to-end step with HOST inputs: pinned host -> device copies of the real
  images and the noise, the iteration, a device -> host read of the two losses -
  blocking (step_host) or pipelined (submit_host / result: the copies of iteration
  i+1 overlap the compute of iteration i);
* data-parallel training: one process per GPU, each on its own 64-image shard;
  between *_backward and *_apply the gradient arena of the network being updated
  is summed over ranks with one all-reduce, and Adam divides by the world size.
  Replicas start from the same seed and apply identical updates, so parameters
  stay identical on every rank.  comm="abi" (the default): the NCCL communicator
  lives behind the C ABI (dcg_dp_*; torch.distributed only carries its 128-byte
  id to the ranks) and dcg_trainer_step runs the whole iteration - collectives
  included - as one CUDA graph.  comm="torch": the collectives are
  torch.distributed.all_reduce calls between the library's phases.
"""
import contextlib
import ctypes

import torch

from . import _lib
from ._lib import TrainerConfig, check, lib


class _CudaView:
    """Minimal __cuda_array_interface__ carrier so torch can wrap a raw device pointer."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False),
                                         "version": 3, "strides": None}


class Trainer:
    def __init__(self, batch=64, precision=_lib.PREC_TF32, fuse=True, g_leaky=False, lr=2e-4, beta1=0.5,
                 beta2=0.999, eps=1e-8, seed=234, world=1, device=None, process_group=None, comm="abi",
                 share_g_forward=False):
        self.device = torch.device(device if device is not None else "cuda:%d" % torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        self.batch, self.world, self.group = batch, world, process_group
        self.cfg = TrainerConfig(batch, world, precision, 1 if fuse else 0, 1 if g_leaky else 0, lr, beta1,
                                 beta2, eps, seed, 1 if share_g_forward else 0)
        self._h = ctypes.c_void_p()
        # The trainer replays its node lists as CUDA graphs, which cannot be captured on the legacy
        # default stream: when that is the caller's current stream the trainer works on a stream of its
        # own and every method orders itself against the caller's stream on entry and exit.
        caller = torch.cuda.current_stream(self.device)
        self._own_stream = caller.cuda_stream == 0
        # high priority: the library's side streams (weight / bias gradients) run at the default one, so
        # blocks of the critical path are scheduled first when both have work ready
        self.stream = torch.cuda.Stream(self.device, priority=-1) if self._own_stream else caller
        self._dp = ctypes.c_void_p()
        if world > 1 and comm == "abi":
            self._dp = self._make_communicator(world, process_group)
        check(lib.dcg_trainer_create_dp(ctypes.byref(self._h), ctypes.byref(self.cfg), self.stream.cuda_stream, self._dp))
        self._views = {}
        self.x = self.tensor("x").view(batch, 64, 64, 3)
        self.z = self.tensor("z").view(batch, 100)
        self.g_out = self.tensor("g_out").view(batch, 64, 64, 3)
        self.d_loss, self.g_loss = self.tensor("d_loss"), self.tensor("g_loss")
        self.d_grads, self.g_grads = self.tensor("d_grads"), self.tensor("g_grads")
        self._pipe = None   # staging of the end-to-end path, built on first use
        self._comm = None   # communication stream of the data-parallel step, built on first use

    def _make_communicator(self, world, group):
        """dcg_dp_init on every rank: rank 0 makes the NCCL id, torch.distributed broadcasts its bytes."""
        import torch.distributed as dist
        rank = dist.get_rank(group)
        ident = (ctypes.c_ubyte * _lib.DP_ID_BYTES)()
        if rank == 0:
            check(lib.dcg_dp_unique_id(ident))
        on_gpu = dist.get_backend(group) == "nccl"
        carrier = torch.tensor(list(ident), dtype=torch.uint8, device=self.device if on_gpu else "cpu")
        dist.broadcast(carrier, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        ident = (ctypes.c_ubyte * _lib.DP_ID_BYTES)(*carrier.cpu().tolist())
        dp = ctypes.c_void_p()
        check(lib.dcg_dp_init(ctypes.byref(dp), rank, world, ident))
        return dp

    def dp_info(self):
        """(rank, world, NCCL version) of the communicator behind the C ABI, or None."""
        if not self._dp:
            return None
        r, w, v = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        check(lib.dcg_dp_info(self._dp, ctypes.byref(r), ctypes.byref(w), ctypes.byref(v)))
        return r.value, w.value, v.value

    def allreduce(self, tensor):
        """In-place sum of a device tensor over the ranks on the trainer's stream (communicator behind
        the C ABI when there is one, else torch.distributed)."""
        if self.world == 1:
            return
        with self._on_stream():
            if self._dp:
                check(lib.dcg_dp_allreduce(self._dp, tensor.data_ptr(), tensor.numel(), self.stream.cuda_stream))
            else:
                torch.distributed.all_reduce(tensor, group=self.group)

    # ---- device tensors ------------------------------------------------------
    def tensor(self, name):
        """Zero-copy torch view (1-D, fp32) of a trainer tensor; see dcg_trainer_tensor for names."""
        if name not in self._views:
            ptr, n = ctypes.c_void_p(), ctypes.c_size_t()
            check(lib.dcg_trainer_tensor(self._h, name.encode(), ctypes.byref(ptr), ctypes.byref(n)))
            self._views[name] = torch.as_tensor(_CudaView(ptr.value, n.value), device=self.device)
        return self._views[name]

    def arena_bytes(self):
        return int(lib.dcg_trainer_arena_bytes(self._h))

    # ---- phases ----------------------------------------------------------------
    @contextlib.contextmanager
    def _on_stream(self):
        """Runs the body on the trainer's stream, after what the caller's stream has enqueued so far;
        the caller's stream then waits for the body."""
        if not self._own_stream:
            yield
            return
        caller = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(caller)
        with torch.cuda.stream(self.stream):
            yield
        caller.wait_stream(self.stream)

    def generate(self):
        with self._on_stream():
            check(lib.dcg_trainer_generate(self._h))
        return self.g_out

    def d_fwd_bwd(self):
        """Discriminator forward + backward on self.x against labels of ones (all layer gradients)."""
        with self._on_stream():
            check(lib.dcg_trainer_d_fwd_bwd(self._h))

    def d_backward(self):
        """G forward, D on fake and real, d_loss, D gradients (no update)."""
        with self._on_stream():
            check(lib.dcg_trainer_d_backward(self._h))

    def g_backward(self):
        """G forward, D on fake, g_loss, G gradients (no update)."""
        with self._on_stream():
            check(lib.dcg_trainer_g_backward(self._h))

    def _allreduce(self, grads):
        if self.world > 1:
            torch.distributed.all_reduce(grads, group=self.group)

    def _step(self):
        """Body of one iteration; runs with the trainer's stream current."""
        if self.world == 1 or self._dp:
            check(lib.dcg_trainer_step(self._h))   # the whole iteration, one CUDA graph once warmed up
            return
        # Data parallel: the discriminator's gradients are summed over ranks on a communication stream
        # while this stream already computes the generator's forward pass of the first G update, which
        # reads neither the discriminator's gradients nor its parameters.
        scale = 1.0 / self.world
        check(lib.dcg_trainer_d_backward(self._h))
        if self._comm is None:
            self._comm = torch.cuda.Stream(self.device)
        main = torch.cuda.current_stream(self.device)
        self._comm.wait_stream(main)
        with torch.cuda.stream(self._comm):
            self._allreduce(self.d_grads)
        check(lib.dcg_trainer_g_backward_part(self._h, 0))
        main.wait_stream(self._comm)
        check(lib.dcg_trainer_d_apply(self._h, scale))
        check(lib.dcg_trainer_g_backward_part(self._h, 1))
        self._allreduce(self.g_grads)
        check(lib.dcg_trainer_g_apply(self._h, scale))
        check(lib.dcg_trainer_g_backward(self._h))
        self._allreduce(self.g_grads)
        check(lib.dcg_trainer_g_apply(self._h, scale))

    def step(self):
        """One training iteration on inputs already resident in self.x / self.z."""
        with self._on_stream():
            self._step()

    # ---- end to end: host inputs in, losses out ---------------------------------------------
    _RING = 32   # iterations that may be in flight between submit_host and result

    def _pipeline(self):
        """Staging for submit_host, built on first use: two device slots for the inputs, filled by a
        copy stream while the previous iteration computes, and a ring of pinned loss pairs."""
        if getattr(self, "_pipe", None) is None:
            B, dev = self.batch, self.device
            self._pipe = {
                "copy": torch.cuda.Stream(dev),
                "xs": [torch.empty((B, 64, 64, 3), device=dev) for _ in range(2)],
                "zs": [torch.empty((B, 100), device=dev) for _ in range(2)],
                "hx": [torch.empty((B, 64, 64, 3)).pin_memory() for _ in range(2)],
                "xs8": [torch.empty((B, 64, 64, 3), dtype=torch.uint8, device=dev) for _ in range(2)],
                "hx8": [torch.empty((B, 64, 64, 3), dtype=torch.uint8).pin_memory() for _ in range(2)],
                "hz": [torch.empty((B, 100)).pin_memory() for _ in range(2)],
                "copied": [torch.cuda.Event() for _ in range(2)],    # slot's host -> device copy done
                "consumed": [torch.cuda.Event() for _ in range(2)],  # slot read by its iteration
                "loss": torch.empty((self._RING, 2)).pin_memory(),
                "done": [torch.cuda.Event() for _ in range(self._RING)],
                "n": 0,
            }
        return self._pipe

    def submit_host(self, x_host, z_host):
        """Enqueues one end-to-end iteration and returns a ticket for result(): the host -> device
        copy of x_host [B,64,64,3] and z_host [B,100] (HOST arrays; pinned torch tensors are copied
        from directly, anything else is staged through pinned memory first) runs on a copy stream
        and overlaps the iteration submitted before; the losses are read back into pinned memory.
        x_host may also hold uint8 pixel values: the bytes are copied as they are (a quarter of the
        traffic) and scaled to [-1, 1] on the device, bit for bit what celeba::load computes on the
        host (src/datasets/celeba.cu:29).  At most _RING iterations may be outstanding."""
        p = self._pipeline()
        n = p["n"]
        p["n"] = n + 1
        slot, ring = n % 2, n % self._RING
        if n >= self._RING:
            p["done"][ring].synchronize()   # the ring entry is about to be reused: its reader must have had its chance
        if n >= 2:
            p["consumed"][slot].synchronize()   # the slot's previous iteration has taken its inputs
        xh, zh = torch.as_tensor(x_host), torch.as_tensor(z_host)
        as_bytes = xh.dtype == torch.uint8
        if as_bytes:
            if not (xh.is_pinned() and xh.is_contiguous()):
                p["hx8"][slot].copy_(xh.reshape(p["hx8"][slot].shape))
                xh = p["hx8"][slot]
        elif not (xh.is_pinned() and xh.dtype == torch.float32 and xh.is_contiguous()):
            p["hx"][slot].copy_(xh.reshape(p["hx"][slot].shape))
            xh = p["hx"][slot]
        if not (zh.is_pinned() and zh.dtype == torch.float32 and zh.is_contiguous()):
            p["hz"][slot].copy_(zh.reshape(p["hz"][slot].shape))
            zh = p["hz"][slot]
        with torch.cuda.stream(p["copy"]):
            (p["xs8"] if as_bytes else p["xs"])[slot].copy_(xh.reshape(p["xs"][slot].shape), non_blocking=True)
            p["zs"][slot].copy_(zh.reshape(p["zs"][slot].shape), non_blocking=True)
            p["copied"][slot].record()
        with self._on_stream():
            self.stream.wait_event(p["copied"][slot])
            if as_bytes:   # decode on the device, straight into the trainer's input tensor
                check(lib.dcg_u8_to_unit(p["xs8"][slot].data_ptr(), self.x.data_ptr(), self.x.numel(), self.stream.cuda_stream))
            else:
                self.x.copy_(p["xs"][slot], non_blocking=True)   # device -> device, a few microseconds
            self.z.copy_(p["zs"][slot], non_blocking=True)
            p["consumed"][slot].record()
            self._step()
            p["loss"][ring, 0:1].copy_(self.d_loss, non_blocking=True)
            p["loss"][ring, 1:2].copy_(self.g_loss, non_blocking=True)
            p["done"][ring].record()
        return n

    def result(self, ticket):
        """(d_loss, g_loss) of the iteration submit_host returned `ticket` for; waits for it."""
        p = self._pipeline()
        assert p["n"] - self._RING <= ticket < p["n"], "ticket no longer (or not yet) in the ring"
        ring = ticket % self._RING
        p["done"][ring].synchronize()
        return float(p["loss"][ring, 0]), float(p["loss"][ring, 1])

    def step_host(self, x_host, z_host):
        """End-to-end iteration: x_host [B,64,64,3] and z_host [B,100] are HOST arrays (numpy or
        CPU torch); returns (d_loss, g_loss) as Python floats read back from the device."""
        return self.result(self.submit_host(x_host, z_host))

    # ---- checkpoints -----------------------------------------------------------------------------
    def save(self, path, wait=False):
        """Snapshot of variables, Adam moments and step counters; the file is written by a host thread
        while training continues (wait=True, save_wait() or the next save / load joins it)."""
        with self._on_stream():
            check(lib.dcg_trainer_save(self._h, str(path).encode()))
        if wait:
            self.save_wait()

    def save_wait(self):
        check(lib.dcg_trainer_save_wait(self._h))

    def load(self, path):
        with self._on_stream():
            check(lib.dcg_trainer_load(self._h, str(path).encode()))

    h2d_bytes_per_step = property(lambda self: self.batch * (64 * 64 * 3 + 100) * 4)
    h2d_bytes_per_step_u8 = property(lambda self: self.batch * (64 * 64 * 3 + 100 * 4))
    d2h_bytes_per_step = property(lambda self: 8)

    def step_mode(self):
        """'graph' once the whole iteration replays as one CUDA graph, 'warmup' before, 'eager' if capturing it failed."""
        return {2: "graph", 1: "warmup", 0: "eager"}.get(int(lib.dcg_trainer_step_mode(self._h)), "unknown")

    def dp_mode(self):
        """'fused' (sum + Adam + broadcast as one kernel over peer memory), 'nccl' (all-reduce + replicated Adam) or 'none'."""
        return {2: "fused", 1: "nccl", 0: "none"}.get(int(lib.dcg_trainer_dp_mode(self._h)), "unknown")

    def launches_per_step(self):
        return int(lib.dcg_trainer_step_launches(self._h))

    def close(self):
        """Releases the trainer.  Data parallel: collective - every rank calls it."""
        if self._h:
            self._views.clear()
            lib.dcg_trainer_destroy(self._h)
            self._h = ctypes.c_void_p()
        if getattr(self, "_dp", None):
            torch.cuda.synchronize(self.device)
            lib.dcg_dp_finalize(self._dp)
            self._dp = ctypes.c_void_p()

    def __del__(self):
        # A data-parallel trainer is torn down collectively (close() on every rank): never from the
        # garbage collector, where the ranks would not meet.  Process exit releases it anyway.
        try:
            if not getattr(self, "_dp", None):
                self.close()
        except Exception:
            pass
