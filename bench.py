#!/usr/bin/env python
"""Benchmark of the DCGAN training iteration on the B200 convolution / Adam hot path.

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU code, host cores
    python bench.py --sweep                                   # per-layer conv roofline sweep

A step is one training iteration exactly as dcgan/main.cu:378-391 runs it - one discriminator
update and two generator updates, each recomputing its forward passes - at batch 64 per GPU
(weak scaling: N GPUs train 64*N images per step; gradients are averaged with one all-reduce
per update).  Inputs are synthetic with the data's shapes and ranges: images ~ U(-1,1)
[64,64,64,3], z ~ U(-1,1) [64,100], weights ~ N(0,0.02), seeded.

One JSON line is printed by rank 0:
  value      images/s over all GPUs, device-timed (CUDA events, max over ranks), inputs resident in HBM;
             the K steps are timed as a block, the block is repeated until at least a second of device
             time has been measured, and the median block is reported (blocks, min, max alongside)
  e2e        the same through Trainer.submit_host / result: every step's own pinned host -> device copies
             of its inputs and a device -> host read of both losses inside the timed region, the copies
             of step i+1 overlapping the compute of step i
  roofline   the tensor-path convolution kernel: algorithmic FLOPs / event-timed duration of its
             launches inside profiled steps, against the TF32 peak (half the measured dense bf16 peak)
  cpu_baseline  the reference's CPU code (oracle/_ref) on a bounded, FLOP-weighted sample of the same
             iteration at batch 1, one thread; plus, where the reference tree was built against this
             backend (dcgan-cuda_b200/shim), its MCPU mode (4 pool threads) on the generator forward
  gen_images_per_s / d_fwd_bwd_ms   BASELINE configs[0] (generator forward, leaky) and configs[1]
             (discriminator forward + backward on real images) at batch 64, device-timed
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH = 64
MIN_TIMED_S = 1.0   # device time measured at least, whatever --steps is
METRIC = "dcgan_train_images_per_s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    except (OSError, ValueError):
        p = dict(FALLBACK_PEAKS)
        p["_source"] = "fallback"
        return p


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: read-only NVML queries from a
    thread of this process every 10 ms (nvidia-smi every 100 ms where NVML cannot be imported)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # nvmlClocksEventReason bits: sw_power_cap 0x4, hw_slowdown 0x8, sw_thermal 0x20, hw_thermal 0x40
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.stop_flag = None
        self.sm, self.mx, self.reasons = [], [], set()

    def _nvml_index(self):
        """NVML enumerates all GPUs of the machine; CUDA_VISIBLE_DEVICES may remap the ordinals."""
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            parts = [p.strip() for p in vis.split(",") if p.strip()]
            if self.gpu < len(parts) and parts[self.gpu].isdigit():
                return int(parts[self.gpu])
        return self.gpu

    def start(self):
        try:
            import threading

            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._nvml_index())
            self.mx.append(float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)))
            self.stop_flag = threading.Event()

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        bits = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                        for name, bit in self.REASON_BITS.items():
                            if bits & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    self.stop_flag.wait(0.01)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                    "sm_min_mhz": min(self.sm) if self.sm else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                    "samples": len(self.sm), "reasons": sorted(self.reasons), "source": "nvml, 10 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        sm.append(float(parts[1]))
                        mx.append(float(parts[2]))
                    except ValueError:
                        continue
                    for name, val in zip(names, parts[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi, 100 ms"}


def synthetic_batches(rank, count):
    """`count` host batches of (images, z) ~ U(-1,1), pinned, seeded per rank (234 + rank)."""
    import torch
    g = torch.Generator().manual_seed(234 + rank)
    out = []
    for _ in range(count):
        x = (torch.rand((BATCH, 64, 64, 3), generator=g) * 2 - 1).pin_memory()
        z = (torch.rand((BATCH, 100), generator=g) * 2 - 1).pin_memory()
        out.append((x, z))
    return out


class CpuSampler:
    """The reference's CPU code on the batch-1 training iteration, advanced in bounded slices.

    advance(budget_s) runs the iteration's operator sequence from where the previous slice stopped
    for about budget_s seconds (it stops at a convolution boundary; finished iterations restart),
    and extrapolates images/s from the algorithmic convolution FLOPs done in the slice."""

    def __init__(self):
        import numpy as np
        import oracle
        from oracle import dcgan_model as M
        self.M = M
        self.be, self.kind = oracle.reference(), "reference"
        if self.be is None:
            self.be, self.kind = oracle.port(), "port"
        rng = np.random.default_rng(234)
        self.st = M.init_state(rng, 1)
        self.x = rng.uniform(-1, 1, (1, 64, 64, 3)).astype(np.float32)
        self.z = rng.uniform(-1, 1, (1, 100)).astype(np.float32)
        self.gen = None

    def advance(self, budget_s):
        M = self.M
        flops, ops = 0.0, 0
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < budget_s:
            if self.gen is None:
                self.gen = M.train_iteration(self.be, self.st, self.x, self.z)
            try:
                _, f = next(self.gen)
                flops += f
                ops += 1
            except StopIteration:
                self.gen = None
        elapsed = time.perf_counter() - t0
        per_image = M.iteration_flops(1)
        return {"value": (flops / per_image) / elapsed, "seconds": elapsed, "ops": ops, "kind": self.kind,
                "fraction_of_iteration": flops / per_image}


def mcpu_generator_baseline(mode="MCPU", batch=4):
    """BASELINE configs[0] (generator forward, leaky) through the reference's own ops graph in its
    RT_MODE=MCPU mode - rt::optimize + ThreadPoolRunner(4), src/ops/graph.cu:32,180-192 - on this box's
    host cores.  Needs the reference tree built against this repository's backend
    (dcgan-cuda_b200/shim/build_reference.py leaves the binary under shim/_ref_build/); None otherwise.
    The pool has 4 worker threads whatever the core count, and convolutions are not split across them
    (src/runtime/optimizer.cu:239-246), so the batch only scales the run time: a batch of 4 keeps the
    sample to seconds."""
    exe = os.path.join(ROOT, "dcgan-cuda_b200", "shim", "_ref_build", "bin", "dcgan_graph_driver")
    if not os.access(exe, os.X_OK):
        return None
    with tempfile.TemporaryDirectory() as tmp:
        t0 = time.perf_counter()
        try:
            res = subprocess.run([exe, "gen", str(batch), "1", os.path.join(tmp, "out.bin"), "leaky"], cwd=tmp,
                                 env=dict(os.environ, RT_MODE=mode), capture_output=True, text=True, timeout=600)
        except (OSError, subprocess.TimeoutExpired):
            return None
        wall = time.perf_counter() - t0
    if res.returncode != 0:
        return None
    try:
        ms = json.loads(res.stdout.strip().splitlines()[-1])["ms"][0]
    except (ValueError, KeyError, IndexError):
        return None
    return {"mode": mode, "workload": "configs[0]: generator forward through ops::Graph::run", "batch": batch,
            "images_per_s": batch / (ms * 1e-3), "run_ms": ms, "threads": 4 if mode == "MCPU" else 1,
            "nproc": os.cpu_count(), "wall_s": wall}


def run_reference(args, rank):
    """--impl reference: the reference's own CPU implementation of the iteration, host cores."""
    if rank != 0:
        return
    per_step = max(0.5, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    sampler = CpuSampler()
    for _ in range(args.warmup):
        sampler.advance(per_step)
    fracs, secs = [], []
    kind = sampler.kind
    for _ in range(args.steps):
        r = sampler.advance(per_step)
        fracs.append(r["fraction_of_iteration"])
        secs.append(r["seconds"])
    value = sum(fracs) / sum(secs) if secs else 0.0   # images per second over the whole timed run
    sample = ("per step ~%.1f s of the batch-1 iteration's convolution sequence (src/cpu/ops.hxx compiled "
              "-O2), images/s extrapolated by algorithmic FLOPs" % per_step)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(secs) if secs else None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[2]: full DCGAN training iteration (1 D update + 2 G updates), "
                               "batch 64 per GPU; CPU arm runs a bounded batch-1 sample", "global_batch": BATCH},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": 1, "kind": kind, "sample": sample,
                         "mcpu_cfg0": mcpu_generator_baseline("MCPU"), "cpu_cfg0": mcpu_generator_baseline("CPU")},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def profile_steps(pkg, trainer, steps):
    """Event-timed launch groups of `steps` iterations: rows of (name, calls, ms, flops)."""
    lib, L = pkg.lib, pkg._lib
    ctx = lib.dcg_trainer_context(trainer._h)
    L.check(lib.dcg_context_profile_begin(ctx))
    for _ in range(steps):
        trainer.step()
    rows = (L.ProfileRow * 256)()
    n = ctypes.c_int()
    L.check(lib.dcg_context_profile_end(ctx, rows, 256, ctypes.byref(n)))
    out = []
    for i in range(min(n.value, 256)):
        r = rows[i]
        out.append({"name": r.name.decode(), "calls": int(r.calls), "ms": r.ms, "flops": r.flops})
    return out


def run_ours(args, rank, local_rank, world):
    os.environ.setdefault("DCG_PROFILE_REPEAT", "4")   # read by the library when profiling starts
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda:%d" % local_rank)
    if world > 1:
        # NCCL_DEBUG=VERSION makes NCCL print its version banner on stdout, next to the JSON line
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, "launch with torchrun --nproc-per-node equal to --gpus"

    precision = {"tf32": pkg.PREC_TF32, "3xtf32": pkg.PREC_3XTF32, "fp32": pkg.PREC_FP32}[args.precision]
    trainer = pkg.Trainer(batch=BATCH, precision=precision, fuse=True, seed=234, world=world, comm=args.comm)
    batches = synthetic_batches(rank, 4)
    trainer.x.copy_(batches[0][0])
    trainer.z.copy_(batches[0][1])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing -------------------------------------------------------------
    # K steps between two CUDA events on the launching stream, barrier + synchronize on both sides, max
    # over ranks = one block.  Blocks are repeated until at least MIN_TIMED_S of device time has been
    # measured (a 20-step block is 30 ms: too short for the clocks to be sampled or to settle), and
    # the median block is the reported one.
    for _ in range(args.warmup):
        trainer.step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    block_ms, host_ms, launches = [], [], 0
    while True:
        barrier()
        launches0 = pkg.launches_total()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        h0 = time.perf_counter()
        for _ in range(args.steps):
            trainer.step()
        host_ms.append((time.perf_counter() - h0) * 1e3 / args.steps)   # host time to enqueue a step (no sync)
        e1.record()
        barrier()
        launches = pkg.launches_total() - launches0
        block_ms.append(max_over_ranks(e0.elapsed_time(e1)))
        if sum(block_ms) >= 1e3 * MIN_TIMED_S or len(block_ms) >= 200:
            break
    pkg._lib.check(pkg.lib.dcg_device_status())
    ms_total = statistics.median(block_ms)
    host_enqueue_ms = statistics.median(host_ms)
    ms_per_step = ms_total / args.steps
    value = world * BATCH / (ms_per_step * 1e-3)

    # ---- end to end: host inputs in, losses out, every step -------------------------------------
    for i in range(min(3, args.warmup)):
        trainer.step_host(*batches[i % len(batches)])
    barrier()
    # every step: its own pinned host -> device copy of images and z, the iteration, a device -> host
    # read of both losses; submitted back to back (the copies of step i+1 overlap the compute of step
    # i, as a data loader's prefetch does) and collected with a lag, so the timed region holds all of
    # it for all K steps
    t0 = time.perf_counter()
    losses = None
    lag = 8
    tickets = []
    for i in range(args.steps):
        tickets.append(trainer.submit_host(*batches[i % len(batches)]))
        if len(tickets) > lag:
            losses = trainer.result(tickets.pop(0))
    for tk in tickets:
        losses = trainer.result(tk)
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    # the same with the images as uint8 pixel values (what a JPEG decoder hands over): a quarter of the
    # host -> device bytes, the scaling to [-1, 1] done on the device as celeba::load does it on the host
    batches_u8 = [(((x + 1) * 127.5).clamp(0, 255).to(torch.uint8).pin_memory(), z) for x, z in batches]
    trainer.step_host(*batches_u8[0])
    barrier()
    t0 = time.perf_counter()
    tickets = []
    for i in range(args.steps):
        tickets.append(trainer.submit_host(*batches_u8[i % len(batches_u8)]))
        if len(tickets) > lag:
            trainer.result(tickets.pop(0))
    for tk in tickets:
        trainer.result(tk)
    torch.cuda.synchronize()
    e2e_u8_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    clocks = sampler.stop()
    if clocks.get("sm_mhz"):
        clocks["ms_per_step_x_sm_mhz"] = ms_per_step * clocks["sm_mhz"]
    e2e_value = world * BATCH * args.steps / e2e_s

    # ---- data parallel: replicas must have stayed bit-identical; what one gradient sum costs ----------
    dp_extra = {}
    if world > 1:
        params = torch.cat([trainer.tensor("d_params"), trainer.tensor("g_params")])
        # an order-independent 64-bit checksum of the parameter bits: min and max over ranks must agree
        bits = params.view(torch.int32).to(torch.int64)
        mine = torch.stack([bits.sum(), (bits * (torch.arange(bits.numel(), device=dev) % 1021 + 1)).sum()])
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        identical = bool(torch.equal(lo, hi))
        if not identical:
            raise SystemExit("rank %d: parameter replicas differ after the timed region" % rank)
        dp_extra["replicas_identical"] = identical
        us = {}
        for name, buf in (("d", trainer.d_grads), ("g", trainer.g_grads)):
            scratch = buf.clone()
            for _ in range(3):
                trainer.allreduce(scratch)
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with trainer._on_stream():
                a0.record()
            for _ in range(20):
                trainer.allreduce(scratch)
            with trainer._on_stream():
                a1.record()
            barrier()
            us[name] = 1e3 * max_over_ranks(a0.elapsed_time(a1)) / 20
        dp_extra["allreduce_us"] = us   # back to back, outside the timed region: an upper bound on what a step exposes
        dp_extra["allreduce_bytes"] = {"d": trainer.d_grads.numel() * 4, "g": trainer.g_grads.numel() * 4}
        info = trainer.dp_info()
        dp_extra["comm"] = ("communicator behind the C ABI (dcg_dp_*, NCCL %s); update = %s; whole iteration = one CUDA graph"
                            % (info[2], {"fused": "one kernel over peer memory (gradient sum + Adam + parameter broadcast)",
                                         "nccl": "ncclAllReduce + replicated Adam"}.get(trainer.dp_mode(), "?"))) if info \
            else "torch.distributed all_reduce between the library's phases"
        dp_extra["dp_mode"] = trainer.dp_mode()

    # ---- BASELINE configs[0] and configs[1] at batch 64 (device-timed, inputs resident) ---------------
    def timed(fn, reps):   # rank 0 only: no collective in here
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / reps
    extra_cfg = {}
    if rank == 0 and not args.no_extra_configs:
        d_ms = timed(trainer.d_fwd_bwd, 200)
        gen = pkg.Trainer(batch=BATCH, precision=precision, fuse=True, seed=234, world=1, g_leaky=True)
        gen.z.copy_(batches[0][1])
        g_ms = timed(gen.generate, 400)
        gen.close()
        # a second, separately named workload: the first G run of an iteration re-uses the generator forward
        # pass of the D run instead of recomputing it (same numbers, 5 launches fewer); never the headline
        sh = pkg.Trainer(batch=BATCH, precision=precision, fuse=True, seed=234, world=1, share_g_forward=True)
        sh.x.copy_(batches[0][0])
        sh.z.copy_(batches[0][1])
        s_ms = timed(sh.step, 300)
        sh.close()
        extra_cfg = {"gen_images_per_s": BATCH / (g_ms * 1e-3), "gen_ms": g_ms, "d_fwd_bwd_ms": d_ms,
                     "d_fwd_bwd_images_per_s": BATCH / (d_ms * 1e-3),
                     "shared_g_forward": {"ms_per_step": s_ms, "images_per_s": BATCH / (s_ms * 1e-3),
                                          "note": "not the benchmarked workload: dcgan/main.cu:378-391 recomputes"}}
    barrier()

    # ---- per-kernel view of the step (event-timed launch groups) --------------------------------
    peaks = read_peaks()
    traffic = read_ncu_traffic()
    # launch groups of three more steps, each between two CUDA events on the trainer's stream; a
    # convolution group is launched DCG_PROFILE_REPEAT times between its events (same operands, same
    # results) so that the pair measures device time per launch, not launch plus inter-kernel gap
    rows = profile_steps(pkg, trainer, 3)
    torch.cuda.synchronize()
    total_ms = sum(r["ms"] for r in rows) or 1.0
    conv = [r for r in rows if r["name"].startswith("conv_") and r["flops"] > 0]
    conv_ms = sum(r["ms"] for r in conv)
    conv_flops = sum(r["flops"] for r in conv)
    tf32_peak = peaks["bf16_tflops"] / 2.0
    achieved = conv_flops / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
    roofline = {
        "kernel": "conv_tc_kernel and its specialisations conv_dxf_kernel / conv_fwd_short_kernel / conv_dx3_kernel (tcgen05 implicit-GEMM "
                  "conv: fwd, dx, dk launch groups of the step, each timed over %s back-to-back launches)"
                  % os.environ.get("DCG_PROFILE_REPEAT", "1"),
        "bound": "tensor", "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
        "frac": achieved / tf32_peak if tf32_peak else None,
        "peak_source": "%s: dense bf16 %.1f TFLOP/s / 2 for TF32" % (peaks["_source"], peaks["bf16_tflops"]),
        "share_of_step": conv_ms / total_ms,
        # dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu capture summary
        "traffic": traffic.get("dram_bytes_per_launch_mean"), "traffic_source": traffic.get("source"),
    }
    kernels = sorted(rows, key=lambda r: -r["ms"])[:14]
    kernel_table = [{"name": r["name"], "calls_per_step": r["calls"] / 3.0, "us_per_call": 1e3 * r["ms"] / r["calls"],
                     "share": r["ms"] / total_ms,
                     "tflops": (r["flops"] / (r["ms"] * 1e-3) / 1e12) if r["flops"] > 0 and r["ms"] > 0 else None}
                    for r in kernels]

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = CpuSampler().advance(args.cpu_seconds)
        cpu = {"value": r["value"], "unit": "images/s", "cores": 1, "kind": r["kind"],
               "sample": "%.1f s (%d convolution calls, %.2f of one iteration) of the batch-1 training iteration, "
                         "images/s extrapolated by algorithmic FLOPs" % (r["seconds"], r["ops"],
                                                                        r["fraction_of_iteration"]),
               "mcpu_cfg0": mcpu_generator_baseline("MCPU")}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"tf32": "tf32", "3xtf32": "3xtf32", "fp32": "f32"}[args.precision], "data": "synthetic",
            "config": {"workload": "configs[2]: full DCGAN training iteration (1 D update + 2 G updates, forwards "
                                   "recomputed per update as dcgan/main.cu:378-391), batch 64 per GPU",
                       "global_batch": BATCH * world, "parallelism": "dp%d" % world,
                       "l2": "no flush: every step streams through the trainer's %.0f MB arena of activations, "
                             "gradients and Adam state, several times the 126 MB L2" % (trainer.arena_bytes() / 2 ** 20),
                       "adam": "lr 2e-4 beta1 0.5 beta2 0.999 eps 1e-8"},
            "steps_per_s": 1e3 / ms_per_step,
            "blocks": len(block_ms), "block_ms_min": min(block_ms), "block_ms_max": max(block_ms),
            "timed_s": sum(block_ms) * 1e-3,
            "conv_tflops": achieved,
            "host_enqueue_ms_per_step": host_enqueue_ms, "step_mode": trainer.step_mode(),
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": trainer.h2d_bytes_per_step,
                    "d2h_bytes_per_step": trainer.d2h_bytes_per_step, "losses_last": losses},
            "e2e_u8": {"value": world * BATCH * args.steps / e2e_u8_s, "unit": "images/s",
                       "h2d_bytes_per_step": trainer.h2d_bytes_per_step_u8, "d2h_bytes_per_step": trainer.d2h_bytes_per_step,
                       "note": "images as uint8 pixel values, decoded on the device"},
            "gpu_launches": launches,
            "gpu_launches_per_step": launches / args.steps,
            "roofline": roofline,
            "kernels": kernel_table,
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        line.update(extra_cfg)
        line.update(dp_extra)
        print(json.dumps(line))
    trainer.close()
    if world > 1:
        dist.destroy_process_group()


def read_ncu_traffic():
    """DRAM bytes per launch of the dominant kernel, from the summary committed with the ncu capture."""
    path = os.path.join(ROOT, "profiles", "conv_tc_kernel_D2_b64.json")
    try:
        with open(path) as f:
            d = json.load(f)
        per_mode = [m["dram_bytes_read"] + m["dram_bytes_write"] for m in d["modes"].values()]
        return {"dram_bytes_per_launch_mean": sum(per_mode) / len(per_mode), "source": "profiles/conv_tc_kernel_D2_b64.json: " + d["note"]}
    except (OSError, ValueError, KeyError, ZeroDivisionError):
        return {}


def cta_timeline(pkg):
    """Per-CTA phases of the last tensor-path launch (library built-in trace, DCG_TC_DEBUG=8): median / max
    over CTAs, in microseconds of the GPU's global timer."""
    import numpy as np
    buf = (ctypes.c_ulonglong * (1024 * 8))()
    pkg.lib.dcg_debug_cta_trace.argtypes = [ctypes.c_void_p]
    pkg.lib.dcg_debug_cta_trace.restype = ctypes.c_int
    pkg._lib.check(pkg.lib.dcg_debug_cta_trace(buf))
    a = np.frombuffer(buf, dtype=np.uint64).reshape(1024, 8).astype(np.int64)
    a = a[a[:, 0] > 0]
    if len(a) == 0:
        return None
    a = a[a[:, 0] > a[:, 0].max() - 500000]   # rows of earlier, larger grids are still in the buffer: last launch only
    rel = (a[:, :6] - a[:, 0].min()) / 1e3
    d = np.diff(rel, axis=1)
    out = {"ctas": int(len(a)), "sms": int(len(set(a[:, 6].tolist()))),
           "first_to_last_end": float(rel[:, 5].max()), "entry_max": float(rel[:, 0].max())}
    for i, nm in enumerate(["setup", "main_loop", "hand_over", "meet", "finish"]):
        out[nm] = {"median": float(np.median(d[:, i])), "max": float(d[:, i].max())}
    return out


def run_sweep(args):
    """Config 4: the eight DCGAN conv shapes x {fwd, dx, dk} x batch, isolated, L2 flushed."""
    import torch
    import __graft_entry__ as entry
    pkg = entry.load_package()
    F = pkg.functional
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    peaks = read_peaks()
    tf32_peak = peaks["bf16_tflops"] / 2.0
    flush = torch.empty(256 * 2 ** 20 // 4, device=dev)
    rows = []
    precs = {"tf32": pkg.PREC_TF32, "3xtf32": pkg.PREC_3XTF32, "fp32": pkg.PREC_FP32}
    for prec_name in args.sweep_precisions:
      prec = precs[prec_name]
      for B in args.sweep_batches:
        for name, H, C, O in (("D0/G3", 64, 3, 64), ("D1/G2", 32, 64, 128), ("D2/G1", 16, 128, 256),
                              ("D3/G0", 8, 256, 512)):
            if args.sweep_layers and name.split("/")[0] not in args.sweep_layers:
                continue
            x = torch.rand(B, H, H, C, device=dev) * 2 - 1
            k = torch.randn(5, 5, C, O, device=dev) * 0.02
            dy = torch.rand(B, H // 2, H // 2, O, device=dev) * 2 - 1
            y, dx, dk = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(k)
            flops = 2.0 * B * (H // 2) ** 2 * 25 * C * O
            # operand sets to rotate through for the back-to-back timing: together larger than L2
            n_sets = max(2, min(16, -(-(256 * 2 ** 20) // ((x.numel() + dy.numel()) * 4))))
            xs, dys = [x] + [x.clone() for _ in range(n_sets - 1)], [dy] + [dy.clone() for _ in range(n_sets - 1)]
            b2b = {"fwd": lambda i: F.conv2d_fwd(xs[i], k, out=y, precision=prec),
                   "dx": lambda i: F.conv2d_dx(dys[i], k, (H, H), out=dx, precision=prec),
                   "dk": lambda i: F.conv2d_dk(xs[i], dys[i], (5, 5), out=dk, precision=prec)}
            ops = (("fwd", lambda: F.conv2d_fwd(x, k, out=y, precision=prec)),
                   ("dx", lambda: F.conv2d_dx(dy, k, (H, H), out=dx, precision=prec)),
                   ("dk", lambda: F.conv2d_dk(x, dy, (5, 5), out=dk, precision=prec)))
            for op, fn in ops:
                if args.sweep_ops and op not in args.sweep_ops:
                    continue
                for _ in range(3):
                    fn()
                times = []
                for _ in range(args.sweep_iters):
                    flush.zero_()
                    s, t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    s.record()
                    fn()
                    t.record()
                    torch.cuda.synchronize()
                    times.append(s.elapsed_time(t))
                med = statistics.median(times)
                # back to back: n_calls launches between two events, operands rotating through the sets (so they
                # come from HBM, not L2), which takes the launch latency of an isolated call out of the figure
                n_calls = max(16, n_sets)
                reps = []
                for _ in range(5):
                    s, t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    s.record()
                    for i in range(n_calls):
                        b2b[op](i % n_sets)
                    t.record()
                    torch.cuda.synchronize()
                    reps.append(s.elapsed_time(t) / n_calls)
                bb = statistics.median(reps)
                tflops = flops / (bb * 1e-3) / 1e12
                rows.append({"precision": prec_name, "layer": name, "op": op, "batch": B, "us_isolated": med * 1e3,
                             "us": bb * 1e3, "tflops": tflops, "frac_tf32_peak": tflops / tf32_peak})
                if int(os.environ.get("DCG_TC_DEBUG", "0") or 0) & 8 and hasattr(pkg.lib, "dcg_debug_cta_trace"):
                    rows[-1]["cta_timeline_us"] = cta_timeline(pkg)
    pkg._lib.check(pkg.lib.dcg_device_status())
    print(json.dumps({"sweep": rows, "tf32_peak_tflops": tf32_peak, "peak_source": peaks["_source"],
                      "timing": "us: back to back - 16+ launches between two CUDA events, operands rotating through sets "
                                "that together exceed L2, median of 5; us_isolated: one launch between two events, median of "
                                "%d, 256 MB L2 flush before each (includes the launch latency)" % args.sweep_iters}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--precision", choices=["tf32", "3xtf32", "fp32"], default="tf32")
    ap.add_argument("--comm", choices=["abi", "torch"], default="abi",
                    help="N > 1: communicator behind the C ABI (default) or torch.distributed collectives")
    ap.add_argument("--sweep-precisions", nargs="+", default=["tf32"], choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-configs", action="store_true", help="skip the configs[0] / configs[1] timings")
    ap.add_argument("--cpu-seconds", type=float, default=20.0)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--sweep-batches", type=int, nargs="+", default=[64, 256, 1024])
    ap.add_argument("--sweep-iters", type=int, default=30)
    ap.add_argument("--sweep-layers", nargs="*", default=None, help="subset of D0 D1 D2 D3")
    ap.add_argument("--sweep-ops", nargs="*", default=None, help="subset of fwd dx dk")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.sweep:
        return run_sweep(args)
    if args.impl == "reference":
        return run_reference(args, rank)
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
