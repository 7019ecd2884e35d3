#!/usr/bin/env python
"""Benchmark of the SC training hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
                    [--skip-layers] [--skip-vgg] [--no-cpu-baseline] [--no-graph]

Headline: one "step" is one training step (SC forward through the CUDA library, backward through the
float guide, SGD on the fp32 master copy) of the 4-layer SC CNN on a synthetic batch of 256 images per
GPU (uniform [0,1) 3x32x32 inputs, uniform labels, random-init weights, stream length 128, 1d_bin,
LFSR, load_unit = load_wait = 2).  For N > 1 launch with torchrun: one process per GPU, gradients
all-reduced with NCCL, per-GPU batch fixed (weak scaling).  K steps are timed as one block between
barriers; the block is repeated until about a second of device time has been measured and the median
block is reported.

Two more blocks ride in the same JSON line:
* ``layers`` (1 GPU only): the single-layer configurations -- the 32x3x32x32 conv, the 1024x4096 linear layer at
  four stream lengths, the 256x256x16x16 3x3 layer in 1d_bin and full_or -- with SC bit-ops/s and the
  fraction of the measured LOP3 peak, and the reference's own CUDA kernel timed on the same GPU where its
  build is present;
* ``vgg11`` (every N): the VGG-11-style SC CNN at a global batch of 2048 images split evenly over the ranks
  (strong scaling), gradients averaged by a bucketed all-reduce that overlaps the backward pass.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the reference's own CPU kernel for the
path (sc.cpp built unmodified) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

PER_GPU_BATCH = 256
BIT_LENGTH = 128
VGG_GLOBAL_BATCH = 2048
# where the reference arm leaves its result for the native arm's cpu_baseline (same box, same run)
REFERENCE_ARM_CACHE = os.path.join(tempfile.gettempdir(), "geo_b200_reference_arm.json")


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80}
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._halt.wait(0.05)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def build_model(workload, device):
    from geo_b200 import network

    torch.manual_seed(0)
    if workload == "tiny_cnn":
        net = network.CONV_tiny_add_partial()
        net.err, net.z_unit, net.load_unit, net.load_wait = [7] * 4, [3, 3, 4, 4], [2] * 4, [2] * 4
    else:
        net = network.VGG11_add_partial()
    return net.to(device)


class Timer:
    """Blocks of steps between barriers, timed with CUDA events on the launching stream, maximum over ranks."""

    def __init__(self, device, dist):
        self.device, self.dist = device, dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def block(self, fn, steps):
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        self.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.device)
        if self.dist is not None:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def median_block(self, fn, steps, target_ms=1000.0, max_blocks=60):
        """Repeats the K-step block until ``target_ms`` of device time is covered; returns (median ms of a block,
        number of blocks).  Every rank takes the same number of blocks (decided from the all-reduced first one)."""
        first = self.block(fn, steps)
        n = int(min(max_blocks, max(1, math.ceil(target_ms / max(first, 1e-3)))))
        times = [first] + [self.block(fn, steps) for _ in range(n - 1)]
        times.sort()
        return times[len(times) // 2], len(times)


def count_library_kernels(fn):
    """Kernels of this library (namespace geo::) launched by ``fn()``, counted from a CUPTI trace; None where
    the tracer is unavailable (for instance under another profiler)."""
    if os.environ.get("GEO_BENCH_NO_TRACE"):
        return None
    try:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        n = 0
        for ev in prof.events():
            if "geo::" in ev.name:
                n += 1
        return n or None
    except Exception:
        return None


def run_native(args):
    from geo_b200 import ops
    from geo_b200.dp import GradientAllReduce
    from geo_b200.train import TrainStep

    rank, world, local = _dist_env()
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    ops._lib.lib()  # fail loudly if the CUDA library is missing
    timer = Timer(device, dist)

    net = build_model("tiny_cnn", device)
    hook = GradientAllReduce(world) if world > 1 else None
    step = TrainStep(net, lr=2e-3, optim="SGD", grad_hook=hook, graph=not args.no_graph)

    B = PER_GPU_BATCH
    g = torch.Generator().manual_seed(1234 + rank)
    nbatch = 4  # rotate through a few batches; the per-step working set is far larger than L2
    host_x = [torch.rand(B, 3, 32, 32, generator=g).pin_memory() for _ in range(nbatch)]
    host_y = [torch.randint(0, 10, (B,), generator=g).pin_memory() for _ in range(nbatch)]
    dev_x = [x.to(device) for x in host_x]
    dev_y = [y.to(device) for y in host_y]

    def resident_step(i):
        x = dev_x[i % nbatch]
        step(x.clone() if args.no_graph else x, dev_y[i % nbatch])

    losses = []

    def e2e_step(i):
        if args.no_graph:
            x = host_x[i % nbatch].to(device, non_blocking=True)
            y = host_y[i % nbatch].to(device, non_blocking=True)
        else:  # the pinned host batch is copied straight into the graph's input buffers
            x, y = host_x[i % nbatch], host_y[i % nbatch]
        loss, _ = step(x, y)
        losses.append(loss.item())  # device -> host read of the step's result

    for i in range(args.warmup):
        resident_step(i)
    sampler = ClockSampler(local)
    sampler.start()
    total_ms, nblocks = timer.median_block(resident_step, args.steps)
    clocks = sampler.stop()
    e2e_ms, e2e_blocks = timer.median_block(e2e_step, args.steps)

    # roofline of the dominant kernel: the same step run eagerly (a graph replay cannot be bracketed
    # kernel by kernel) with CUDA events around every SC accumulate launch
    eager = TrainStep(net, lr=2e-3, optim="SGD", grad_hook=hook, graph=False)
    for i in range(2):
        eager(dev_x[i % nbatch].clone(), dev_y[i % nbatch])
    ops.STATS.reset()
    ops.STATS.profile = True
    nprof = min(args.steps, 5)
    for i in range(nprof):
        eager(dev_x[i % nbatch].clone(), dev_y[i % nbatch])
    torch.cuda.synchronize()
    ops.STATS.profile = False
    bookkept = ops.STATS.launches // nprof
    lop3 = sum(r[0] for r in ops.STATS.records)
    lop3_executed = sum(r[4] for r in ops.STATS.records)
    nbytes = sum(r[1] for r in ops.STATS.records)
    acc_ms = sum(r[2].elapsed_time(r[3]) for r in ops.STATS.records)
    n_acc = max(len(ops.STATS.records), 1)
    traced = count_library_kernels(lambda: eager(dev_x[0].clone(), dev_y[0]))   # every rank: the step holds a collective
    per_step = traced if traced else bookkept

    vgg = None if args.skip_vgg else run_vgg11(device, rank, world, dist, timer)

    images = B * world * args.steps
    out = None
    if rank == 0:
        peak_lop3, _ = ops.measure_lop3_peak()
        hbm_peak, how = _peaks()
        achieved = lop3 / (acc_ms * 1e-3) if acc_ms > 0 else 0.0
        out = {
            "metric": "SC-CNN train images/s", "value": images / (total_ms * 1e-3), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32 AND/OR/popcount + f32 guide",
            "data": "synthetic",
            "config": {"workload": f"tiny_cnn: 4-layer SC CNN training step (conv3-32-32-64 5x5, fc 4x4), "
                                   f"batch {B}/GPU, L={BIT_LENGTH}, 1d_bin, lfsr, load 2/2, SGD",
                       "per_gpu_batch": B, "global_batch": B * world, "parallelism": f"dp{world}",
                       "launch": "eager" if args.no_graph else ("whole step replayed as one CUDA graph" if world == 1 else
                                                             "two CUDA graphs per step (forward+backward, update) around the NCCL all-reduce"),
                       "timing": f"median of {nblocks} blocks of {args.steps} steps (each block between barriers, CUDA events, "
                                 f"max over ranks); e2e: median of {e2e_blocks} blocks",
                       "l2": "per-step working set (activation streams, guide tensors) exceeds the 126 MB L2; "
                             "4 input batches rotated; no explicit flush"},
            "e2e": {"value": images / (e2e_ms * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": B * 3 * 32 * 32 * 4 + B * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": per_step * args.steps,
            "gpu_launches_source": ("kernels named geo::* in a CUPTI trace of one eager step" if traced else
                                    "per-call bookkeeping of the Python front end") + f": {per_step} per step",
            "clocks": clocks,
            "roofline": {"bound": "int_alu", "kernel": "geo::accumulate_rows_kernel (conv2, conv3) / geo::accumulate_short_kernel (conv1) / geo::accumulate_kernel (fc): SC AND/OR/popcount",
                         "achieved": achieved / 1e12, "peak": peak_lop3 / 1e12, "unit": "TLOP3/s",
                         "frac": achieved / peak_lop3 if peak_lop3 else None,
                         # achieved / frac use the definition's count (2 * MAC * packs).  The sign-sorted kernel
                         # issues one logic op per weight instead of two, so the ops it executes are fewer:
                         "executed_frac": (lop3_executed / (acc_ms * 1e-3)) / peak_lop3 if acc_ms > 0 and peak_lop3 else None,
                         "executed_over_algorithmic": lop3_executed / lop3 if lop3 else None,
                         # the other half of the headline metric: one LOP3 = 32 AND-multiplies with their accumulation
                         "sc_bitops_per_s": achieved * 32,
                         "peak_source": "measured live: unrolled independent LOP3 chains on all SMs",
                         "launches_timed": len(ops.STATS.records), "avg_launch_ms": acc_ms / n_acc,
                         "traffic": ACC_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the step's four "
                                           "accumulate launches (profiles/accumulate_kernel_cnn_layers_dram_traffic.md)",
                         "hbm": {"achieved": nbytes / (acc_ms * 1e-3) / 1e9 if acc_ms > 0 else 0.0, "peak": hbm_peak,
                                 "unit": "GB/s", "peak_source": how + " (MEASURED_PEAKS.json)"}},
        }
        if vgg is not None:
            out["vgg11"] = vgg
        if world == 1 and not args.skip_layers:
            out["layers"] = run_layers(peak_lop3)
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return out


# DRAM bytes per accumulate launch of the default workload (4-layer CNN, 256 images), mean of the four
# layers' launches: 16.07 + 61.35 + 24.04 + 4.80 MB read, < 0.1 MB written (one ncu capture).
ACC_DRAM_BYTES_PER_LAUNCH = 34.95e6


def run_vgg11(device, rank, world, dist, timer):
    """VGG-11-style SC CNN, global batch 2048 split evenly over the ranks: ms per step and images/s of the
    whole job, the bytes every rank all-reduces per step and how much of that exchange is not hidden behind
    the backward pass (step time with the collectives minus step time with the same packing but no
    collective).  Launched eagerly: at 256 or more images per GPU the step is far longer than its launches."""
    from geo_b200.dp import BucketedGradientAllReduce
    from geo_b200.train import TrainStep

    if VGG_GLOBAL_BATCH % world:
        return {"skipped": f"global batch {VGG_GLOBAL_BATCH} does not divide over {world} ranks"}
    B = VGG_GLOBAL_BATCH // world
    net = build_model("vgg11", device)
    params = list(net.parameters())
    hook = BucketedGradientAllReduce(params, world, bucket_bytes=4 << 20) if world > 1 else None
    step = TrainStep(net, lr=2e-3, optim="SGD", grad_hook=hook, graph=False)
    g = torch.Generator().manual_seed(4321 + rank)
    xs = [torch.rand(B, 3, 32, 32, generator=g).to(device) for _ in range(2)]
    ys = [torch.randint(0, 10, (B,), generator=g).to(device) for _ in range(2)]

    def one(i):
        step(xs[i % 2].clone(), ys[i % 2])

    for i in range(3):
        one(i)
    first = timer.block(one, 2) / 2
    steps = int(min(40, max(4, math.ceil(1000.0 / max(first, 1e-3)))))
    ms = timer.block(one, steps) / steps
    exposed = None
    if hook is not None:
        hook.collective = False
        timer.block(one, 2)
        ms_quiet = timer.block(one, steps) / steps
        hook.collective = True
        exposed = ms - ms_quiet
    out = {"workload": f"vgg11: VGG-11-style SC CNN (8 conv3x3 64..512, 3 fc as 1x1), global batch {VGG_GLOBAL_BATCH} "
                       f"split evenly = {B}/GPU, L={BIT_LENGTH}, 1d_bin, lfsr, load 2/2, SGD, eager launches",
           "n_gpus": world, "scaling": "strong", "per_gpu_batch": B, "steps_timed": steps, "ms_per_step": ms,
           "images_per_s": VGG_GLOBAL_BATCH / (ms * 1e-3),
           "allreduce_bytes_per_step": hook.bytes_per_step if hook is not None else 0,
           "allreduce_buckets": len(hook.buckets) if hook is not None else 0,
           "allreduce_exposed_ms": exposed}
    if hook is not None:
        hook.remove()
    del step, net, xs, ys
    torch.cuda.empty_cache()
    return out


def run_layers(peak_lop3):
    """Single-layer forward numbers on this GPU, and the reference's CUDA kernel beside them where it is built."""
    from geo_b200 import bench_layers

    rows = []
    for name in ("c1", "c3_L32", "c3_L64", "c3_L128", "c3_L256", "c4_1d", "c4_full_or"):
        r = bench_layers.run_config(name, reps=7, peak=peak_lop3)
        rows.append({"config": name, "mode": r["mode"], "L": r["L"], "ms_accumulate": r["ms_accumulate"],
                     "ms_forward": r["ms_forward"], "sc_bitops_per_s": r["sc_bitops_per_s"],
                     "frac": r["frac_of_lop3_peak"], "executed_frac": r["executed_frac_of_lop3_peak"],
                     "sign_sorted": r["sign_sorted"], "kernel": r["kernel"]})
        torch.cuda.empty_cache()
    return {"unit": "fraction of the measured LOP3 peak (definition: 2*MAC*packs logic ops per forward)",
            "rows": rows, "reference_gpu_kernel": reference_gpu_kernel()}


def reference_gpu_kernel():
    """The reference's own CUDA extension (sc_cuda.cpp + sc_cuda_kernel.cu built unmodified for sm_100a) on the
    single conv and on the second conv of the 4-layer CNN: its output must equal this library's before its time
    counts.  A baseline leg; absent build -> a note instead of numbers."""
    try:
        from oracle import ref_loader  # baseline leg only

        ext = ref_loader.ref_sc_extension_cuda()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference CUDA build could not be loaded: {type(e).__name__}"}
    if ext is None:
        return {"unavailable": "reference CUDA build is not present"}
    from geo_b200 import bench_layers, ops

    rows = []
    for name in ("c1", "c2conv2"):
        ash, wsh, pad, L, mode, lu, lw, _ = bench_layers.CONFIGS[name]
        g = torch.Generator().manual_seed(0)
        a = bench_layers._q7(torch.rand(*ash, generator=g)).cuda()
        w = bench_layers._q7(torch.rand(*wsh, generator=g) * 2 - 1).cuda()
        kw = dict(total_width=7, load_width=lu, load_wait_w=lw, load_wait_a=lw)
        mine = ops.sc_conv2d(a, w, L, mode, pad, **kw)

        def ref():
            # sc_cuda.cpp:47-63 pads the last dimension by padding[0] and dimension 2 by padding[1]
            return ext.conv2d_add_partial_variable_acc(a, w, L, (pad[1], pad[0]), (1, 1), 7, lu, lw, False, 2)

        y = ref()
        torch.cuda.synchronize()
        if not (int(y.abs().sum()) > 0 and torch.equal(y, mine)):
            rows.append({"config": name, "error": "reference kernel output differs from this library's"})
            continue
        ts = []
        for _ in range(3):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ref()
            torch.cuda.synchronize()
            ts.append((time.perf_counter() - t0) * 1e3)
        ours = bench_layers._time(lambda: ops.sc_conv2d(a, w, L, mode, pad, **kw), 5)
        rows.append({"config": name, "reference_gpu_kernel_ms": min(ts), "this_library_ms": ours,
                     "outputs_equal": True,
                     "timing": "host clock around the call with a device synchronise on both sides (the reference "
                               "allocates managed memory and launches on the legacy stream inside the call), best of 3"})
    return {"rows": rows}


def _cpu_model_and_sample(batch):
    from oracle.cpu_step import CpuTinyCNN  # CPU baseline leg only

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    model = CpuTinyCNN(BIT_LENGTH)
    g = torch.Generator().manual_seed(7)
    x = torch.rand(batch, 3, 32, 32, generator=g)
    y = torch.randint(0, 10, (batch,), generator=g)
    return model, x, y, cores


def cpu_baseline(seconds=12.0, batch=64, min_steps=2):
    """Training step of the same model on the host cores with the reference's CPU kernel (or the C restatement
    when that build is absent), on a bounded sample: batches of ``batch`` images.  When the reference arm
    (``--impl reference``) ran on this box within the last hour its measurement is reused instead of timing
    the same thing twice."""
    try:
        with open(REFERENCE_ARM_CACHE) as f:
            cached = json.load(f)
        if time.time() - cached["when"] < 3600:
            c = dict(cached["cpu_baseline"])
            c["sample"] += " [measured by the reference arm of this run, not repeated]"
            return c
    except Exception:  # noqa: BLE001
        pass
    model, x, y, cores = _cpu_model_and_sample(batch)
    model.step(x.clone(), y)  # warm-up
    n, t0 = 0, time.perf_counter()
    while n < min_steps or time.perf_counter() - t0 < seconds:
        model.step(x.clone(), y)
        n += 1
    dt = time.perf_counter() - t0
    return {"value": n * batch / dt, "unit": "images/s", "cores": cores, "kind": model.kind,
            "sample": f"{n} steps of batch {batch} of the same model (CPU SC forward without progressive loading, "
                      f"which the reference's CPU kernel does not implement)"}


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores.  One step = the headline's batch of 256
    images, fed as four micro-batches of 64 (each with its own optimiser step, as the reference's loop does for
    batches of 64); the whole run is bounded to a few minutes."""
    rank, world, _ = _dist_env()
    if rank != 0:
        return None
    micro, per_step = 64, PER_GPU_BATCH // 64
    model, x, y, cores = _cpu_model_and_sample(micro)
    for _ in range(max(1, min(args.warmup, 2))):
        model.step(x.clone(), y)
    budget = 150.0   # seconds for the timed steps; the step count is cut if one step is too slow for K of them
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        for _ in range(per_step):
            model.step(x.clone(), y)
        done += 1
        if time.perf_counter() - t0 > budget:
            break
    dt = time.perf_counter() - t0
    v = done * PER_GPU_BATCH / dt
    sample = (f"{done} steps; each step = {PER_GPU_BATCH} images as {per_step} micro-batches of {micro} through the same "
              f"model on the CPU (sc.cpp has no progressive loading: load_unit 8 instead of 2)")
    cpu = {"value": v, "unit": "images/s", "cores": cores, "kind": model.kind, "sample": sample}
    try:
        with open(REFERENCE_ARM_CACHE, "w") as f:
            json.dump({"when": time.time(), "cpu_baseline": cpu}, f)
    except OSError:
        pass
    return {
        "impl": "reference", "metric": "SC-CNN train images/s", "value": v, "unit": "images/s", "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": dt / done * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u32 AND/OR/popcount + f32 guide", "data": "synthetic",
        "config": {"workload": f"tiny_cnn: 4-layer SC CNN training step (conv3-32-32-64 5x5, fc 4x4), "
                               f"batch {PER_GPU_BATCH}/GPU, L={BIT_LENGTH}, 1d_bin, lfsr, load 2/2, SGD",
                   "per_gpu_batch": PER_GPU_BATCH, "sample": sample},
        "cpu_baseline": cpu,
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--skip-layers", action="store_true", help="leave out the single-layer block")
    ap.add_argument("--skip-vgg", action="store_true", help="leave out the VGG-11 (global batch 2048) block")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of one CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    out = run_reference(args) if args.impl == "reference" else run_native(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
