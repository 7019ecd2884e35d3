#!/usr/bin/env python
"""Benchmark of the SC training hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--workload tiny_cnn|vgg11]

One "step" is one training step (SC forward through the CUDA library, backward through the
float guide, SGD on the fp32 master copy) of the 4-layer SC CNN on a synthetic batch of 256
images per GPU (uniform [0,1) 3x32x32 inputs, uniform labels, random-init weights, stream
length 128, 1d_bin, LFSR, load_unit = load_wait = 2).  For N > 1 launch with torchrun: one
process per GPU, gradients all-reduced with NCCL, per-GPU batch fixed (weak scaling).

Prints ONE JSON line (rank 0).  ``--impl reference`` times the reference's own CPU kernel for the
path (sc.cpp built unmodified) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

PER_GPU_BATCH = 256
BIT_LENGTH = 128


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
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


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

    net = build_model(args.workload, device)
    hook = GradientAllReduce(world) if world > 1 else None
    step = TrainStep(net, lr=2e-3, optim="SGD", grad_hook=hook, graph=not args.no_graph)

    B = PER_GPU_BATCH
    g = torch.Generator().manual_seed(1234 + rank)
    nbatch = 4  # rotate through a few batches; the per-step working set is far larger than L2
    host_x = [torch.rand(B, 3, 32, 32, generator=g).pin_memory() for _ in range(nbatch)]
    host_y = [torch.randint(0, 10, (B,), generator=g).pin_memory() for _ in range(nbatch)]
    dev_x = [x.to(device) for x in host_x]
    dev_y = [y.to(device) for y in host_y]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

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
    total_ms = timed(resident_step, args.steps)
    clocks = sampler.stop()
    e2e_ms = timed(e2e_step, args.steps)

    # roofline of the dominant kernel: the same step run eagerly (a graph replay cannot be bracketed
    # kernel by kernel) with CUDA events around every SC accumulate launch; the same pass counts the
    # launches of this library's kernels per step
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
    launches = ops.STATS.launches // nprof * args.steps
    lop3 = sum(r[0] for r in ops.STATS.records)
    lop3_executed = sum(r[4] for r in ops.STATS.records)
    nbytes = sum(r[1] for r in ops.STATS.records)
    acc_ms = sum(r[2].elapsed_time(r[3]) for r in ops.STATS.records)
    n_acc = max(len(ops.STATS.records), 1)

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
            "config": {"workload": f"{args.workload}: 4-layer SC CNN training step (conv3-32-32-64 5x5, fc 4x4), "
                                   f"batch {B}/GPU, L={BIT_LENGTH}, 1d_bin, lfsr, load 2/2, SGD"
                       if args.workload == "tiny_cnn" else
                       f"vgg11: VGG-11-style SC CNN training step, batch {B}/GPU, L={BIT_LENGTH}, 1d_bin, lfsr, SGD",
                       "per_gpu_batch": B, "global_batch": B * world, "parallelism": f"dp{world}",
                       "launch": "eager" if args.no_graph else ("whole step replayed as one CUDA graph" if world == 1 else
                                                             "two CUDA graphs per step (forward+backward, update) around the NCCL all-reduce"),
                       "l2": "per-step working set (activation streams, guide tensors) exceeds the 126 MB L2; "
                             "4 input batches rotated; no explicit flush"},
            "e2e": {"value": images / (e2e_ms * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": B * 3 * 32 * 32 * 4 + B * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "int_alu", "kernel": "geo::accumulate_sorted_kernel / geo::accumulate_kernel (SC AND/OR/popcount)",
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
                         "traffic": ACC_DRAM_BYTES_PER_LAUNCH if (args.workload == "tiny_cnn" and B == 256) else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, mean over the step's four "
                                           "accumulate launches (profiles/accumulate_kernel_cnn_layers_dram_traffic.md)",
                         "hbm": {"achieved": nbytes / (acc_ms * 1e-3) / 1e9 if acc_ms > 0 else 0.0, "peak": hbm_peak,
                                 "unit": "GB/s", "peak_source": how + " (MEASURED_PEAKS.json)"}},
        }
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(seconds=12.0)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return out


# DRAM bytes per accumulate launch of the default workload (4-layer CNN, 256 images), mean of the four
# layers' launches: 16.07 + 61.31 + 23.99 + 4.80 MB read, < 0.1 MB written (one ncu capture).
ACC_DRAM_BYTES_PER_LAUNCH = 26.54e6


def cpu_baseline(seconds=12.0, batch=64, min_steps=2):
    """Training step of the same model on the host cores with the reference's CPU kernel (or the
    C restatement when that build is absent), on a bounded sample: batches of ``batch`` images."""
    import oracle  # noqa: F401  (checker / CPU baseline only)
    from oracle.cpu_step import CpuTinyCNN

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    model = CpuTinyCNN(BIT_LENGTH)
    g = torch.Generator().manual_seed(7)
    x = torch.rand(batch, 3, 32, 32, generator=g)
    y = torch.randint(0, 10, (batch,), generator=g)
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
    rank, world, _ = _dist_env()
    if rank != 0:
        return None
    from oracle.cpu_step import CpuTinyCNN

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    batch = 64
    model = CpuTinyCNN(BIT_LENGTH)
    g = torch.Generator().manual_seed(7)
    x = torch.rand(batch, 3, 32, 32, generator=g)
    y = torch.randint(0, 10, (batch,), generator=g)
    for _ in range(max(1, min(args.warmup, 2))):
        model.step(x.clone(), y)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.step(x.clone(), y)
    dt = time.perf_counter() - t0
    v = args.steps * batch / dt
    sample = f"each step = one batch of {batch} images (of the 256-image batch) through the same model on the CPU"
    return {
        "impl": "reference", "metric": "SC-CNN train images/s", "value": v, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u32 AND/OR/popcount + f32 guide", "data": "synthetic",
        "config": {"workload": "tiny_cnn: 4-layer SC CNN training step, L=128, 1d_bin, lfsr, SGD", "sample": sample},
        "cpu_baseline": {"value": v, "unit": "images/s", "cores": cores, "kind": model.kind, "sample": sample},
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="tiny_cnn", choices=["tiny_cnn", "vgg11"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of one CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    out = run_reference(args) if args.impl == "reference" else run_native(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
