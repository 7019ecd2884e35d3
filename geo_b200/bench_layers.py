"""Single-layer SC forward benchmark (1 GPU): the layer configurations the reference's headline
numbers are quoted on, timed stage by stage with CUDA events.

    python -m geo_b200.bench_layers [--config NAME ...] [--batch B] [--reps R] [--no-peak]

Prints one JSON line per configuration: milliseconds of weight-stream generation, activation-stream
generation and accumulation, algorithmic LOP3/s of the accumulation kernel against the measured
LOP3 rate of the device, and SC bit-ops/s of the whole forward (2 * MAC * stream length).
``--batch`` shrinks the batch (for profiler captures of a small case).
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib, ops

# name: (act shape, weight shape, (pad_h, pad_w), L, mode, load_unit, load_wait, z_unit)
CONFIGS = {
    # single SC conv, the reference's CPU-runnable case
    "c1": ((32, 3, 32, 32), (32, 3, 5, 5), (2, 2), 64, "1d_bin", 8, 1, 1024),
    # the four layers of the 4-layer CNN at batch 256 (training defaults: L=128, load 2/2)
    "c2conv1": ((256, 3, 32, 32), (32, 3, 5, 5), (2, 2), 128, "1d_bin", 2, 2, 1024),
    "c2conv2": ((256, 32, 16, 16), (32, 32, 5, 5), (2, 2), 128, "1d_bin", 2, 2, 1024),
    "c2conv3": ((256, 32, 8, 8), (64, 32, 5, 5), (2, 2), 128, "1d_bin", 2, 2, 1024),
    "c2fc1": ((256, 64, 4, 4), (10, 64, 4, 4), (0, 0), 128, "1d_bin", 2, 2, 1024),
    # SC linear 1024x4096 . 4096x4096, OR in groups of 16, stream lengths 32..256
    "c3_L32": ((1024, 4096, 1, 1), (4096, 4096, 1, 1), (0, 0), 32, "yz_bin", 8, 1, 16),
    "c3_L64": ((1024, 4096, 1, 1), (4096, 4096, 1, 1), (0, 0), 64, "yz_bin", 8, 1, 16),
    "c3_L128": ((1024, 4096, 1, 1), (4096, 4096, 1, 1), (0, 0), 128, "yz_bin", 8, 1, 16),
    "c3_L256": ((1024, 4096, 1, 1), (4096, 4096, 1, 1), (0, 0), 256, "yz_bin", 8, 1, 16),
    # VGG-style 3x3 layer, the largest single-layer case: full OR vs partial binary
    "c4_full_or": ((256, 256, 16, 16), (256, 256, 3, 3), (1, 1), 256, "full_or", 8, 1, 1024),
    "c4_1d": ((256, 256, 16, 16), (256, 256, 3, 3), (1, 1), 256, "1d_bin", 8, 1, 1024),
    "c4_z": ((256, 256, 16, 16), (256, 256, 3, 3), (1, 1), 256, "z_bin", 8, 1, 1024),
    "c4_yz16": ((256, 256, 16, 16), (256, 256, 3, 3), (1, 1), 256, "yz_bin", 8, 1, 16),
    "c4_2d": ((256, 256, 16, 16), (256, 256, 3, 3), (1, 1), 256, "2d_bin", 8, 1, 1024),
    "c4_full_bin": ((256, 256, 16, 16), (256, 256, 3, 3), (1, 1), 256, "full_bin", 8, 1, 1024),
    # layers of the VGG-11-style network at 256 images (L=128, load 2/2)
    "c5conv1": ((256, 3, 32, 32), (64, 3, 3, 3), (1, 1), 128, "1d_bin", 2, 2, 1024),
    "c5conv2": ((256, 64, 16, 16), (128, 64, 3, 3), (1, 1), 128, "1d_bin", 2, 2, 1024),
    "c5conv4": ((256, 256, 8, 8), (256, 256, 3, 3), (1, 1), 128, "1d_bin", 2, 2, 1024),
    "c5conv6": ((256, 512, 4, 4), (512, 512, 3, 3), (1, 1), 128, "1d_bin", 2, 2, 1024),
    "c5conv8": ((256, 512, 2, 2), (512, 512, 3, 3), (1, 1), 128, "1d_bin", 2, 2, 1024),
    "c5fc1": ((256, 512, 1, 1), (512, 512, 1, 1), (0, 0), 128, "1d_bin", 2, 2, 1024),
}


def _q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


def _time(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(reps):
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def run_config(name, batch=None, reps=10, peak=None, device="cuda:0", guide=False, first_layer=False):
    ash, wsh, pad, L, mode, lu, lw, z = CONFIGS[name]
    if batch:
        ash = (batch,) + tuple(ash[1:])
    dev = torch.device(device)
    g = torch.Generator().manual_seed(0)
    a = _q7(torch.rand(*ash, generator=g)).to(dev)
    w = _q7(torch.rand(*wsh, generator=g) * 2 - 1).to(dev)
    kw = dict(z_unit=z, total_width=7, load_width=lu, load_wait_w=lw, load_wait_a=lw)
    d = ops.desc_for(a, w, L, mode, pad, **kw)
    lop3, nbytes = ops.algorithmic_work(d)
    wprep = ops.prepare_weights(w, d)
    astr = ops.generate_act_streams(a, d)
    out = ops.accumulate(astr, wprep, d)
    ws = torch.empty(_lib.size_query("geo_sc_conv2d_workspace_bytes", d), dtype=torch.uint8, device=dev)
    t_w = _time(lambda: ops.prepare_weights(w, d), reps)
    t_a = _time(lambda: ops.generate_act_streams(a, d), reps)
    t_c = _time(lambda: ops.accumulate(astr, wprep, d, out), reps)
    t_all = _time(lambda: ops.sc_conv2d(a, w, L, mode, pad, workspace=ws, out=out, **kw), reps)
    t_g = None
    if guide:
        go = torch.randn(ops.out_shape(d), generator=g).to(dev)
        # first_layer: what the first layer of a network asks for (no activation gradient, inputs
        # already quantised by the layer)
        t_g = _time(lambda: ops.guide_backward(a, w, go, d, need_act=not first_layer, quantized=first_layer), reps)
    rate = lop3 / (t_c * 1e-3)
    G, K, NT, Opad = _lib.group_geometry(d)
    executed = ops.executed_lop3(d)
    return {"config": name, "kernel": _lib.accumulate_kernel(d), "sign_sorted": bool(_lib.is_sign_sorted(d)),
            "executed_frac_of_lop3_peak": executed / (t_c * 1e-3) / peak if peak else None, "act": list(ash), "weight": list(wsh), "L": L, "mode": mode, "groups": G, "members": K,
            "ms_weight_streams": t_w, "ms_act_streams": t_a, "ms_accumulate": t_c, "ms_forward": t_all,
            "ms_guide_backward": t_g, "guide_tflops": (6 * lop3 / (2 * ((L + 31) // 32)) * 2 / (t_g * 1e-3) / 1e12) if t_g else None,
            "lop3": lop3, "tlop3_per_s": rate / 1e12, "frac_of_lop3_peak": rate / peak if peak else None,
            "sc_bitops_per_s": lop3 * 32 * (L / (32 * ((L + 31) // 32))) / (t_all * 1e-3),
            "hbm_gb_per_s": nbytes / (t_all * 1e-3) / 1e9}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", nargs="*", default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--no-peak", action="store_true")
    ap.add_argument("--guide", action="store_true", help="also time the fp32 guide backward (dgrad + wgrad)")
    ap.add_argument("--first-layer", action="store_true",
                    help="with --guide: weight gradient only, inputs promised quantised")
    a = ap.parse_args(argv)
    names = a.config or ["c1", "c2conv1", "c2conv2", "c2conv3", "c2fc1", "c4_1d", "c4_full_or"]
    peak = None
    if not a.no_peak:
        peak, _ = ops.measure_lop3_peak()
        print(json.dumps({"lop3_peak_per_s": peak, "lanes_per_clk_per_sm_at_1965MHz": peak / 148 / 1.965e9}))
    for n in names:
        print(json.dumps(run_config(n, a.batch, a.reps, peak, guide=a.guide, first_layer=a.first_layer)), flush=True)


if __name__ == "__main__":
    main()
