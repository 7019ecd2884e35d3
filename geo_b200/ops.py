"""Torch-tensor front end of the C ABI (``include/geo_sc.h``), through ctypes.

Every function takes CUDA tensors, runs on torch's current stream and raises if the native
library is missing or reports an error.  There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import MODES, ConvDesc, check, make_desc  # noqa: F401


class _Stats:
    """Launch accounting for the benchmark: ``launches`` counts kernels of this library enqueued
    since the last reset; with ``profile`` on, every accumulate launch is bracketed by CUDA events
    on the launching stream and recorded as (algorithmic LOP3 count, algorithmic bytes, start, end)."""

    def __init__(self):
        self.launches = 0
        self.profile = False
        self.records = []

    def reset(self):
        self.launches = 0
        self.records = []


STATS = _Stats()


def algorithmic_work(desc):
    """(LOP3 count, HBM bytes) of one SC forward by definition: 2*MAC*packs 32-bit logic ops, and
    fp32 activations + fp32 weights in, int32 counts out."""
    B, O, Ho, Wo = out_shape(desc)
    mac = B * O * Ho * Wo * desc.c_in * desc.k_h * desc.k_w
    packs = (desc.bit_length + 31) // 32
    nbytes = 4 * (desc.batch * desc.c_in * desc.h_in * desc.w_in + O * desc.c_in * desc.k_h * desc.k_w
                  + B * O * Ho * Wo)
    return 2 * mac * packs, nbytes


def live_tap_fraction(desc):
    """Fraction of the (output pixel, filter tap) pairs whose input pixel lies inside the unpadded image: the
    rest meets the all-zero streams of the padding, which the tap-tile kernel skips."""
    def axis(n, pad, k):
        out = n + 2 * pad - k + 1
        live = sum(1 for o in range(out) for t in range(k) if 0 <= o + t - pad < n)
        return live / float(out * k)
    return axis(desc.h_in, desc.pad_h, desc.k_h) * axis(desc.w_in, desc.pad_w, desc.k_w)


def executed_lop3(desc):
    """32-bit logic ops the accumulation kernel actually issues for the OR accumulation: the definition's
    count for the dense kernel, at most half of it for the sign-sorted kernels (one op per weight instead of
    one per weight and polarity; members whose four weights are all zero are skipped on top of that), and of
    that half only the taps inside the image for the tap-tile kernel (at batch sizes that fill a tile with one
    border class; smaller batches skip less)."""
    lop3, _ = algorithmic_work(desc)
    if not _lib.is_sign_sorted(desc):
        return lop3
    if _lib.accumulate_kernel(desc) == "sorted_taps":
        return int(lop3 // 2 * live_tap_fraction(desc))
    return lop3 // 2


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("geo_b200 SC kernels run on CUDA tensors only (there is no CPU path)")


def desc_for(act, weight, bit_length, mode="1d_bin", padding=(0, 0), **kw):
    """Descriptor for ``act`` [B,C,H,W] and ``weight`` [O,C,K2,K3]; ``padding`` = (pad_h, pad_w)."""
    B, C, H, W = act.shape
    O, C2, K2, K3 = weight.shape
    if C != C2:
        raise ValueError(f"channel mismatch: input has {C}, weight has {C2}")
    return make_desc(B, C, H, W, O, K2, K3, bit_length, mode, pad_h=int(padding[0]), pad_w=int(padding[1]), **kw)


def out_shape(desc):
    return (desc.batch, desc.c_out, desc.h_in + 2 * desc.pad_h - desc.k_h + 1,
            desc.w_in + 2 * desc.pad_w - desc.k_w + 1)


def sc_conv2d(act, weight, bit_length, mode="1d_bin", padding=(0, 0), workspace=None, out=None, **kw):
    """SC conv2d forward -> int32 [B,O,Ho,Wo] (positive minus negative bit counts)."""
    _require_cuda(act, weight)
    a = act.detach().to(torch.float32).contiguous()
    w = weight.detach().to(torch.float32).contiguous()
    d = desc_for(a, w, bit_length, mode, padding, **kw)
    nbytes = _lib.size_query("geo_sc_conv2d_workspace_bytes", d)
    with torch.cuda.device(a.device):
        if workspace is None or workspace.numel() < nbytes:
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=a.device)
        if out is None:
            out = torch.empty(out_shape(d), dtype=torch.int32, device=a.device)
        check(_lib.lib().geo_sc_conv2d_forward(ctypes.byref(d), a.data_ptr(), w.data_ptr(), out.data_ptr(),
                                               workspace.data_ptr(), workspace.numel(), _stream_ptr(a.device)),
              "geo_sc_conv2d_forward")
    STATS.launches += 3
    return out


def sc_conv2d_staged(act, weight, bit_length, mode="1d_bin", padding=(0, 0), wprep=None, astreams=None, **kw):
    """Same result as :func:`sc_conv2d` through the three stage entry points; ``wprep`` may hold
    weight streams prepared earlier for the same weights and descriptor geometry, ``astreams`` the
    activation streams of ``act`` for this descriptor (the fused layer epilogue of the previous layer
    produces them)."""
    _require_cuda(act, weight)
    d = desc_for(act, weight, bit_length, mode, padding, **kw)
    if wprep is None:
        wprep = prepare_weights(weight, d)
    if astreams is None:
        astreams = generate_act_streams(act, d)
    if STATS.profile:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream(act.device))
        out = accumulate(astreams, wprep, d)
        e1.record(torch.cuda.current_stream(act.device))
        STATS.records.append(algorithmic_work(d) + (e0, e1, executed_lop3(d)))
        return out
    return accumulate(astreams, wprep, d)


def sc_linear(act, weight, bit_length, z_unit=16, **kw):
    """SC linear forward: act [B,F], weight [O,F] -> int32 [B,O]; OR inside groups of ``z_unit``
    inputs, binary accumulation across groups."""
    _require_cuda(act, weight)
    a = act.detach().to(torch.float32).contiguous()
    w = weight.detach().to(torch.float32).contiguous()
    B, F = a.shape
    O, F2 = w.shape
    if F != F2:
        raise ValueError("feature mismatch")
    d = make_desc(B, F, 1, 1, O, 1, 1, bit_length, "yz_bin", z_unit=z_unit, **kw)
    nbytes = _lib.size_query("geo_sc_conv2d_workspace_bytes", d)
    with torch.cuda.device(a.device):
        ws = torch.empty(nbytes, dtype=torch.uint8, device=a.device)
        out = torch.empty((B, O), dtype=torch.int32, device=a.device)
        check(_lib.lib().geo_sc_linear_forward(ctypes.byref(d), a.data_ptr(), w.data_ptr(), out.data_ptr(),
                                               ws.data_ptr(), ws.numel(), _stream_ptr(a.device)),
              "geo_sc_linear_forward")
    STATS.launches += 3
    return out


def prepare_weights(weight, desc):
    """Packed weight streams + activation offset table as one uint8 buffer (layout in geo_sc.h)."""
    _require_cuda(weight)
    w = weight.detach().to(torch.float32).contiguous()
    nbytes = _lib.size_query("geo_sc_weight_prep_bytes", desc)
    with torch.cuda.device(w.device):
        buf = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
        check(_lib.lib().geo_sc_prepare_weights(ctypes.byref(desc), w.data_ptr(), buf.data_ptr(), nbytes,
                                                _stream_ptr(w.device)), "geo_sc_prepare_weights")
    STATS.launches += 1
    return buf


def generate_act_streams(act, desc):
    """Packed activation streams, int32 view [B,P,C,Hp,Wp]."""
    _require_cuda(act)
    a = act.detach().to(torch.float32).contiguous()
    nbytes = _lib.size_query("geo_sc_act_stream_bytes", desc)
    with torch.cuda.device(a.device):
        buf = torch.empty(nbytes, dtype=torch.uint8, device=a.device)
        check(_lib.lib().geo_sc_generate_act_streams(ctypes.byref(desc), a.data_ptr(), buf.data_ptr(), nbytes,
                                                     _stream_ptr(a.device)), "geo_sc_generate_act_streams")
    STATS.launches += 1
    return buf


def accumulate(astreams, wprep, desc, out=None):
    _require_cuda(astreams, wprep)
    with torch.cuda.device(astreams.device):
        if out is None:
            out = torch.empty(out_shape(desc), dtype=torch.int32, device=astreams.device)
        check(_lib.lib().geo_sc_accumulate(ctypes.byref(desc), astreams.data_ptr(), wprep.data_ptr(), out.data_ptr(),
                                           _stream_ptr(astreams.device)), "geo_sc_accumulate")
    STATS.launches += 1
    return out


def guide_backward(act, weight, grad_out, desc, need_act=True, need_weight=True, quantized=False):
    """Gradient of the float guide: (grad_act or None, grad_weight or None).

    ``quantized=True`` is the caller's promise that ``act`` and ``weight`` are multiples of 2^-8
    (or coarser) inside [-1, 1]; the tensor-core kernels then run alone, and a broken promise
    yields NaN gradients (checked on the device)."""
    _require_cuda(act, weight, grad_out)
    a = act.detach().to(torch.float32).contiguous()
    w = weight.detach().to(torch.float32).contiguous()
    go = grad_out.detach().to(torch.float32).contiguous()
    if tuple(go.shape) != out_shape(desc):
        raise ValueError(f"grad_out has shape {tuple(go.shape)}, expected {out_shape(desc)}")
    nbytes = _lib.size_query("geo_sc_guide_backward_bytes", desc)
    dev = w.device
    with torch.cuda.device(dev):
        scratch = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
        ga = torch.empty((desc.batch, desc.c_in, desc.h_in, desc.w_in), dtype=torch.float32, device=dev) \
            if need_act else None
        gw = torch.empty((desc.c_out, desc.c_in, desc.k_h, desc.k_w), dtype=torch.float32, device=dev) \
            if need_weight else None
        name = "geo_sc_guide_backward_quantized" if quantized else "geo_sc_guide_backward"
        check(getattr(_lib.lib(), name)(ctypes.byref(desc), a.data_ptr(), w.data_ptr(), go.data_ptr(),
                                        ga.data_ptr() if need_act else None,
                                        gw.data_ptr() if need_weight else None, scratch.data_ptr(),
                                        scratch.numel(), _stream_ptr(dev)), name)
    per_family = 3 + (2 if need_weight else 0) + (2 if need_act else 0)   # prep x2, forward, wgrad+reduce, prep+dgrad
    if desc.mode in (MODES["1d_bin"], MODES["full_or"], MODES["2d_bin"], MODES["full_bin"]):
        STATS.launches += per_family + (1 if quantized else per_family)
    else:
        STATS.launches += per_family
    return ga, gw


def _bn_scratch(batch, channels, device):
    n = ctypes.c_size_t(0)
    check(_lib.lib().geo_sc_bn_fixed_scratch_bytes(batch, channels, ctypes.byref(n)), "geo_sc_bn_fixed_scratch_bytes")
    return torch.empty(n.value, dtype=torch.uint8, device=device)


def _ptr(t):
    return t.data_ptr() if t is not None else None


def bn_fixed_forward(x, weight, bias, running_mean, running_var, training, momentum, eps):
    """Quantised batch norm forward -> (out, save_mean, save_invstd, scale); updates the running
    statistics in place in training mode.  x is [B,C,H,W] or [B,C], fp32, contiguous."""
    _require_cuda(x)
    xc = x.detach().to(torch.float32).contiguous()
    B, C = xc.shape[0], xc.shape[1]
    spatial = xc.numel() // (B * C)
    dev = xc.device
    with torch.cuda.device(dev):
        out = torch.empty_like(xc)
        mean = torch.empty(C, dtype=torch.float32, device=dev)
        invstd = torch.empty(C, dtype=torch.float32, device=dev)
        scale = torch.empty(1, dtype=torch.float32, device=dev)
        scratch = _bn_scratch(B, C, dev)
        check(_lib.lib().geo_sc_bn_fixed_forward(B, C, spatial, int(bool(training)), float(eps), float(momentum),
                                                 xc.data_ptr(), _ptr(weight), _ptr(bias), _ptr(running_mean),
                                                 _ptr(running_var), out.data_ptr(), mean.data_ptr(), invstd.data_ptr(),
                                                 scale.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                                 _stream_ptr(dev)), "geo_sc_bn_fixed_forward")
    STATS.launches += 5 if training else 2
    return out, mean, invstd, scale


def bn_fixed_backward(x, grad_out, weight, mean, invstd, training, need_affine=True):
    """Gradient of the (unquantised) batch normalisation -> (grad_x, grad_weight, grad_bias)."""
    _require_cuda(x, grad_out)
    xc = x.detach().to(torch.float32).contiguous()
    go = grad_out.detach().to(torch.float32).contiguous()
    B, C = xc.shape[0], xc.shape[1]
    spatial = xc.numel() // (B * C)
    dev = xc.device
    with torch.cuda.device(dev):
        gx = torch.empty_like(xc)
        gw = torch.empty(C, dtype=torch.float32, device=dev) if need_affine else None
        gb = torch.empty(C, dtype=torch.float32, device=dev) if need_affine else None
        scratch = _bn_scratch(B, C, dev)
        check(_lib.lib().geo_sc_bn_fixed_backward(B, C, spatial, int(bool(training)), xc.data_ptr(), go.data_ptr(),
                                                  _ptr(weight), mean.data_ptr(), invstd.data_ptr(), gx.data_ptr(),
                                                  _ptr(gw), _ptr(gb), scratch.data_ptr(), scratch.numel(),
                                                  _stream_ptr(dev)), "geo_sc_bn_fixed_backward")
    STATS.launches += 3
    return gx, gw, gb


def bn_pool_act_supported(x):
    """Whether the one-pass batch norm + 2x2 average pool + hardtanh applies to ``x``."""
    return x.is_cuda and x.dim() == 4 and x.shape[2] % 2 == 0 and x.shape[3] % 4 == 0 and x.shape[2] >= 2


def bn_pool_act_forward(x, weight, bias, running_mean, running_var, training, momentum, eps):
    """hardtanh(avg_pool2d(bn_fixed(x), 2), 0, 1) -> (out, save_mean, save_invstd, scale, w_q, b_q)."""
    _require_cuda(x)
    xc = x.detach().to(torch.float32).contiguous()
    B, C, H, W = xc.shape
    dev = xc.device
    with torch.cuda.device(dev):
        out = torch.empty((B, C, H // 2, W // 2), dtype=torch.float32, device=dev)
        stats = torch.empty((4, C), dtype=torch.float32, device=dev)     # mean, invstd, w_q, b_q
        scale = torch.empty(1, dtype=torch.float32, device=dev)
        scratch = _bn_scratch(B, C, dev)
        check(_lib.lib().geo_sc_bn_pool_act_forward(
            B, C, H, W, int(bool(training)), float(eps), float(momentum), xc.data_ptr(), _ptr(weight), _ptr(bias),
            _ptr(running_mean), _ptr(running_var), out.data_ptr(), stats[0].data_ptr(), stats[1].data_ptr(),
            stats[2].data_ptr(), stats[3].data_ptr(), scale.data_ptr(), scratch.data_ptr(), scratch.numel(),
            _stream_ptr(dev)), "geo_sc_bn_pool_act_forward")
    STATS.launches += 5 if training else 2
    return out, stats[0], stats[1], scale, stats[2], stats[3]


def bn_pool_act_backward(x, grad_out, weight, mean, invstd, wq, bq, training, need_affine=True):
    """Gradient of :func:`bn_pool_act_forward` -> (grad_x, grad_weight, grad_bias)."""
    _require_cuda(x, grad_out)
    xc = x.detach().to(torch.float32).contiguous()
    go = grad_out.detach().to(torch.float32).contiguous()
    B, C, H, W = xc.shape
    dev = xc.device
    with torch.cuda.device(dev):
        gx = torch.empty_like(xc)
        gw = torch.empty(C, dtype=torch.float32, device=dev) if need_affine else None
        gb = torch.empty(C, dtype=torch.float32, device=dev) if need_affine else None
        scratch = _bn_scratch(B, C, dev)
        check(_lib.lib().geo_sc_bn_pool_act_backward(
            B, C, H, W, int(bool(training)), xc.data_ptr(), go.data_ptr(), _ptr(weight), mean.data_ptr(),
            invstd.data_ptr(), wq.data_ptr(), bq.data_ptr(), gx.data_ptr(), _ptr(gw), _ptr(gb), scratch.data_ptr(),
            scratch.numel(), _stream_ptr(dev)), "geo_sc_bn_pool_act_backward")
    STATS.launches += 3
    return gx, gw, gb


def quantize(x, prec):
    """clamp(round(x * 2^prec), +-(2^prec - 1)) / 2^prec of a CUDA tensor as one kernel."""
    _require_cuda(x)
    xc = x.detach().to(torch.float32).contiguous()
    with torch.cuda.device(xc.device):
        y = torch.empty_like(xc)
        check(_lib.lib().geo_sc_quantize(xc.data_ptr(), y.data_ptr(), xc.numel(), int(prec), _stream_ptr(xc.device)),
              "geo_sc_quantize")
    STATS.launches += 1
    return y


def counts_to_float(counts, bit_length):
    """SC bit counts (int32, CUDA) -> float32 counts / bit_length as one kernel."""
    _require_cuda(counts)
    c = counts.contiguous()
    if c.dtype != torch.int32:
        raise TypeError(f"counts must be int32, got {c.dtype}")
    with torch.cuda.device(c.device):
        y = torch.empty(c.shape, dtype=torch.float32, device=c.device)
        check(_lib.lib().geo_sc_counts_to_float(c.data_ptr(), y.data_ptr(), c.numel(), int(bit_length),
                                                _stream_ptr(c.device)), "geo_sc_counts_to_float")
    STATS.launches += 1
    return y


def pool_act_forward(x):
    """hardtanh(avg_pool2d(x, 2), 0, 1) for x [B,C,H,W]."""
    _require_cuda(x)
    xc = x.detach().to(torch.float32).contiguous()
    B, C, H, W = xc.shape
    with torch.cuda.device(xc.device):
        y = torch.empty((B, C, H // 2, W // 2), dtype=torch.float32, device=xc.device)
        check(_lib.lib().geo_sc_pool_act_forward(B * C, H, W, xc.data_ptr(), y.data_ptr(), _stream_ptr(xc.device)),
              "geo_sc_pool_act_forward")
    STATS.launches += 1
    return y


def pool_act_backward(x, grad_y):
    _require_cuda(x, grad_y)
    xc = x.detach().to(torch.float32).contiguous()
    gy = grad_y.detach().to(torch.float32).contiguous()
    B, C, H, W = xc.shape
    with torch.cuda.device(xc.device):
        gx = torch.empty_like(xc)
        check(_lib.lib().geo_sc_pool_act_backward(B * C, H, W, xc.data_ptr(), gy.data_ptr(), gx.data_ptr(),
                                                  _stream_ptr(xc.device)), "geo_sc_pool_act_backward")
    STATS.launches += 1
    return gx


def act_streams_canonical(buf, desc):
    """View the activation-stream buffer as int32 [B,C,Hp,Wp,P] (the oracle's layout)."""
    P = (desc.bit_length + 31) // 32
    Hp, Wp = desc.h_in + 2 * desc.pad_h, desc.w_in + 2 * desc.pad_w
    batch_innermost, Bp = _lib.act_stream_layout(desc)
    n = Bp * P * desc.c_in * Hp * Wp
    if batch_innermost:   # [pack][c][Hp][Wp][batch padded to 4]
        v = buf[: n * 4].view(torch.int32).view(P, desc.c_in, Hp, Wp, Bp)[..., : desc.batch]
        return v.permute(4, 1, 2, 3, 0).contiguous()
    v = buf[: n * 4].view(torch.int32).view(desc.batch, P, desc.c_in, Hp, Wp)
    return v.permute(0, 2, 3, 4, 1).contiguous()


def weight_streams_canonical(buf, desc):
    """Decode the prepared-weight buffer to int32 [2,O,C,K2,K3,P] (the oracle's layout)."""
    G, K, Kp, NT, Opad = _lib.group_geometry_full(desc)
    P = (desc.bit_length + 31) // 32
    O, C, K2, K3 = desc.c_out, desc.c_in, desc.k_h, desc.k_w
    n = P * G * Kp * Opad * 2
    v = buf[: n * 4].view(torch.int32).view(P, G, Kp, Opad, 2)[:, :, :K, :O, :]
    mode = desc.mode
    if mode == _lib.MODE_1D:        # g = kx, k = c*K2+ky
        v = v.reshape(P, K3, C, K2, O, 2).permute(5, 4, 2, 3, 1, 0)
    elif mode == _lib.MODE_Z:       # g = c, k = ky*K3+kx
        v = v.reshape(P, C, K2, K3, O, 2).permute(5, 4, 1, 2, 3, 0)
    elif mode == _lib.MODE_YZ:      # g = zp*K3+kx, k = cz*K2+ky, c = zp*z+cz (channels past C are zero fill)
        z = min(desc.z_unit, C)
        zp = (C + z - 1) // z
        v = v.reshape(P, zp, K3, z, K2, O, 2).permute(6, 5, 1, 3, 4, 2, 0).reshape(2, O, zp * z, K2, K3, P)[:, :, :C]
    elif mode == _lib.MODE_2D:      # g = ky*K3+kx, k = c
        v = v.reshape(P, K2, K3, C, O, 2).permute(5, 4, 3, 1, 2, 0)
    elif mode == _lib.MODE_FULL_BIN:   # g = (c*K2+ky)*K3+kx, one member
        v = v.reshape(P, C, K2, K3, O, 2).permute(5, 4, 1, 2, 3, 0)
    else:                           # g = 0, k = (c*K2+ky)*K3+kx
        v = v.reshape(P, C, K2, K3, O, 2).permute(5, 4, 1, 2, 3, 0)
    return v.contiguous()


def measure_lop3_peak():
    """Measured 32-bit logic-op rate of the current device, ops/s."""
    rate, ms = ctypes.c_double(0), ctypes.c_double(0)
    check(_lib.lib().geo_sc_measure_lop3_peak(ctypes.byref(rate), ctypes.byref(ms)), "geo_sc_measure_lop3_peak")
    return rate.value, ms.value


def epilogue_forward(counts, in_bit_length, next_desc, weight, bias, running_mean, running_var, training, momentum, eps,
                     prec=7):
    """Bit counts of one SC layer -> the next layer's rounded activation and packed streams in one pass (batch norm
    with folded 7-bit scale / shift, 2x2 average pool, hardtanh(0, 1), rounding, stream generation).
    ``next_desc`` describes the next layer (its input is the pooled tensor).
    Returns (activation, streams, save_mean, save_invstd, scale, w_q, b_q)."""
    _require_cuda(counts)
    c = counts.contiguous()
    if c.dtype != torch.int32:
        raise TypeError(f"counts must be int32, got {c.dtype}")
    B, C, H, W = c.shape
    if (B, C, H, W) != (next_desc.batch, next_desc.c_in, 2 * next_desc.h_in, 2 * next_desc.w_in):
        raise ValueError(f"counts {tuple(c.shape)} do not pool to the next layer's input "
                         f"({next_desc.batch}, {next_desc.c_in}, {next_desc.h_in}, {next_desc.w_in})")
    dev = c.device
    nbytes = _lib.size_query("geo_sc_act_stream_bytes", next_desc)
    with torch.cuda.device(dev):
        act = torch.empty((B, C, H // 2, W // 2), dtype=torch.float32, device=dev)
        streams = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        stats = torch.empty((4, C), dtype=torch.float32, device=dev)     # mean, invstd, w_q, b_q
        scale = torch.empty(1, dtype=torch.float32, device=dev)
        scratch = _bn_scratch(B, C, dev)
        check(_lib.lib().geo_sc_epilogue_forward(
            ctypes.byref(next_desc), int(in_bit_length), int(prec), int(bool(training)), float(eps), float(momentum),
            c.data_ptr(), _ptr(weight), _ptr(bias), _ptr(running_mean), _ptr(running_var), act.data_ptr(),
            stats[0].data_ptr(), stats[1].data_ptr(), stats[2].data_ptr(), stats[3].data_ptr(), scale.data_ptr(),
            streams.data_ptr(), nbytes, scratch.data_ptr(), scratch.numel(), _stream_ptr(dev)), "geo_sc_epilogue_forward")
    STATS.launches += (6 if training else 3)
    return act, streams, stats[0], stats[1], scale, stats[2], stats[3]


def epilogue_backward(counts, in_bit_length, grad_out, weight, mean, invstd, wq, bq, training, need_affine=True):
    """Gradient of :func:`epilogue_forward` with respect to the layer's value counts / bit_length and the batch-norm
    affine parameters -> (grad_x, grad_weight, grad_bias)."""
    _require_cuda(counts, grad_out)
    c = counts.contiguous()
    go = grad_out.detach().to(torch.float32).contiguous()
    B, C, H, W = c.shape
    dev = c.device
    with torch.cuda.device(dev):
        gx = torch.empty((B, C, H, W), dtype=torch.float32, device=dev)
        gw = torch.empty(C, dtype=torch.float32, device=dev) if need_affine else None
        gb = torch.empty(C, dtype=torch.float32, device=dev) if need_affine else None
        scratch = _bn_scratch(B, C, dev)
        check(_lib.lib().geo_sc_epilogue_backward(
            B, C, H, W, int(in_bit_length), int(bool(training)), c.data_ptr(), go.data_ptr(), _ptr(weight), mean.data_ptr(),
            invstd.data_ptr(), wq.data_ptr(), bq.data_ptr(), gx.data_ptr(), _ptr(gw), _ptr(gb), scratch.data_ptr(),
            scratch.numel(), _stream_ptr(dev)), "geo_sc_epilogue_backward")
    STATS.launches += 3
    return gx, gw, gb
