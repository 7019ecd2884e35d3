"""SC conv2d forward fused with its float guide as one autograd function.

Forward value: SC bit counts / bit_length (from the CUDA library).  Backward: gradient of the
reference's float guide (utils_functional.py:611-634): with w+ = clamp(w, 0, 100),
w- = -clamp(w, -100, 0) and y±_g the plain convolution restricted to binary-accumulated group g,

    out = sum_g (1 - exp(-y+_g)) - sum_g (1 - exp(-y-_g))
    d out / d y+_g = exp(-y+_g),   d out / d y-_g = -exp(-y-_g)

so that grad_w and grad_a are convolutions of grad_out * exp(-y±_g) with the activations and
the clamped weights.  clamp passes the gradient on both of its branches at w == 0.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ops


def _guide_pos_neg(a, weight, mode, z_unit):
    w_pos = weight.clamp(0, 100)
    w_neg = -(weight.clamp(-100, 0))
    C, K3, Wp = a.size(1), weight.size(3), a.size(3)
    if mode == "full_or":
        return 1 - torch.exp(-F.conv2d(a, w_pos)), 1 - torch.exp(-F.conv2d(a, w_neg))
    if mode == "1d_bin":
        groups = [(0, C, j) for j in range(K3)]
    elif mode == "z_bin":
        groups = [(c, c + 1, None) for c in range(C)]
    else:
        z = min(z_unit, C)
        groups = [(c, min(c + z, C), j) for c in range(0, C, z) for j in range(K3)]
    pos = neg = None
    for c0, c1, j in groups:
        if j is None:
            a_g, wp_g, wn_g = a[:, c0:c1], w_pos[:, c0:c1], w_neg[:, c0:c1]
        else:
            a_g = a[:, c0:c1, :, j:Wp - K3 + j + 1]
            wp_g, wn_g = w_pos[:, c0:c1, :, j:j + 1], w_neg[:, c0:c1, :, j:j + 1]
        p = 1 - torch.exp(-F.conv2d(a_g, wp_g))
        n = 1 - torch.exp(-F.conv2d(a_g, wn_g))
        pos = p if pos is None else pos + p
        neg = n if neg is None else neg + n
    return pos, neg


class _SCConv2dGuide(torch.autograd.Function):
    @staticmethod
    def forward(ctx, activation, weight, bit_length, mode, pad_h, pad_w, z_unit, total_width, load_width,
                load_wait_w, load_wait_a):
        counts = ops.sc_conv2d_staged(activation, weight, bit_length, mode, (pad_h, pad_w), z_unit=z_unit,
                                      total_width=total_width, load_width=load_width, load_wait_w=load_wait_w,
                                      load_wait_a=load_wait_a)
        ctx.save_for_backward(activation, weight)
        ctx.cfg = (mode, pad_h, pad_w, z_unit)
        return counts.to(torch.float32) / bit_length

    @staticmethod
    def backward(ctx, grad_out):
        activation, weight = ctx.saved_tensors
        mode, pad_h, pad_w, z_unit = ctx.cfg
        tf32 = torch.backends.cudnn.allow_tf32
        torch.backends.cudnn.allow_tf32 = False  # the guide gradient is specified in fp32
        try:
            with torch.enable_grad():
                a = activation.detach().to(torch.float32).requires_grad_(True)
                w = weight.detach().to(torch.float32).requires_grad_(True)
                pos, neg = _guide_pos_neg(F.pad(a, (pad_w, pad_w, pad_h, pad_h)), w, mode, z_unit)
                need = [t for t, n in ((a, ctx.needs_input_grad[0]), (w, ctx.needs_input_grad[1])) if n]
                grads = torch.autograd.grad(pos - neg, need, grad_out.to(torch.float32)) if need else ()
        finally:
            torch.backends.cudnn.allow_tf32 = tf32
        grads = list(grads)
        ga = grads.pop(0).to(activation.dtype) if ctx.needs_input_grad[0] else None
        gw = grads.pop(0).to(weight.dtype) if ctx.needs_input_grad[1] else None
        return (ga, gw) + (None,) * 9


def sc_conv2d_with_guide(activation, weight, bit_length, mode, pad_h=0, pad_w=0, z_unit=1024, total_width=7,
                         load_width=8, load_wait_w=1, load_wait_a=1):
    """SC conv2d value with the guide's gradient; ``pad_h`` / ``pad_w`` pad dimensions 2 / 3."""
    return _SCConv2dGuide.apply(activation, weight, bit_length, mode, pad_h, pad_w, z_unit, total_width, load_width,
                                load_wait_w, load_wait_a)
