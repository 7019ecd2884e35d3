"""SC conv2d forward and its float guide as one autograd function over the native kernels.

Forward value: SC bit counts / bit_length.  Backward: gradient of the reference's float guide
(utils_functional.py:611-634): with w+ = clamp(w, 0, 100), w- = -clamp(w, -100, 0) and y±_g the
plain convolution restricted to binary-accumulated group g,

    out = sum_g (1 - exp(-y+_g)) - sum_g (1 - exp(-y-_g))

The guide's own value is never used (the reference overwrites it with the SC result), so the
forward pass computes nothing for it: activations and weights are saved and the backward pass
evaluates exp(-y±_g) and both gradients in one native call.
"""
from __future__ import annotations

import torch

from . import ops


class _SCConv2dGuide(torch.autograd.Function):
    @staticmethod
    def forward(ctx, activation, weight, bit_length, mode, pad_h, pad_w, z_unit, total_width, load_width,
                load_wait_w, load_wait_a, quantized=False, weight_cache=None, generator="lfsr", seed=0, astreams=None):
        kw = dict(z_unit=z_unit, total_width=total_width, load_width=load_width, load_wait_w=load_wait_w,
                  load_wait_a=load_wait_a, generator=generator, seed=seed)
        wprep = None
        if weight_cache is not None:
            # weight streams depend on the weights and on everything in the descriptor but the batch
            key = (tuple(activation.shape[1:]), tuple(weight.shape), bit_length, mode, pad_h, pad_w) + tuple(kw.values())
            wprep = weight_cache.get(key)
            if wprep is None:
                wprep = ops.prepare_weights(weight, ops.desc_for(activation, weight, bit_length, mode, (pad_h, pad_w), **kw))
                weight_cache[key] = wprep
        counts = ops.sc_conv2d_staged(activation, weight, bit_length, mode, (pad_h, pad_w), wprep=wprep,
                                      astreams=astreams, **kw)
        need_a, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if need_a or need_w:
            ctx.quantized = bool(quantized)
            ctx.desc = ops.desc_for(activation, weight, bit_length, mode, (pad_h, pad_w), **kw)
            ctx.save_for_backward(activation, weight)
        return ops.counts_to_float(counts, bit_length)

    @staticmethod
    def backward(ctx, grad_out):
        activation, weight = ctx.saved_tensors
        ga, gw = ops.guide_backward(activation, weight, grad_out, ctx.desc, ctx.needs_input_grad[0],
                                    ctx.needs_input_grad[1], quantized=ctx.quantized)
        if ga is not None:
            ga = ga.to(activation.dtype)
        if gw is not None:
            gw = gw.to(weight.dtype)
        return (ga, gw) + (None,) * 14


def sc_conv2d_with_guide(activation, weight, bit_length, mode, pad_h=0, pad_w=0, z_unit=1024, total_width=7,
                         load_width=8, load_wait_w=1, load_wait_a=1, quantized=False, weight_cache=None,
                         generator="lfsr", seed=0, astreams=None):
    """SC conv2d value with the guide's gradient; ``pad_h`` / ``pad_w`` pad dimensions 2 / 3.
    ``quantized``: the caller's promise of :func:`geo_b200.ops.guide_backward`.  ``weight_cache``: a dict
    owned by the caller in which the packed weight streams are kept between calls; the caller empties
    it whenever the weights change.  ``generator`` 'lfsr' or 'acc' (sampling without replacement, streams
    selected by ``seed``).  ``astreams``: packed activation streams of ``activation`` for exactly this
    descriptor, when the caller already has them (the fused epilogue of the previous layer)."""
    return _SCConv2dGuide.apply(activation, weight, bit_length, mode, pad_h, pad_w, z_unit, total_width, load_width,
                                load_wait_w, load_wait_a, quantized, weight_cache, generator, seed, astreams)
