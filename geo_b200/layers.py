"""Host-side mirror of the reference's SC layers (``utils_class.py``): same class names,
constructor and ``forward`` arguments, buffers and in-place side effects."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import functional as sc_f


class Conv2d_Add_Partial(nn.Conv2d):
    """SC conv2d with partial binary accumulation (utils_class.py:11-35).

    Keeps a full-precision copy of the weights in the buffer ``weight_org``; every forward
    re-quantises ``weight`` from it and quantises the input in place (straight-through)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("weight_org", self.weight.data.clone())

    def forward(self, input, prec=7, err=7, forward="1d_bin", generator="lfsr", z_unit=8, legacy=False, load_unit=8,
                load_wait_w=2, load_wait_a=2):
        input.data = sc_f.quantize(input.data, prec=prec)
        self.weight.data = sc_f.quantize(self.weight_org, prec=prec)
        return sc_f.conv2d_generic(input, self.weight, bit_length=2 ** err, padding=self.padding, stride=self.stride,
                                   forward=forward, generator=generator, legacy=legacy, z_unit=z_unit,
                                   load_unit=load_unit, load_wait_w=load_wait_w, load_wait_a=load_wait_a)


def _fixed_affine(module, x, reduce_dims):
    """Quantised normalisation shared by the two BatchNorm variants (utils_class.py:43-65,74-93):
    the autograd graph is that of ``F.batch_norm``; the value is ``x * w_q + b_q`` with the folded
    scale and shift quantised to 7 bits under one power-of-two range."""
    out = F.batch_norm(x, module.running_mean, module.running_var, module.weight, module.bias,
                       training=module.training)
    if module.training:
        mean = x.mean(dim=reduce_dims)
        var = x.var(dim=reduce_dims, unbiased=False)
    else:
        mean, var = module.running_mean, module.running_var
    if module.affine:
        weight, bias = module.weight.data, module.bias.data
    else:
        weight, bias = 1, 0
    inv = torch.sqrt(var + module.eps)
    w_n = (weight / inv).detach()
    b_n = (bias - mean * weight / inv).detach()
    w_n, module.scale = sc_f.quantize_shift(w_n)
    b_n, _ = sc_f.quantize_shift(b_n, module.scale)
    return out, w_n, b_n


class BatchNorm2d_fixed(nn.BatchNorm2d):
    """Quantised 2d batch norm (utils_class.py:37-65)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("scale", None)

    def forward(self, x):
        out, w_n, b_n = _fixed_affine(self, x, (0, 2, 3))
        out.data = (x.data * w_n.reshape(-1, 1, 1) + b_n.reshape(-1, 1, 1)).to(out.dtype)
        return out


class BatchNorm1d_fixed(nn.BatchNorm1d):
    """Quantised 1d batch norm (utils_class.py:67-93)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("scale", None)

    def forward(self, x):
        out, w_n, b_n = _fixed_affine(self, x, (0,))
        out.data = (x.data * w_n + b_n).to(out.dtype)
        return out
