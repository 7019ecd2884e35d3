"""Host-side mirror of the reference's SC layers (``utils_class.py``): same class names,
constructor and ``forward`` arguments, buffers and in-place side effects."""
from __future__ import annotations

import torch
import torch.nn as nn

from . import functional as sc_f
from . import ops


class Conv2d_Add_Partial(nn.Conv2d):
    """SC conv2d with partial binary accumulation (utils_class.py:11-35).

    Keeps a full-precision copy of the weights in the buffer ``weight_org``; every forward
    re-quantises ``weight`` from it and quantises the input in place (straight-through).

    In evaluation mode the quantised weights and their packed streams are kept between calls and
    rebuilt when ``weight_org`` changes.  The change is noticed through the tensor's version counter,
    which in-place operations on ``weight_org`` advance but writes through ``weight_org.data`` (some
    optimisers and checkpoint loaders) do not: after such a write call :meth:`invalidate_stream_cache`.
    ``load_state_dict`` does so by itself."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("weight_org", self.weight.data.clone())
        # evaluation mode: quantised weights and their packed streams are kept while weight_org is unchanged
        self._stream_cache = {}
        self._stream_cache_tag = None
        self.register_load_state_dict_post_hook(lambda module, incompatible: module.invalidate_stream_cache())

    def invalidate_stream_cache(self):
        """Forget the quantised weights and packed weight streams kept for evaluation mode."""
        self._stream_cache.clear()
        self._stream_cache_tag = None

    def forward(self, input, prec=7, err=7, forward="1d_bin", generator="lfsr", z_unit=8, legacy=False, load_unit=8,
                load_wait_w=2, load_wait_a=2):
        input.data = sc_f.quantize(input.data, prec=prec)
        cache = None
        if self.training:
            self._stream_cache_tag = None
            self.weight.data = sc_f.quantize(self.weight_org, prec=prec)
        else:
            tag = (self.weight_org.data_ptr(), self.weight_org._version, prec)
            if tag != self._stream_cache_tag:
                self._stream_cache.clear()
                self._stream_cache_tag = tag
                self.weight.data = sc_f.quantize(self.weight_org, prec=prec)
            cache = self._stream_cache
        return sc_f.conv2d_generic(input, self.weight, bit_length=2 ** err, padding=self.padding, stride=self.stride,
                                   forward=forward, generator=generator, legacy=legacy, z_unit=z_unit,
                                   load_unit=load_unit, load_wait_w=load_wait_w, load_wait_a=load_wait_a,
                                   quantized=prec <= 8,  # k / 2^prec with |k| < 2^8 is exact in bf16
                                   weight_cache=cache)


class Linear_Or(nn.Linear):
    """SC linear layer with OR accumulation.  The reference's LeNet model asks for ``utils_class.Linear_Or``
    (network.py:204-206) but the class is missing from utils_class.py; this one follows ``Conv2d_Add_Partial``
    (utils_class.py:11-35): a full-precision ``weight_org`` buffer, weights and inputs quantised at every
    forward, value and gradient from ``linear_generic`` (utils_functional.py:302-404)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("weight_org", self.weight.data.clone())

    def forward(self, input, prec=7, err=7, generator="lfsr", forward="full_or"):
        input.data = sc_f.quantize(input.data, prec=prec)
        self.weight.data = sc_f.quantize(self.weight_org, prec=prec)
        out = sc_f.linear_generic(input, self.weight, bit_length=2 ** err, generator=generator, forward=forward)
        if self.bias is not None:
            out = out + self.bias
        return out


class _BatchNormFixed(torch.autograd.Function):
    """Value: x * w_q + b_q (folded, 7-bit quantised scale and shift).  Gradient: that of the plain
    batch normalisation, as in the reference, where F.batch_norm provides the graph and the
    quantised value is written over its output (utils_class.py:44-65)."""

    @staticmethod
    def forward(ctx, x, weight, bias, module):
        momentum = module.momentum
        if momentum is None:
            raise NotImplementedError("cumulative moving average (momentum=None) is not provided")
        out, mean, invstd, scale = ops.bn_fixed_forward(
            x, weight.detach() if weight is not None else None, bias.detach() if bias is not None else None,
            module.running_mean, module.running_var, module.training, momentum, module.eps)
        module.scale = scale.reshape(())
        ctx.training = module.training
        ctx.has_affine = weight is not None
        ctx.save_for_backward(x, weight, mean, invstd)
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, mean, invstd = ctx.saved_tensors
        gx, gw, gb = ops.bn_fixed_backward(x, grad_out, weight.detach() if weight is not None else None, mean, invstd,
                                           ctx.training, ctx.has_affine)
        return gx.to(x.dtype).view_as(x), gw, gb, None


class BatchNorm2d_fixed(nn.BatchNorm2d):
    """Quantised 2d batch norm (utils_class.py:37-65)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("scale", None)

    def forward(self, x):
        return _BatchNormFixed.apply(x, self.weight if self.affine else None, self.bias if self.affine else None, self)


class BatchNorm1d_fixed(nn.BatchNorm1d):
    """Quantised 1d batch norm (utils_class.py:67-93)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.register_buffer("scale", None)

    def forward(self, x):
        return _BatchNormFixed.apply(x, self.weight if self.affine else None, self.bias if self.affine else None, self)


class _BatchNormPoolHardtanh(torch.autograd.Function):
    """``hardtanh(avg_pool2d(bn(x), 2), 0, 1)`` with ``bn`` a ``BatchNorm2d_fixed``: value and gradients of the
    composition, one native pass per direction."""

    @staticmethod
    def forward(ctx, x, weight, bias, module):
        if module.momentum is None:
            raise NotImplementedError("cumulative moving average (momentum=None) is not provided")
        out, mean, invstd, scale, wq, bq = ops.bn_pool_act_forward(
            x, weight.detach() if weight is not None else None, bias.detach() if bias is not None else None,
            module.running_mean, module.running_var, module.training, module.momentum, module.eps)
        module.scale = scale.reshape(())
        ctx.training = module.training
        ctx.has_affine = weight is not None
        ctx.save_for_backward(x, weight, mean, invstd, wq, bq)
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, mean, invstd, wq, bq = ctx.saved_tensors
        gx, gw, gb = ops.bn_pool_act_backward(x, grad_out, weight.detach() if weight is not None else None, mean,
                                              invstd, wq, bq, ctx.training, ctx.has_affine)
        return gx.to(x.dtype), gw, gb, None


def bn_pool_hardtanh(bn, x):
    """``nn.Hardtanh(0, 1)(nn.AvgPool2d(2)(bn(x)))`` for a ``BatchNorm2d_fixed`` module ``bn`` (network.py:168-184);
    one pass per direction where the shape allows (even height, width a multiple of 4), else the two layers."""
    if ops.bn_pool_act_supported(x):
        return _BatchNormPoolHardtanh.apply(x, bn.weight if bn.affine else None, bn.bias if bn.affine else None, bn)
    return _PoolHardtanh.apply(bn(x))


class _PoolHardtanh(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return ops.pool_act_forward(x).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        (x,) = ctx.saved_tensors
        return ops.pool_act_backward(x, grad_y).to(x.dtype)


class AvgPool2Hardtanh(nn.Module):
    """``nn.Hardtanh(0, 1)(nn.AvgPool2d(2)(x))`` -- the activation between the reference's SC layers
    (network.py:168-184) -- as one native pass in each direction."""

    def forward(self, x):
        return _PoolHardtanh.apply(x)
