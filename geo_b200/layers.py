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

    def requantize_weight(self, prec=7):
        """``weight`` re-quantised from ``weight_org`` (every call in training mode, on change in evaluation mode);
        returns the dict in which packed weight streams may be kept, or None in training mode."""
        if self.training:
            self._stream_cache_tag = None
            self.weight.data = sc_f.quantize(self.weight_org, prec=prec)
            return None
        tag = (self.weight_org.data_ptr(), self.weight_org._version, prec)
        if tag != self._stream_cache_tag:
            self._stream_cache.clear()
            self._stream_cache_tag = tag
            self.weight.data = sc_f.quantize(self.weight_org, prec=prec)
        return self._stream_cache

    def forward(self, input, prec=7, err=7, forward="1d_bin", generator="lfsr", z_unit=8, legacy=False, load_unit=8,
                load_wait_w=2, load_wait_a=2, astreams=None):
        """``astreams`` (an extension over the reference): the packed streams of ``input`` for this very call,
        made by the fused epilogue of the layer in front; ``input`` is then already rounded to ``prec`` bits."""
        if astreams is None:
            input.data = sc_f.quantize(input.data, prec=prec)
        cache = self.requantize_weight(prec)
        return sc_f.conv2d_generic(input, self.weight, bit_length=2 ** err, padding=self.padding, stride=self.stride,
                                   forward=forward, generator=generator, legacy=legacy, z_unit=z_unit,
                                   load_unit=load_unit, load_wait_w=load_wait_w, load_wait_a=load_wait_a,
                                   quantized=prec <= 8,  # k / 2^prec with |k| < 2^8 is exact in bf16
                                   weight_cache=cache, astreams=astreams)


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


# Set to False to run every SC block as its separate layers (the tests compare the two forms).
FUSE_EPILOGUE = True


class _SCBlock(torch.autograd.Function):
    """One SC layer with everything up to the next SC layer's input: SC conv2d (value: bit counts / bit_length,
    gradient: the float guide's) -> ``BatchNorm2d_fixed`` -> ``AvgPool2d(2)`` -> ``Hardtanh(0, 1)`` -> the rounding
    the next ``Conv2d_Add_Partial`` applies to its input -> that layer's packed activation streams
    (network.py:165-184, utils_class.py:32-33,37-65).  Between the accumulation kernel and the next layer's
    accumulation kernel the activations make one trip through memory: the bit counts are read (twice more for the
    batch statistics), the rounded activation and the streams are written.  Outputs equal the separate layers'
    bit for bit; the backward pass is theirs too, reading the bit counts where they read the float value."""

    @staticmethod
    def forward(ctx, activation, weight, bn_weight, bn_bias, bn, sc, next_desc, weight_cache, astreams):
        d = ops.desc_for(activation, weight, sc["bit_length"], sc["mode"], (sc["pad_h"], sc["pad_w"]),
                         **{k: sc[k] for k in ("z_unit", "total_width", "load_width", "load_wait_w", "load_wait_a")})
        wprep = None
        if weight_cache is not None:
            key = (tuple(activation.shape[1:]), tuple(weight.shape)) + tuple(sorted(sc.items()))
            wprep = weight_cache.get(key)
            if wprep is None:
                wprep = weight_cache[key] = ops.prepare_weights(weight, d)
        counts = ops.sc_conv2d_staged(activation, weight, sc["bit_length"], sc["mode"], (sc["pad_h"], sc["pad_w"]),
                                      wprep=wprep, astreams=astreams,
                                      **{k: sc[k] for k in ("z_unit", "total_width", "load_width", "load_wait_w", "load_wait_a")})
        act, streams, mean, invstd, scale, wq, bq = ops.epilogue_forward(
            counts, sc["bit_length"], next_desc, bn_weight.detach() if bn_weight is not None else None,
            bn_bias.detach() if bn_bias is not None else None, bn.running_mean, bn.running_var, bn.training, bn.momentum,
            bn.eps)
        bn.scale = scale.reshape(())
        ctx.desc, ctx.bit_length, ctx.training, ctx.has_affine = d, sc["bit_length"], bn.training, bn_weight is not None
        ctx.save_for_backward(activation, weight, counts, bn_weight, mean, invstd, wq, bq)
        ctx.mark_non_differentiable(streams)
        return act, streams

    @staticmethod
    def backward(ctx, grad_act, _grad_streams):
        activation, weight, counts, bn_weight, mean, invstd, wq, bq = ctx.saved_tensors
        gx, gbw, gbb = ops.epilogue_backward(counts, ctx.bit_length, grad_act,
                                             bn_weight.detach() if bn_weight is not None else None, mean, invstd, wq, bq,
                                             ctx.training, ctx.has_affine)
        ga, gw = ops.guide_backward(activation, weight, gx, ctx.desc, ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                    quantized=True)
        return ga, gw, gbw, gbb, None, None, None, None, None


def sc_block(conv, bn, x, conv_kwargs, next_conv, next_kwargs, astreams=None, prec=7):
    """``hardtanh(avg_pool2d(bn(conv(x, **conv_kwargs)), 2), 0, 1)`` for a ``Conv2d_Add_Partial`` followed by a
    ``BatchNorm2d_fixed``, together with what ``next_conv(., **next_kwargs)`` would do to its input first: returns
    ``(y, streams)`` where ``y`` is already rounded to ``prec`` bits and ``streams`` are its packed streams for
    ``next_conv`` (pass both on: ``next_conv(y, astreams=streams, **next_kwargs)``).  One fused pass where it
    applies -- CUDA tensors, LFSR generators, an even pooled width, ``momentum`` set -- else the separate layers and
    ``streams`` None.  ``astreams``: streams of ``x`` from the block in front."""
    sc = sc_f.resolve_sc_arguments(conv.padding, conv.stride, dict(conv_kwargs, bit_length=2 ** conv_kwargs.get("err", 7)))
    Ho = x.shape[2] + 2 * sc["pad_h"] - conv.kernel_size[0] + 1
    Wo = x.shape[3] + 2 * sc["pad_w"] - conv.kernel_size[1] + 1
    fused = (FUSE_EPILOGUE and x.is_cuda and sc["generator"] == "lfsr" and bn.momentum is not None and Ho % 2 == 0 and Wo % 4 == 0
             and Ho >= 2 and prec <= 8)
    nsc = None
    if fused:
        nsc = sc_f.resolve_sc_arguments(next_conv.padding, next_conv.stride,
                                        dict(next_kwargs, bit_length=2 ** next_kwargs.get("err", 7)))
        fused = nsc["generator"] == "lfsr"
    if not fused:
        y = conv(x, astreams=astreams, **conv_kwargs)
        return bn_pool_hardtanh(bn, y), None
    if astreams is None:
        x.data = sc_f.quantize(x.data, prec=prec)
    cache = conv.requantize_weight(prec)
    sc.pop("generator")
    nsc.pop("generator")
    next_desc = ops.make_desc(x.shape[0], conv.out_channels, Ho // 2, Wo // 2, next_conv.out_channels,
                              next_conv.kernel_size[0], next_conv.kernel_size[1], nsc.pop("bit_length"), nsc.pop("mode"), **nsc)
    return _SCBlock.apply(x, conv.weight, bn.weight if bn.affine else None, bn.bias if bn.affine else None, bn, sc,
                          next_desc, cache, astreams)
