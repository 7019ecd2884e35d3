"""Host-side mirror of the reference's SC functional layer (``utils_functional.py``).

Same public names, keyword arguments, defaults and error behaviour for the accelerated path:
``quantize`` (utils_functional.py:33-39), ``quantize_shift`` (:41-57), ``conv2d_generic``
(:406-634) and ``linear_generic`` (:302-404).  The stochastic-computing result comes from the
CUDA library through the C ABI; the float "guide" whose autograd is the training backward
(:611-634) comes from the native guide kernels.  All six accumulation modes (``1d_bin``, ``z_bin``,
``yz_bin``, ``full_or``, and ``2d_bin`` / ``full_bin``, which the reference only simulates bit by bit)
and the ``lfsr``, ``acc`` and ``rand`` generators run natively.  The bit-serial simulation itself
(``legacy=True``) and CPU tensors are outside this package: ``NotImplementedError`` / ``RuntimeError``.
"""
from __future__ import annotations

import torch

from . import ops
from .guide import sc_conv2d_with_guide

prec_default = 7  # 8-bit integers, one bit for the sign (utils_functional.py:28)

_ACCELERATED_MODES = ("1d_bin", "z_bin", "yz_bin", "full_or", "2d_bin", "full_bin")


def quantize(input, prec=8):
    """Round to ``prec`` fractional bits and clamp to (-1, 1) (utils_functional.py:33-39)."""
    if (input.is_cuda and input.dtype == torch.float32 and not input.requires_grad and isinstance(prec, int)
            and 0 <= prec <= 23):
        return ops.quantize(input, prec)      # the same arithmetic as one native kernel
    levels = 2 ** prec
    return (input * levels).round().clamp(-levels + 1, levels - 1) / levels


def quantize_shift(tensor, scale=None, scale_only=False):
    """7-bit quantisation with a power-of-two range (utils_functional.py:41-57)."""
    if scale_only:
        scale = 2 ** torch.ceil(torch.log2(torch.mean(tensor) * 2))
        return torch.ones_like(tensor) * scale, scale
    if scale is None:
        scale = 2 ** torch.ceil(torch.log2(torch.mean(tensor) * 3))
    q = ((tensor / scale) * 128).round().clamp(-127, 127) / 128
    return q * scale, scale


_seed_counter = [0]


def _next_seed(gen):
    """Seed of the next call of a random generator: a process-wide counter, so that a run is reproducible and
    successive calls draw different streams."""
    if gen == "lfsr":
        return 0
    _seed_counter[0] += 1
    return _seed_counter[0]


def _pair(v):
    if isinstance(v, (tuple, list)):
        return int(v[0]), int(v[1])
    return int(v), int(v)


def resolve_sc_arguments(padding, stride, kwargs):
    """The keyword arguments of :func:`conv2d_generic` turned into the native descriptor's fields, with the
    reference's defaults and the rules of utils_functional.py:489-516 (padding order, which modes take loading
    arguments, full_or ignoring the generator); raises for what only the bit-serial simulation provides."""
    bit_length = kwargs.get("bit_length", 128)
    generator = kwargs.get("generator", None)
    forward = kwargs.get("forward", "full_or")
    legacy = kwargs.get("legacy", False)
    load_unit = kwargs.get("load_unit", 8)
    load_wait_w = kwargs.get("load_wait_w", 1)
    load_wait_a = kwargs.get("load_wait_a", 1)
    z_unit = kwargs.get("z_unit", 1024)

    if legacy:
        raise NotImplementedError("legacy=True is the reference's bit-serial PyTorch simulation; "
                                  "this package only provides the accelerated kernels")
    if forward not in _ACCELERATED_MODES:
        raise NotImplementedError(f"forward={forward!r} exists only in the reference's bit-serial simulation")
    if generator in ("acc", "rand"):
        # 'acc': every stream holds exactly as many ones as its level (utils_functional.py:157-176); 'rand':
        # independent bits (:92-102).  The reference's are random; these are counter-based hashes whose
        # streams are selected by ``seed`` (keyword, default: a counter that advances with every call).
        gen = generator
    elif generator == "lfsr" or forward == "full_or":
        # full_or ignores the generator argument in the reference (utils_functional.py:511-514) and does so here
        gen = "lfsr"
    else:
        raise NotImplementedError(f"generator={generator!r} with forward={forward!r} is not provided; use 'lfsr', 'acc' or 'rand'")
    sh, sw = _pair(stride)
    if (sh, sw) != (1, 1):
        raise ValueError("stride must be 1: the reference's SC kernels ignore the stride argument "
                         "(sc_cuda_kernel.cu:1732-1834), so no other stride has a defined result")
    p0, p1 = _pair(padding)
    if forward in ("full_or", "2d_bin", "full_bin"):
        # The reference's full_or kernel takes no loading arguments (sc_cuda.cpp:21-32); 2d_bin and full_bin
        # exist only in its bit-serial simulation, which has no progressive loading (utils_functional.py:516-609).
        load_unit, load_wait_w, load_wait_a = 8, 1, 1
    elif forward in ("1d_bin", "z_bin"):
        load_wait_a = load_wait_w  # one load_wait for both operands (sc_cuda.cpp:47-63)
    return dict(bit_length=int(bit_length), mode=forward, pad_h=p1, pad_w=p0, z_unit=int(z_unit),
                total_width=prec_default, load_width=int(load_unit), load_wait_w=int(load_wait_w),
                load_wait_a=int(load_wait_a), generator=gen)


def conv2d_generic(activation, weight, padding, stride, **kwargs):
    """SC conv2d with a float guide for back-propagation (utils_functional.py:406-634).

    Keyword arguments (defaults as in the reference): ``bit_length`` 128, ``prec`` 128,
    ``share`` True, ``generator`` None, ``forward`` 'full_or', ``legacy`` False, ``load_unit`` 8,
    ``load_wait_w`` 1, ``load_wait_a`` 1, ``z_unit`` 1024.  One extension over the reference:
    ``quantized`` (default False) promises that both operands went through :func:`quantize` with
    ``prec`` <= 8, which lets the backward pass run on the tensor-core kernels alone; ``weight_cache``
    (default None) is a dict in which the packed weight streams are kept between calls -- the caller
    empties it when the weights change; ``astreams`` (default None) are the packed activation streams of
    ``activation`` for this very call, when the fused epilogue of the previous layer has made them.

    ``padding`` follows the reference's convention ``F.pad(x, (p[0], p[0], p[1], p[1]))``: the
    last dimension is padded by ``padding[0]``, dimension 2 by ``padding[1]``
    (utils_functional.py:492-516).  The value returned is the SC bit count divided by
    ``bit_length``; its gradient is the gradient of the guide.
    """
    r = resolve_sc_arguments(padding, stride, kwargs)
    gen = r["generator"]
    return sc_conv2d_with_guide(activation, weight, r["bit_length"], r["mode"], pad_h=r["pad_h"], pad_w=r["pad_w"],
                                z_unit=r["z_unit"], total_width=r["total_width"], load_width=r["load_width"],
                                load_wait_w=r["load_wait_w"], load_wait_a=r["load_wait_a"],
                                quantized=bool(kwargs.get("quantized", False)),
                                weight_cache=kwargs.get("weight_cache", None) if gen == "lfsr" else None,
                                generator=gen, seed=int(kwargs["seed"]) if "seed" in kwargs else _next_seed(gen),
                                astreams=kwargs.get("astreams", None) if gen == "lfsr" else None)


def linear_generic(activation, weight, **kwargs):
    """SC linear layer (utils_functional.py:302-404): ``bit_length`` 128, ``generator`` None,
    ``forward`` 'full_or' (or 'full_bin'), ``share`` True.  One extension over the reference: ``z_unit`` (default:
    all inputs, i.e. full OR) ORs inside groups of ``z_unit`` inputs and adds across groups.
    Shared generators (``share=True``, the reference default) and the LFSR generator only.
    Unlike the reference's simulation, levels are quantised as the extension does
    (sc_cuda.cpp:51-55); the two coincide for 7-bit inputs at ``bit_length`` 128."""
    bit_length = kwargs.get("bit_length", 128)
    generator = kwargs.get("generator", None)
    forward = kwargs.get("forward", "full_or")
    share = kwargs.get("share", True)
    if forward not in ("full_or", "full_bin"):
        raise NotImplementedError(f"forward={forward!r} is not a mode of linear_generic")
    if generator != "lfsr" or not share:
        raise NotImplementedError("only generator='lfsr' with share=True is provided")
    if activation.dim() != 2:
        raise ValueError("linear_generic expects activations of shape [batch, features]")
    z_unit = int(kwargs.get("z_unit", activation.shape[1]))
    a4 = activation.unsqueeze(-1).unsqueeze(-1)
    w4 = weight.unsqueeze(-1).unsqueeze(-1)
    # full_or: OR inside groups of z_unit inputs (all of them by default); full_bin: every product bit counted
    mode = "yz_bin" if forward == "full_or" else "full_bin"
    out = sc_conv2d_with_guide(a4, w4, int(bit_length), mode, pad_h=0, pad_w=0, z_unit=z_unit,
                               total_width=prec_default, load_width=8, load_wait_w=1, load_wait_a=1)
    return out.flatten(1)


def sc_forward_counts(activation, weight, bit_length, forward="1d_bin", padding=(0, 0), **kw):
    """Raw SC bit counts (int32), no guide: a thin alias of :func:`geo_b200.ops.sc_conv2d` with the
    reference's padding convention."""
    p0, p1 = _pair(padding)
    return ops.sc_conv2d(activation, weight, bit_length, forward, (p1, p0), **kw)
