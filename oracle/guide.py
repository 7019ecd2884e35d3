"""fp32 PyTorch restatement of the reference's float "guide" forward, whose autograd is the
training backward.  TEST INFRASTRUCTURE ONLY (the checker for the native guide kernels).

Follows utils_functional.py:189-296 (the per-mode guide functions) and :611-634 (how the guide
is combined with the SC result): the weights are split into ``w+ = clamp(w, 0, 100)`` and
``w- = -clamp(w, -100, 0)``; every binary-accumulated group g contributes ``1 - exp(-conv(a_g, w±_g))``;
the value is replaced by the SC result while the graph of the guide is kept.
Run it on CPU, or on a GPU with TF32 convolutions disabled.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _or_approx(a, w):
    return 1 - torch.exp(-F.conv2d(a, w))


def guide_pos_neg(a_padded, weight, mode, z_unit=1024):
    """(pos, neg) guide values for an already padded activation tensor."""
    w_pos = weight.clamp(0, 100)
    w_neg = -(weight.clamp(-100, 0))
    a = a_padded.to(w_pos.dtype)
    C = a.size(1)
    K3 = weight.size(3)
    Wp = a.size(3)
    pos, neg = [], []
    if mode == "full_or":      # utils_functional.py:189-210
        return _or_approx(a, w_pos), _or_approx(a, w_neg)
    if mode == "full_bin":     # :617-619, the plain convolution
        return F.conv2d(a, w_pos), F.conv2d(a, w_neg)
    if mode == "1d_bin":       # :235-252, one slice per filter column
        groups = [(slice(0, C), j) for j in range(K3)]
    elif mode == "z_bin":      # :254-270, one slice per input channel
        groups = [(slice(c, c + 1), None) for c in range(C)]
    elif mode == "yz_bin":     # :272-296, z_unit channels x one filter column
        groups = [(slice(c, min(c + z_unit, C)), j) for c in range(0, C, z_unit) for j in range(K3)]
    elif mode == "2d_bin":     # :212-233, one slice per filter tap
        K2, Hp = weight.size(2), a.size(2)
        for i in range(K2):
            for j in range(K3):
                a_g = a[:, :, i:Hp - K2 + i + 1, j:Wp - K3 + j + 1]
                pos.append(_or_approx(a_g, w_pos[:, :, i:i + 1, j:j + 1]))
                neg.append(_or_approx(a_g, w_neg[:, :, i:i + 1, j:j + 1]))
        return torch.stack(pos, 0).sum(0), torch.stack(neg, 0).sum(0)
    else:
        raise ValueError(mode)
    for cs, j in groups:
        if j is None:
            a_g, wp_g, wn_g = a[:, cs], w_pos[:, cs], w_neg[:, cs]
        else:
            a_g = a[:, cs, :, j:Wp - K3 + j + 1]
            wp_g, wn_g = w_pos[:, cs, :, j:j + 1], w_neg[:, cs, :, j:j + 1]
        pos.append(_or_approx(a_g, wp_g))
        neg.append(_or_approx(a_g, wn_g))
    return torch.stack(pos, 0).sum(0), torch.stack(neg, 0).sum(0)


def guide_output(activation, weight, mode, pad_h=0, pad_w=0, z_unit=1024, sc_value=None):
    """Guide output with autograd graph; if ``sc_value`` is given it replaces the value
    (utils_functional.py:632-634: result_pos.data = SC/L, result_neg.data = 0)."""
    a = F.pad(activation, (pad_w, pad_w, pad_h, pad_h))
    pos, neg = guide_pos_neg(a, weight, mode, z_unit)
    if sc_value is not None:
        pos.data = sc_value.to(pos.dtype)
        neg.data = torch.zeros_like(neg)
    return pos - neg


def guide_grads(activation, weight, grad_out, mode, pad_h=0, pad_w=0, z_unit=1024):
    """(grad_activation, grad_weight) of the guide for upstream gradient ``grad_out``."""
    with torch.enable_grad():
        a = activation.detach().clone().requires_grad_(True)
        w = weight.detach().clone().requires_grad_(True)
        out = guide_output(a, w, mode, pad_h, pad_w, z_unit)
        ga, gw = torch.autograd.grad(out, (a, w), grad_out)
    return ga, gw
