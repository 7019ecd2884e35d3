"""Test helper: lets the host-side Python stack (layers, network, train step, data-parallel hook)
run on CPU tensors by standing the CPU oracle in for the three native entry points it calls.
Used only by the CPU tests of host logic; the product has no such path."""
import torch

import oracle
from oracle import guide as oracle_guide

_MODE_NAMES = {0: "1d_bin", 1: "z_bin", 2: "yz_bin", 3: "full_or"}


def install(monkeypatch):
    from geo_b200 import ops

    def sc_conv2d_staged(act, weight, bit_length, mode="1d_bin", padding=(0, 0), wprep=None, **kw):
        y = oracle.conv2d(act.detach(), weight.detach(), bit_length, mode, pad_h=padding[0], pad_w=padding[1], **kw)
        return torch.from_numpy(y)

    def guide_forward(act, weight, desc):
        return act.detach().clone()

    def guide_backward(weight, saved, grad_out, desc, need_act=True, need_weight=True):
        ga, gw = oracle_guide.guide_grads(saved, weight.detach(), grad_out, _MODE_NAMES[desc.mode], desc.pad_h,
                                          desc.pad_w, z_unit=desc.z_unit)
        return (ga if need_act else None), (gw if need_weight else None)

    monkeypatch.setattr(ops, "sc_conv2d_staged", sc_conv2d_staged)
    monkeypatch.setattr(ops, "guide_forward", guide_forward)
    monkeypatch.setattr(ops, "guide_backward", guide_backward)
