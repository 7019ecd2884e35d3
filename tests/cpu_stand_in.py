"""Test helper: lets the host-side Python stack (layers, network, train step, data-parallel hook)
run on CPU tensors by standing the CPU oracle in for the three native entry points it calls.
Used only by the CPU tests of host logic; the product has no such path."""
import torch

import oracle
from oracle import guide as oracle_guide

_MODE_NAMES = {0: "1d_bin", 1: "z_bin", 2: "yz_bin", 3: "full_or", 4: "2d_bin", 5: "full_bin"}


def install(monkeypatch):
    from geo_b200 import ops

    def sc_conv2d_staged(act, weight, bit_length, mode="1d_bin", padding=(0, 0), wprep=None, astreams=None,
                         generator="lfsr", seed=0, **kw):
        assert generator == "lfsr", "the CPU oracle only has the LFSR generator"
        y = oracle.conv2d(act.detach(), weight.detach(), bit_length, mode, pad_h=padding[0], pad_w=padding[1], **kw)
        return torch.from_numpy(y)

    def guide_backward(act, weight, grad_out, desc, need_act=True, need_weight=True, quantized=False):
        ga, gw = oracle_guide.guide_grads(act.detach(), weight.detach(), grad_out, _MODE_NAMES[desc.mode],
                                          desc.pad_h, desc.pad_w, z_unit=desc.z_unit)
        return (ga if need_act else None), (gw if need_weight else None)

    def bn_fixed_forward(x, weight, bias, running_mean, running_var, training, momentum, eps):
        # utils_class.py:43-65 in plain PyTorch
        dims = (0, 2, 3) if x.dim() == 4 else (0,)
        shape = (-1, 1, 1) if x.dim() == 4 else (-1,)
        if training:
            mean, var = x.mean(dim=dims), x.var(dim=dims, unbiased=False)
            n = x.numel() // x.shape[1]
            running_mean.mul_(1 - momentum).add_(momentum * mean)
            running_var.mul_(1 - momentum).add_(momentum * var * n / max(n - 1, 1))
        else:
            mean, var = running_mean, running_var
        w = weight if weight is not None else 1
        b = bias if bias is not None else 0
        sd = torch.sqrt(var + eps)
        w_n, b_n = w / sd, b - mean * w / sd
        scale = 2 ** torch.ceil(torch.log2(torch.mean(w_n) * 3))
        q = lambda t: ((t / scale) * 128).round().clamp(-127, 127) / 128 * scale  # noqa: E731
        out = x * q(w_n).reshape(shape) + q(b_n).reshape(shape)
        return out, mean.clone(), 1 / sd, scale.reshape(1)

    def bn_fixed_backward(x, grad_out, weight, mean, invstd, training, need_affine=True):
        dims = (0, 2, 3) if x.dim() == 4 else (0,)
        shape = (1, -1, 1, 1) if x.dim() == 4 else (1, -1)
        n = x.numel() // x.shape[1]
        xhat = (x - mean.reshape(shape)) * invstd.reshape(shape)
        sg, sgx = grad_out.sum(dims), (grad_out * xhat).sum(dims)
        w = weight.reshape(shape) if weight is not None else 1
        if training:
            gx = w * invstd.reshape(shape) * (grad_out - sg.reshape(shape) / n - xhat * sgx.reshape(shape) / n)
        else:
            gx = w * invstd.reshape(shape) * grad_out
        return gx, (sgx if need_affine else None), (sg if need_affine else None)

    def pool_act_forward(x):
        return torch.nn.functional.hardtanh(torch.nn.functional.avg_pool2d(x, 2), 0, 1)

    def pool_act_backward(x, grad_y):
        with torch.enable_grad():
            xx = x.detach().clone().requires_grad_(True)
            y = torch.nn.functional.hardtanh(torch.nn.functional.avg_pool2d(xx, 2), 0, 1)
            (gx,) = torch.autograd.grad(y, xx, grad_y)
        return gx

    monkeypatch.setattr(ops, "counts_to_float", lambda counts, bit_length: counts.to(torch.float32) / bit_length)
    monkeypatch.setattr(ops, "bn_pool_act_supported", lambda x: False)   # CPU: batch norm and pooling as two layers
    monkeypatch.setattr(ops, "pool_act_forward", pool_act_forward)
    monkeypatch.setattr(ops, "pool_act_backward", pool_act_backward)
    monkeypatch.setattr(ops, "bn_fixed_forward", bn_fixed_forward)
    monkeypatch.setattr(ops, "bn_fixed_backward", bn_fixed_backward)
    monkeypatch.setattr(ops, "sc_conv2d_staged", sc_conv2d_staged)
    monkeypatch.setattr(ops, "guide_backward", guide_backward)
