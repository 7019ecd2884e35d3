"""CPU training step of the 4-layer SC CNN, for the timed CPU baseline.  TEST INFRASTRUCTURE ONLY.

A self-contained restatement (plain PyTorch CPU ops, nothing from the product package) of what
the reference does for one batch on the CPU: ``network.CONV_tiny_add_partial.forward``
(network.py:164-190) with ``Conv2d_Add_Partial`` (utils_class.py:11-35) calling
``conv2d_generic`` (utils_functional.py:489-494 -> ``sc_extension.conv2d_add_partial_new``),
``BatchNorm*_fixed`` (utils_class.py:37-93), scaled cross-entropy, backward through the float
guide (utils_functional.py:235-252,611-634) and an SGD update of an fp32 master copy
(utils_own.py:81-114).  The SC forward is the reference's own CPU kernel (``sc.cpp`` built
unmodified into oracle/_ref) when it is available, else the C restatement in ``sc_oracle.c``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import guide


def _q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


def _quantize_shift(t, scale=None):
    if scale is None:
        scale = 2 ** torch.ceil(torch.log2(torch.mean(t) * 3))
    return ((t / scale) * 128).round().clamp(-127, 127) / 128 * scale, scale


def sc_forward_fn():
    """(callable, kind): SC 1d_bin forward on CPU tensors -> int32 counts."""
    from . import ref_loader

    ext = ref_loader.ref_sc_extension()
    if ext is not None:
        return (lambda a, w, L, pad: ext.conv2d_add_partial_new(a, w, L, (pad, pad), (1, 1))), "reference"
    import oracle

    def port(a, w, L, pad):
        return torch.from_numpy(oracle.conv2d(a, w, L, "1d_bin", pad_h=pad, pad_w=pad))

    return port, "port"


class CpuTinyCNN:
    LAYERS = ((3, 32, 5, 2), (32, 32, 5, 2), (32, 64, 5, 2), (64, 10, 4, 0))

    def __init__(self, bit_length=128, seed=0, lr=2e-3):
        g = torch.Generator().manual_seed(seed)
        self.L = bit_length
        self.weight_org, self.bn_w, self.bn_b = [], [], []
        for cin, cout, k, _ in self.LAYERS:
            bound = 1.0 / (cin * k * k) ** 0.5  # nn.Conv2d default init (Kaiming uniform, a=sqrt(5))
            self.weight_org.append((torch.rand(cout, cin, k, k, generator=g) * 2 - 1) * bound)
            self.bn_w.append(torch.ones(cout))
            self.bn_b.append(torch.zeros(cout))
        self.sc, self.kind = sc_forward_fn()
        self.master = [w.clone().requires_grad_(True) for w in self.weight_org + self.bn_w + self.bn_b]
        self.opt = torch.optim.SGD(self.master, lr=lr, momentum=0.01)

    def _bn_fixed(self, x, w, b, dims):
        out = F.batch_norm(x, None, None, w, b, training=True)
        mean, var = x.mean(dim=dims), x.var(dim=dims, unbiased=False)
        inv = torch.sqrt(var + 1e-5)
        w_n, scale = _quantize_shift((w.data / inv).detach())
        b_n, _ = _quantize_shift((b.data - mean * w.data / inv).detach(), scale)
        shape = (-1, 1, 1) if x.dim() == 4 else (-1,)
        out.data = x.data * w_n.reshape(shape) + b_n.reshape(shape)
        return out

    def step(self, inputs, targets):
        ws = [_q7(w).requires_grad_(True) for w in self.weight_org]
        bw = [t.clone().requires_grad_(True) for t in self.bn_w]
        bb = [t.clone().requires_grad_(True) for t in self.bn_b]
        x = inputs
        for i, (_, _, _, pad) in enumerate(self.LAYERS):
            x.data = _q7(x.data)
            counts = self.sc(x.data, ws[i].data, self.L, pad)
            x = guide.guide_output(x, ws[i], "1d_bin", pad, pad, sc_value=counts.float() / self.L)
            if i < 3:
                x = self._bn_fixed(x, bw[i], bb[i], (0, 2, 3))
                x = F.hardtanh(F.avg_pool2d(x, 2), 0, 1)
            else:
                x = self._bn_fixed(x.view(-1, 10), bw[i], bb[i], (0,))
        loss = F.cross_entropy(x, targets) * 128.0
        grads = torch.autograd.grad(loss, ws + bw + bb)
        for m, gr in zip(self.master, grads):
            m.grad = gr / 128.0
        self.opt.step()
        n = len(ws)
        with torch.no_grad():
            for i in range(n):
                self.weight_org[i] = self.master[i].data.clamp(-1, 0.999).clone()
                self.bn_w[i] = self.master[n + i].data.clone()
                self.bn_b[i] = self.master[2 * n + i].data.clone()
        return float(loss.detach())
