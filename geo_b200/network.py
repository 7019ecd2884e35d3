"""The models the headline benchmarks are quoted on.

``CONV_tiny_add_partial`` mirrors the reference's 4-layer SC CNN (network.py:126-190; the
training default of main_conv.py), ``VGG16_add_partial`` its VGG-16 (network.py:12-124) and
``CONV_minimal_add_partial`` its LeNet (network.py:192-235): same attribute names (hence the same
state-dict keys), per-layer settings and layer order.  ``VGG11_add_partial`` is the VGG-11-style SC CNN
used for the data-parallel configuration; the reference has no such model file, it is built from the
same layers in the same conv -> BN -> (pool) -> hardtanh order.
"""
from __future__ import annotations

import torch.nn as nn
import torch.nn.functional as F

from . import layers


def _per_layer(values, n):
    values = list(values)
    if len(values) < n:
        values = values + [values[-1]] * (n - len(values))
    return values


class CONV_tiny_add_partial(nn.Module):
    """conv 3->32 5x5, conv 32->32 5x5, conv 32->64 5x5 (each: BN, 2x2 average pool, hardtanh(0,1)),
    then a 4x4 conv 64->classes and a 1d BN.  Per-layer stream length exponent ``err``, OR width
    exponent ``z_unit``, ``load_unit`` and ``load_wait`` are lists indexed by layer, assigned after
    construction exactly as main_conv.py:178-182 does."""

    def __init__(self, num_classes=10, c_ins=3, uniform=False, generator="lfsr", sc_compute="1d_bin", legacy=False,
                 relu=False):
        super().__init__()
        self.bn1 = layers.BatchNorm2d_fixed(32)
        self.bn2 = layers.BatchNorm2d_fixed(32)
        self.bn3 = layers.BatchNorm2d_fixed(64)
        self.bn4 = layers.BatchNorm1d_fixed(num_classes)
        self.conv1 = layers.Conv2d_Add_Partial(3, 32, kernel_size=5, padding=2, bias=False)
        self.conv2 = layers.Conv2d_Add_Partial(32, 32, kernel_size=5, padding=2, bias=False)
        self.conv3 = layers.Conv2d_Add_Partial(32, 64, kernel_size=5, padding=2, bias=False)
        self.fc1 = layers.Conv2d_Add_Partial(64, num_classes, kernel_size=4, padding=0, bias=False)
        self.tanh = nn.Hardtanh(0, 1)
        self.pool = nn.AvgPool2d(2)
        self.pool_tanh = layers.AvgPool2Hardtanh()   # pool followed by tanh, fused
        self.err = [7, 7, 7, 7]
        self.z_unit = [3, 3, 4, 4]
        self.load_unit = [2, 2, 2, 2]
        self.load_wait = [2, 2, 2, 2]
        self.num_classes = num_classes
        self.generator = generator
        self.compute = sc_compute
        self.legacy = legacy
        self.relu = relu
        if uniform:  # larger weights for very short streams (network.py:153-158)
            for conv in (self.conv1, self.conv2):
                conv.weight_org *= 2
                conv.weight.data *= 2

    def _sc_kwargs(self, i):
        # The last layer takes its weight load_wait from entry 2 and its activation load_wait from
        # entry 3 (network.py:186); kept so that per-layer settings mean the same thing.
        wait_w = self.load_wait[2] if i == 3 else self.load_wait[i]
        return dict(err=self.err[i], forward=self.compute, generator=self.generator, z_unit=2 ** self.z_unit[i],
                    legacy=self.legacy, load_unit=self.load_unit[i], load_wait_w=wait_w, load_wait_a=self.load_wait[i])

    def _sc(self, conv, x, i, astreams=None):
        return conv(x, astreams=astreams, **self._sc_kwargs(i))

    def forward(self, x_in, target=None):
        x, streams = x_in, None
        convs = (self.conv1, self.conv2, self.conv3, self.fc1)
        for i, (conv, bn) in enumerate(((self.conv1, self.bn1), (self.conv2, self.bn2), (self.conv3, self.bn3))):
            if self.relu:
                x = self.tanh(self.pool(F.relu(bn(self._sc(conv, x, i, streams)))))
                streams = None
            else:
                # tanh(pool(bn(conv(x)))) and the next layer's input rounding and stream generation, one pass
                # from bit counts to streams where the shapes allow
                x, streams = layers.sc_block(conv, bn, x, self._sc_kwargs(i), convs[i + 1], self._sc_kwargs(i + 1),
                                             astreams=streams)
        x = self._sc(self.fc1, x, 3, streams).view(-1, self.num_classes)
        return self.bn4(x)  # BN at the output stabilises training (network.py:188-189)


class VGG11_add_partial(nn.Module):
    """VGG-11-style SC CNN for 32x32 inputs: eight 3x3 SC convs (64,128,256,256,512,512,512,512;
    2x2 average pool after convs 1,2,4,6,8), then three SC layers 512->512->512->classes written as
    1x1 convs on the 1x1 feature map."""

    WIDTHS = (64, 128, 256, 256, 512, 512, 512, 512)
    POOL_AFTER = (0, 1, 3, 5, 7)

    def __init__(self, num_classes=10, generator="lfsr", sc_compute="1d_bin", legacy=False):
        super().__init__()
        convs, bns, c = [], [], 3
        for wd in self.WIDTHS:
            convs.append(layers.Conv2d_Add_Partial(c, wd, kernel_size=3, padding=1, bias=False))
            bns.append(layers.BatchNorm2d_fixed(wd))
            c = wd
        self.convs = nn.ModuleList(convs)
        self.bns = nn.ModuleList(bns)
        self.fc1 = layers.Conv2d_Add_Partial(512, 512, kernel_size=1, padding=0, bias=False)
        self.fc2 = layers.Conv2d_Add_Partial(512, 512, kernel_size=1, padding=0, bias=False)
        self.fc3 = layers.Conv2d_Add_Partial(512, num_classes, kernel_size=1, padding=0, bias=False)
        self.bnf1 = layers.BatchNorm2d_fixed(512)
        self.bnf2 = layers.BatchNorm2d_fixed(512)
        self.bn_out = layers.BatchNorm1d_fixed(num_classes)
        self.tanh = nn.Hardtanh(0, 1)
        self.pool_tanh = layers.AvgPool2Hardtanh()
        n = len(self.WIDTHS) + 3
        self.err = [7] * n
        self.z_unit = [4] * n
        self.load_unit = [2] * n
        self.load_wait = [2] * n
        self.num_classes = num_classes
        self.generator = generator
        self.compute = sc_compute
        self.legacy = legacy

    def _sc_kwargs(self, i):
        err, zu = _per_layer(self.err, i + 1)[i], _per_layer(self.z_unit, i + 1)[i]
        lu, lw = _per_layer(self.load_unit, i + 1)[i], _per_layer(self.load_wait, i + 1)[i]
        return dict(err=err, forward=self.compute, generator=self.generator, z_unit=2 ** zu, legacy=self.legacy,
                    load_unit=lu, load_wait_w=lw, load_wait_a=lw)

    def _sc(self, conv, x, i, astreams=None):
        return conv(x, astreams=astreams, **self._sc_kwargs(i))

    def forward(self, x, target=None):
        streams = None
        sc_layers = list(self.convs) + [self.fc1]
        for i, (conv, bn) in enumerate(zip(self.convs, self.bns)):
            if i in self.POOL_AFTER:
                x, streams = layers.sc_block(conv, bn, x, self._sc_kwargs(i), sc_layers[i + 1], self._sc_kwargs(i + 1),
                                             astreams=streams)
            else:
                x = self.tanh(bn(self._sc(conv, x, i, streams)))
                streams = None
        n = len(self.convs)
        x = self.tanh(self.bnf1(self._sc(self.fc1, x, n, streams)))
        x = self.tanh(self.bnf2(self._sc(self.fc2, x, n + 1)))
        x = self._sc(self.fc3, x, n + 2).view(-1, self.num_classes)
        return self.bn_out(x)



class VGG16_add_partial(nn.Module):
    """VGG-16 for SC (network.py:12-124).  ``err`` / ``z_unit`` / ``load_unit`` / ``load_wait`` hold six values:
    for conv1-2, conv3-4, conv5-7, conv8-10, conv11-13 and the classifier.  With ``half_pool`` the conv in
    front of a pooling layer runs at half the stream length (not below 32)."""

    WIDTHS = (64, 64, 128, 128, 256, 256, 256, 512, 512, 512, 512, 512, 512)
    STAGE = (0, 0, 1, 1, 2, 2, 2, 3, 3, 3, 4, 4, 4)          # index into the per-stage settings
    POOL_AFTER = (2, 4, 7, 10, 13)                           # 1-based conv numbers followed by pool + dropout

    def __init__(self, uniform=False, sc_compute="1d_bin", generator="lfsr", legacy=False, half_pool=True):
        super().__init__()
        c = 3
        for i, wd in enumerate(self.WIDTHS, start=1):
            setattr(self, f"conv{i}", layers.Conv2d_Add_Partial(c, wd, kernel_size=3, padding=1, bias=False))
            setattr(self, f"bn{i}", layers.BatchNorm2d_fixed(wd))
            c = wd
        for i in range(1, 6):
            setattr(self, f"drop{i}", nn.Dropout2d())
        self.fc1 = layers.Conv2d_Add_Partial(512, 10, kernel_size=1, padding=0, bias=False)
        self.bnfc1 = layers.BatchNorm1d_fixed(10)
        self.pool = nn.AvgPool2d(2)
        self.tanh = nn.Hardtanh(0, 1)
        self.err = [7] * 6
        self.z_unit = [5] * 6
        self.load_unit = [2] * 6
        self.load_wait = [2] * 6
        self.generator = generator
        self.compute = sc_compute
        self.legacy = legacy
        self.half_pool = half_pool
        if min(self.err) < 4:   # larger weights for very short streams (network.py:66-73)
            uniform = True
        if uniform:
            for mod in self.modules():
                if isinstance(mod, nn.Conv2d):
                    mod.weight.data.uniform_()
                    mod.weight_org.uniform_()

    def _sc(self, conv, x, stage, err):
        return conv(x, err=err, forward=self.compute, generator=self.generator, z_unit=2 ** self.z_unit[stage],
                    legacy=self.legacy, load_unit=self.load_unit[stage], load_wait_w=self.load_wait[stage],
                    load_wait_a=self.load_wait[stage])

    def forward(self, x):
        pool_offset = 1 if self.half_pool else 0
        drop = 0
        for i, stage in enumerate(self.STAGE, start=1):
            pooled = i in self.POOL_AFTER
            err = max(self.err[stage] - pool_offset, 5) if pooled else self.err[stage]
            x = self._sc(getattr(self, f"conv{i}"), x, stage, err)
            bn = getattr(self, f"bn{i}")
            if pooled:
                x = layers.bn_pool_hardtanh(bn, x)      # tanh(pool(bn(x)))
                drop += 1
                x = getattr(self, f"drop{drop}")(x)
            else:
                x = self.tanh(bn(x))
        x = self._sc(self.fc1, x, 5, self.err[5]).view(-1, 10)
        return self.bnfc1(x)  # BN at the output stabilises training


class CONV_minimal_add_partial(nn.Module):
    """LeNet for SC on 28x28 single-channel inputs, stream length 32 everywhere (network.py:192-235).  The
    reference's forward ends without a return statement; this one returns the logits."""

    def __init__(self, uniform=False, legacy=False, generator="lfsr", sc_compute="1d_bin"):
        super().__init__()
        self.bn1 = layers.BatchNorm2d_fixed(6)
        self.bn2 = layers.BatchNorm2d_fixed(16)
        self.conv1 = layers.Conv2d_Add_Partial(1, 6, kernel_size=5, padding=2, bias=False)
        self.conv2 = layers.Conv2d_Add_Partial(6, 16, kernel_size=5, padding=0, bias=False)
        self.fc1 = layers.Linear_Or(5 * 5 * 16, 120, bias=False)
        self.fc2 = layers.Linear_Or(120, 84, bias=False)
        self.fc3 = layers.Linear_Or(84, 10, bias=False)
        self.bn = layers.BatchNorm1d_fixed(10, affine=False)
        self.pool = nn.AvgPool2d(2)
        self.tanh = nn.Hardtanh(0, 1)
        self.generator = generator
        self.compute = sc_compute
        if uniform:
            for conv in (self.conv1, self.conv2):
                conv.weight_org *= 2
                conv.weight.data *= 2
        self.err = 5
        self.legacy = legacy

    def forward(self, x):
        for conv, bn in ((self.conv1, self.bn1), (self.conv2, self.bn2)):
            x = conv(x, err=self.err, forward=self.compute, generator=self.generator, legacy=self.legacy)
            x = self.tanh(bn(self.pool(x)))
        x = x.reshape(-1, 16 * 5 * 5)
        x = self.tanh(self.fc1(x, err=self.err, generator=self.generator))
        x = self.tanh(self.fc2(x, err=self.err, generator=self.generator))
        x = self.fc3(x, err=self.err, generator=self.generator)
        return self.bn(x)
