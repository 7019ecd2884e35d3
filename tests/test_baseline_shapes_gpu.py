"""Bit-exact parity at the sizes the headline numbers are quoted on: the single conv (32x3x32x32, 5x5, L=64),
every layer of the 4-layer CNN at batch 256, the 1024x4096 . 4096x4096 linear layer at four stream lengths, the
256x256x16x16 3x3 layer at L=256 in every mode, and the widest layers of the VGG-11-style network.

The CUDA path runs the whole layer; the CPU oracle checks slices of it.  That is a complete check of the sliced
outputs and not an approximation: activation generators restart for every image (sc_cuda_kernel.cu:667-670) and
weight generators do not depend on the output channel (:1757-1763), so an (images, output channels) slice of a
full run equals the oracle run on those images and filters alone.  Slices are chosen to land in the first,
a middle and the last position tile, channel tile and grid.z split of the kernels."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


def _inputs(ashape, wshape, seed, wscale=1.0, levels=128):
    g = torch.Generator().manual_seed(seed)
    a = (torch.rand(*ashape, generator=g) * levels).round().clamp(0, levels - 1) / levels
    w = q7((torch.rand(*wshape, generator=g) * 2 - 1) * wscale)
    return a, w


def _check_slices(oracle_lib, y, a, w, L, mode, pad, slices, **kw):
    for b, o in slices:
        ref = oracle_lib.conv2d(a[b], w[o], L, mode, pad_h=pad[0], pad_w=pad[1], **kw)
        got = y[b][:, o].cpu().numpy()
        assert got.shape == ref.shape
        assert np.array_equal(got, ref), f"{mode} L={L} images {b} channels {o}: max diff {np.abs(got - ref).max()}"


_REF_CPU_SCRIPT = """
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from oracle import ref_loader
ext = ref_loader.ref_sc_extension()
if ext is None:
    sys.exit(3)
d = np.load(sys.argv[2])
y = ext.conv2d_add_partial_new(torch.from_numpy(d["a"]), torch.from_numpy(d["w"]), int(d["L"]), (int(d["pad"]),) * 2, (1, 1))
np.save(sys.argv[3], y.numpy())
"""


def _reference_cpu_kernel(a, w, L, pad, tmp_path):
    """Output of the reference's own CPU kernel (sc.cpp built unmodified), or None where that build is absent.  Run
    in a process of its own: its module is called sc_extension like one of this repository's torch shims, and one
    process cannot hold both."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    inp, out = str(tmp_path / "in.npz"), str(tmp_path / "out.npy")
    np.savez(inp, a=a.numpy(), w=w.numpy(), L=L, pad=pad)
    r = subprocess.run([sys.executable, "-c", _REF_CPU_SCRIPT, root, inp, out], capture_output=True, text=True, timeout=600)
    if r.returncode == 3:
        return None
    assert r.returncode == 0, r.stderr[-2000:]
    return np.load(out)


def test_c1_single_conv_whole_layer(cuda_device, oracle_lib, tmp_path):
    """32x3x32x32 . 32x3x5x5, pad 2, L=64, activations on 1/64 levels, 1d_bin, no progressive loading: the whole
    output against the oracle and, where it is built, against the reference's CPU kernel itself."""
    from geo_b200 import ops

    a, w = _inputs((32, 3, 32, 32), (32, 3, 5, 5), 0, levels=64)
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 64, "1d_bin", (2, 2)).cpu()
    assert np.array_equal(y.numpy(), oracle_lib.conv2d(a, w, 64, "1d_bin", pad_h=2, pad_w=2))
    ref = _reference_cpu_kernel(a, w, 64, 2, tmp_path)
    if ref is not None:
        assert np.array_equal(y.numpy(), ref)
    # the mode the configuration's prose describes (OR inside a channel, binary across channels) is z_bin
    yz = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 64, "z_bin", (2, 2)).cpu().numpy()
    assert np.array_equal(yz, oracle_lib.conv2d(a, w, 64, "z_bin", pad_h=2, pad_w=2))


C2_LAYERS = [
    # act, weight, pad, slices of (images, output channels)
    ((256, 3, 32, 32), (32, 3, 5, 5), (2, 2), [(slice(0, 2), slice(0, 32)), (slice(127, 128), slice(5, 9)),
                                               (slice(255, 256), slice(28, 32))]),
    ((256, 32, 16, 16), (32, 32, 5, 5), (2, 2), [(slice(0, 1), slice(0, 32)), (slice(100, 101), slice(14, 18)),
                                                 (slice(255, 256), slice(29, 32))]),
    ((256, 32, 8, 8), (64, 32, 5, 5), (2, 2), [(slice(0, 2), slice(0, 64)), (slice(77, 79), slice(30, 35)),
                                               (slice(254, 256), slice(60, 64))]),
    ((256, 64, 4, 4), (10, 64, 4, 4), (0, 0), [(slice(0, 256), slice(0, 10))]),
]


@pytest.mark.parametrize("layer", range(4))
def test_c2_training_layers_at_batch_256(cuda_device, oracle_lib, layer):
    """The four layers of the 4-layer CNN as trained: batch 256, L=128, 1d_bin, load_unit = load_wait = 2."""
    from geo_b200 import ops

    ashape, wshape, pad, slices = C2_LAYERS[layer]
    a, w = _inputs(ashape, wshape, 20 + layer, wscale=0.4)
    kw = dict(total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 128, "1d_bin", pad, **kw)
    _check_slices(oracle_lib, y, a, w, 128, "1d_bin", pad, slices, **kw)


@pytest.mark.parametrize("L", [32, 64, 128, 256])
def test_c3_linear_1024x4096(cuda_device, oracle_lib, L):
    """activations 1024x4096, weights 4096x4096, OR in groups of 16 inputs, popcount across the 256 groups."""
    from geo_b200 import ops

    g = torch.Generator().manual_seed(300 + L)
    a = q7(torch.rand(1024, 4096, generator=g))
    w = q7(torch.rand(4096, 4096, generator=g) * 2 - 1)
    y = ops.sc_linear(a.to(cuda_device), w.to(cuda_device), L, z_unit=16).cpu().numpy()
    assert y.shape == (1024, 4096)
    for rows, cols in [(slice(0, 3), slice(0, 64)), (slice(511, 514), slice(2040, 2056)),
                       (slice(1021, 1024), slice(4090, 4096)), (slice(700, 701), slice(1000, 1256))]:
        assert np.array_equal(y[rows, cols], oracle_lib.linear(a[rows], w[cols], L, z_unit=16))


C4_SLICES = [(slice(0, 1), slice(0, 8)), (slice(128, 129), slice(126, 131)), (slice(255, 256), slice(250, 256)),
             (slice(37, 38), slice(60, 68))]


@pytest.mark.parametrize("mode", ["1d_bin", "full_or", "z_bin", "yz_bin", "2d_bin", "full_bin"])
def test_c4_largest_layer(cuda_device, oracle_lib, mode):
    """256x256x16x16 . 256x256x3x3, pad 1, L=256: groups of 768 (1d_bin: 5 sorted chunks) and 2304 members
    (full_or: 15 chunks), 256 members (2d_bin), 144 (yz_bin, z=16), 9 (z_bin) and 1 (full_bin)."""
    from geo_b200 import ops

    a, w = _inputs((256, 256, 16, 16), (256, 256, 3, 3), 400)
    kw = dict(z_unit=16) if mode == "yz_bin" else {}
    ad, wd = a.to(cuda_device), w.to(cuda_device)
    y = ops.sc_conv2d(ad, wd, 256, mode, (1, 1), **kw)
    _check_slices(oracle_lib, y, a, w, 256, mode, (1, 1), C4_SLICES, **kw)
    if mode == "1d_bin":   # any batch split gives the same per-image result
        perm = torch.randperm(256, generator=torch.Generator().manual_seed(1))
        y2 = ops.sc_conv2d(ad[perm.to(cuda_device)], wd, 256, mode, (1, 1), **kw)
        assert torch.equal(y2, y[perm.to(cuda_device)])


def test_c4_ragged_output_channels(cuda_device, oracle_lib):
    """The same layer with 250 output channels: the last 32-channel tile of the sign-sorted kernel is partial."""
    from geo_b200 import ops

    a, w = _inputs((64, 256, 16, 16), (250, 256, 3, 3), 401)
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 256, "1d_bin", (1, 1))
    _check_slices(oracle_lib, y, a, w, 256, "1d_bin", (1, 1),
                  [(slice(0, 1), slice(0, 6)), (slice(63, 64), slice(244, 250)), (slice(31, 32), slice(222, 226))])


C5_LAYERS = [
    # the widest layers of the VGG-11-style network at 256 images per GPU (L=128, 1d_bin, load 2/2)
    ((256, 512, 4, 4), (512, 512, 3, 3), (1, 1)),     # conv6: 1536 members per group
    ((256, 512, 2, 2), (512, 512, 3, 3), (1, 1)),     # conv7/8: 2x2 images, four positions per image
    ((256, 512, 1, 1), (512, 512, 1, 1), (0, 0)),     # the 512 -> 512 classifier layers as 1x1 convs
    ((256, 64, 16, 16), (128, 64, 3, 3), (1, 1)),     # conv2: 192 members
]


@pytest.mark.parametrize("layer", range(len(C5_LAYERS)))
def test_c5_vgg11_layers(cuda_device, oracle_lib, layer):
    from geo_b200 import ops

    ashape, wshape, pad = C5_LAYERS[layer]
    a, w = _inputs(ashape, wshape, 500 + layer, wscale=0.25)
    kw = dict(total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 128, "1d_bin", pad, **kw)
    O = wshape[0]
    _check_slices(oracle_lib, y, a, w, 128, "1d_bin", pad,
                  [(slice(0, 2), slice(0, 8)), (slice(130, 132), slice(O // 2 - 3, O // 2 + 3)),
                   (slice(254, 256), slice(O - 5, O))], **kw)
