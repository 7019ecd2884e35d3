"""Bit-exact parity of the CUDA path (called through the C ABI) with the CPU oracle and the
golden vectors generated from the reference."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MODE_NAMES = {0: "1d_bin", 1: "z_bin", 2: "yz_bin", 3: "full_or", 4: "2d_bin", 5: "full_bin"}


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


def _rand(ashape, wshape, seed, quant=True):
    g = torch.Generator().manual_seed(seed)
    a = torch.rand(*ashape, generator=g)
    w = torch.rand(*wshape, generator=g) * 2 - 1
    return (q7(a), q7(w)) if quant else (a, w)


@pytest.mark.parametrize("L", [8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("mode", ["1d_bin", "z_bin", "yz_bin", "full_or", "2d_bin", "full_bin"])
def test_stream_words_match_oracle(cuda_device, oracle_lib, L, mode):
    from geo_b200 import ops

    a, w = _rand((2, 5, 6, 7), (9, 5, 3, 2), 11 + L)
    for (tw, lu, lww, lwa) in [(7, 8, 1, 1), (7, 2, 2, 2), (7, 1, 3, 5)]:
        kw = dict(z_unit=2, total_width=tw, load_width=lu, load_wait_w=lww, load_wait_a=lwa)
        d = ops.desc_for(a, w, L, mode, (1, 2), **kw)
        asg = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d), d).cpu().numpy()
        wsg = ops.weight_streams_canonical(ops.prepare_weights(w.to(cuda_device), d), d).cpu().numpy()
        aso = oracle_lib.act_streams(oracle_lib.pad_act(a, 1, 2), L, mode, 2, tw, lu, lwa)
        wso = oracle_lib.weight_streams(w, L, mode, 2, tw, lu, lww)
        assert np.array_equal(asg.view(np.uint32), aso)
        assert np.array_equal(wsg.view(np.uint32), wso)


def test_stream_words_of_a_linear_layer_match_oracle(cuda_device, oracle_lib):
    """1x1 images: the stream image is laid out [pack][c][batch]; its words are the oracle's all the same."""
    from geo_b200 import ops

    for B in (5, 8, 203):
        a, w = _rand((B, 12, 1, 1), (9, 12, 1, 1), 77 + B)
        for mode in ("yz_bin", "1d_bin", "full_bin"):
            kw = dict(z_unit=4, total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
            d = ops.desc_for(a, w, 128, mode, (0, 0), **kw)
            asg = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d), d).cpu().numpy()
            aso = oracle_lib.act_streams(oracle_lib.pad_act(a, 0, 0), 128, mode, 4, 7, 2, 2)
            assert np.array_equal(asg.view(np.uint32), aso)
            y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 128, mode, (0, 0), **kw).cpu().numpy()
            assert np.array_equal(y, oracle_lib.conv2d(a, w, 128, mode, pad_h=0, pad_w=0, **kw))


SHAPES = [
    # act, weight, (pad_h, pad_w)
    ((2, 3, 7, 6), (3, 3, 3, 2), (0, 0)),
    ((1, 1, 5, 5), (1, 1, 1, 1), (0, 0)),
    ((3, 5, 9, 8), (7, 5, 2, 4), (1, 0)),
    ((2, 8, 12, 12), (33, 8, 3, 3), (1, 1)),      # 33 output channels: partial 64-wide tile
    ((5, 4, 11, 13), (17, 4, 5, 5), (2, 2)),      # 17 output channels -> 32-wide tile, ragged positions
    ((2, 6, 10, 10), (70, 6, 3, 3), (0, 0)),      # two c_out tiles
    ((3, 16, 4, 4), (10, 16, 4, 4), (0, 0)),      # one position per image, 16-wide tile
    ((1, 40, 6, 6), (8, 40, 3, 3), (1, 1)),       # 120 members per group: several chunks per group
    ((3, 16, 10, 10), (40, 16, 5, 5), (2, 2)),    # long groups, 2 c_out tiles of 32: sign-sorted kernel, ragged tiles
    ((2, 64, 8, 8), (32, 64, 5, 5), (2, 2)),      # 320 members per group: two sorted chunks (1600 = 9 in full_or)
]


@pytest.mark.parametrize("mode", ["1d_bin", "z_bin", "yz_bin", "full_or", "2d_bin", "full_bin"])
@pytest.mark.parametrize("case", range(len(SHAPES)))
def test_conv_matches_oracle(cuda_device, oracle_lib, mode, case):
    from geo_b200 import ops

    ashape, wshape, pad = SHAPES[case]
    for L, (lu, lw) in [(128, (2, 2)), (32, (8, 1)), (256, (8, 1)), (64, (3, 4))]:
        a, w = _rand(ashape, wshape, 100 * case + L, quant=(L != 64))
        kw = dict(z_unit=4, total_width=7, load_width=lu, load_wait_w=lw, load_wait_a=lw)
        y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, pad, **kw).cpu().numpy()
        ref = oracle_lib.conv2d(a, w, L, mode, pad_h=pad[0], pad_w=pad[1], **kw)
        assert y.shape == ref.shape
        assert np.array_equal(y, ref), f"{mode} case {case} L={L}: {np.abs(y - ref).max()} max diff"


def test_random_shapes_modes_and_plans(cuda_device, oracle_lib):
    """Forty seeded random configurations (shape, mode, stream length, loading plan, a third of the weights
    zero) against the oracle; both accumulate kernels are hit (long and short groups)."""
    import random

    from geo_b200 import _lib, ops

    rng = random.Random(5)
    kernels = set()
    for it in range(40):
        mode = rng.choice(["1d_bin", "full_or", "yz_bin", "2d_bin", "z_bin"])
        C, O = rng.choice([8, 16, 24, 40, 64, 100]), rng.choice([17, 32, 33, 48, 64, 70, 96])
        K2, K3 = rng.choice([(3, 3), (5, 5), (1, 1), (2, 4), (3, 1)])
        H, W, B = rng.choice([6, 8, 9, 12]), rng.choice([6, 8, 10, 12]), rng.choice([2, 3, 5, 9])
        ph, pw = rng.choice([(0, 0), (1, 1), (2, 1)])
        L, z = rng.choice([32, 64, 128, 256]), rng.choice([4, 8, 16])
        lu, lw = rng.choice([(8, 1), (2, 2), (1, 3)])
        if H + 2 * ph < K2 or W + 2 * pw < K3:
            continue
        g = torch.Generator().manual_seed(it)
        a = q7(torch.rand(B, C, H, W, generator=g))
        w = q7(torch.rand(O, C, K2, K3, generator=g) * 2 - 1)
        w.view(-1)[::3] = 0
        kw = dict(z_unit=z, total_width=7, load_width=lu, load_wait_w=lw, load_wait_a=lw)
        kernels.add(_lib.is_sign_sorted(ops.desc_for(a, w, L, mode, (ph, pw), **kw)))
        y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, (ph, pw), **kw).cpu().numpy()
        assert np.array_equal(y, oracle_lib.conv2d(a, w, L, mode, pad_h=ph, pad_w=pw, **kw)), (it, mode, L)
    assert kernels == {True, False}


SHORT_GROUP_CASES = [
    # act, weight, pad, mode, z_unit, L: members per group as laid out / what the case is for
    ((4, 3, 8, 8), (8, 3, 1, 3), (0, 1), "1d_bin", 1, 128),      # 3 -> 4 members, one stage per group
    ((4, 2, 8, 8), (20, 2, 3, 3), (1, 1), "1d_bin", 1, 64),      # 6 -> 8
    ((4, 3, 8, 8), (33, 3, 3, 3), (1, 1), "1d_bin", 1, 128),     # 9 -> 12, ragged c_out
    ((4, 3, 10, 8), (32, 3, 5, 5), (2, 2), "1d_bin", 1, 128),    # 15 -> 16: first layer of the 4-layer CNN
    ((3, 6, 9, 12), (16, 6, 5, 5), (2, 2), "z_bin", 1, 32),      # 25 -> 32: two chunks per group
    ((3, 32, 8, 8), (40, 32, 3, 3), (1, 1), "yz_bin", 16, 256),  # 48: three chunks per group
    ((3, 32, 8, 8), (12, 32, 3, 3), (1, 1), "full_or", 1, 128),  # 288 members, c_out padded to 16: six quads' worth of chunks
    ((4, 130, 8, 8), (16, 130, 3, 3), (1, 1), "z_bin", 1, 256),  # P * G * 32 = 33 280: 32-bit running sums
    ((3, 5, 7, 20), (16, 5, 3, 3), (0, 0), "2d_bin", 1, 64),     # ragged last position tile (M = 270)
    ((300, 64, 1, 1), (40, 64, 1, 1), (0, 0), "yz_bin", 16, 128),  # linear layer: batch-innermost image, 16-byte copies, ragged tile
    ((256, 40, 1, 1), (24, 40, 1, 1), (0, 0), "yz_bin", 8, 32),    # linear layer, 8-member groups
    ((203, 24, 1, 1), (16, 24, 1, 1), (0, 0), "yz_bin", 12, 64),   # linear layer, batch not a multiple of 4
]


@pytest.mark.parametrize("case", range(len(SHORT_GROUP_CASES)))
def test_short_group_kernel_matches_oracle(cuda_device, oracle_lib, case):
    """The sign-sorted kernel for short groups at every stage length (4, 8, 12, 16 members), with one and
    several chunks per group, packed and 32-bit running sums, and zero weights (dropped from its lists)."""
    from geo_b200 import _lib, ops

    ashape, wshape, pad, mode, z, L = SHORT_GROUP_CASES[case]
    a, w = _rand(ashape, wshape, 900 + case)
    w.view(-1)[::5] = 0
    kw = dict(z_unit=z, total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
    d = ops.desc_for(a, w, L, mode, pad, **kw)
    assert _lib.is_sign_sorted(d)
    geom = _lib.group_geometry_full(d)
    assert geom[2] < 64 or geom[4] == 16   # short groups as laid out, or a c_out padded to 16
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, pad, **kw).cpu().numpy()
    assert np.array_equal(y, oracle_lib.conv2d(a, w, L, mode, pad_h=pad[0], pad_w=pad[1], **kw))


TAP_TILE_CASES = [
    # act, weight, pad, mode, L
    ((2, 64, 8, 8), (40, 64, 3, 3), (1, 1), "1d_bin", 128),      # one tile mixes every border class (union of live taps)
    ((5, 64, 6, 7), (64, 64, 3, 3), (1, 1), "full_or", 64),      # batch padded 5 -> 8, non-square image
    ((18, 100, 4, 4), (96, 100, 3, 3), (1, 1), "1d_bin", 128),   # 100 channels: ragged last channel chunk
    ((66, 200, 2, 2), (64, 200, 3, 3), (1, 1), "2d_bin", 32),    # 2x2 images: most taps dead; three chunks per tap
    ((12, 64, 5, 5), (33, 64, 5, 5), (2, 2), "1d_bin", 256),     # 5x5 filter, ragged c_out
    ((31, 64, 6, 6), (32, 64, 3, 3), (0, 0), "full_or", 128),    # no padding: no tap is ever dead
    ((6, 64, 3, 9), (64, 64, 3, 3), (2, 1), "1d_bin", 64),       # padding wider than the filter needs: whole groups dead at the border
    ((44, 72, 1, 6), (64, 72, 1, 3), (0, 1), "2d_bin", 128),     # one-row images
    ((64, 128, 4, 4), (128, 128, 3, 3), (1, 1), "1d_bin", 128),  # several tiles, one border class each
]


@pytest.mark.parametrize("case", range(len(TAP_TILE_CASES)))
def test_tap_tile_kernel_matches_oracle(cuda_device, oracle_lib, case):
    """The tap-tile kernel (batch-innermost stream image, dead taps skipped per border class) against the oracle,
    stream words included."""
    from geo_b200 import _lib, ops

    ashape, wshape, pad, mode, L = TAP_TILE_CASES[case]
    a, w = _rand(ashape, wshape, 1300 + case)
    w.view(-1)[::7] = 0
    kw = dict(z_unit=4, total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
    d = ops.desc_for(a, w, L, mode, pad, **kw)
    assert _lib.accumulate_kernel(d) == "sorted_taps"
    assert _lib.act_stream_layout(d) == (True, (ashape[0] + 3) // 4 * 4)
    asg = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d), d).cpu().numpy()
    aso = oracle_lib.act_streams(oracle_lib.pad_act(a, pad[0], pad[1]), L, mode, 4, 7, 2, 2)
    assert np.array_equal(asg.view(np.uint32), aso)
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, pad, **kw).cpu().numpy()
    assert np.array_equal(y, oracle_lib.conv2d(a, w, L, mode, pad_h=pad[0], pad_w=pad[1], **kw))


def test_dense_kernel_on_the_batch_innermost_image(cuda_device, oracle_lib):
    """Layers of the tap-tile kernel whose launch is too small for one of its tiles run on the dense kernel, over
    the same batch-innermost stream image."""
    from geo_b200 import _lib, ops

    for ashape, wshape, pad, mode in [((3, 128, 4, 4), (40, 128, 3, 3), (1, 1), "1d_bin"),
                                      ((2, 64, 5, 3), (32, 64, 3, 3), (1, 1), "full_or"),
                                      ((5, 64, 2, 2), (32, 64, 3, 3), (1, 1), "2d_bin")]:
        a, w = _rand(ashape, wshape, 1700 + ashape[0])
        kw = dict(total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
        d = ops.desc_for(a, w, 128, mode, pad, **kw)
        assert _lib.accumulate_kernel(d) == "dense" and _lib.act_stream_layout(d)[0]
        y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 128, mode, pad, **kw).cpu().numpy()
        assert np.array_equal(y, oracle_lib.conv2d(a, w, 128, mode, pad_h=pad[0], pad_w=pad[1], **kw))


def test_random_configurations_over_every_kernel_family(cuda_device, oracle_lib):
    """150 seeded random configurations drawn per kernel family (wide layers -> tap tiles, narrow long-group layers
    -> row / im2col tiles, short groups, linear layers, anything) with odd batches, ragged c_out, paddings from
    none to wider than the filter needs and zeroed weights, each against the oracle."""
    import random

    from geo_b200 import _lib, ops

    rng = random.Random(20240)
    seen = {}
    done = 0
    while done < 150:
        fam = rng.choice(["taps", "taps", "short", "linear", "rows", "any"])
        if fam == "linear":
            mode = rng.choice(["yz_bin", "1d_bin", "full_or"])
            C, O = rng.choice([16, 48, 64, 100, 256]), rng.choice([10, 16, 40, 64])
            K2 = K3 = H = W = 1
            ph = pw = 0
            B = rng.choice([1, 3, 64, 130, 203, 256, 300])
        else:
            mode = rng.choice({"taps": ["1d_bin", "full_or", "2d_bin"], "rows": ["1d_bin", "full_or", "2d_bin"],
                               "short": ["1d_bin", "z_bin", "yz_bin", "2d_bin"],
                               "any": ["1d_bin", "full_or", "2d_bin", "yz_bin", "z_bin", "full_bin"]}[fam])
            C = rng.choice({"taps": [64, 65, 72, 96, 100, 128, 200], "rows": [16, 24, 32, 40], "short": [1, 2, 3, 4, 6, 8],
                            "any": [3, 8, 20, 64]}[fam])
            O = rng.choice({"taps": [32, 33, 40, 64, 70, 96, 128], "rows": [32, 64, 96], "short": [3, 16, 17, 32, 40, 64],
                            "any": [5, 16, 33, 64]}[fam])
            K2, K3 = rng.choice([(3, 3), (5, 5), (1, 1), (2, 4), (3, 1), (1, 3)])
            H, W = rng.choice([1, 2, 3, 4, 6, 8, 9, 12, 16]), rng.choice([1, 2, 4, 5, 8, 10, 12, 16])
            ph, pw = rng.choice([(0, 0), (1, 1), (2, 2), (2, 1), (0, 1), (3, 0)])
            B = rng.choice([1, 2, 3, 5, 8, 16, 17, 33, 64, 70])
        if H + 2 * ph < K2 or W + 2 * pw < K3:
            continue
        if B * (H + 2 * ph - K2 + 1) * (W + 2 * pw - K3 + 1) * O * C * K2 * K3 > 1.5e8:
            continue
        L, z = rng.choice([8, 32, 64, 128, 256]), rng.choice([1, 2, 4, 8, 16])
        lu, lw = rng.choice([(8, 1), (2, 2), (1, 3)])
        g = torch.Generator().manual_seed(done)
        a = q7(torch.rand(B, C, H, W, generator=g))
        w = q7(torch.rand(O, C, K2, K3, generator=g) * 2 - 1)
        if rng.random() < 0.5:
            w.view(-1)[::rng.choice([2, 3, 5])] = 0
        kw = dict(z_unit=z, total_width=7, load_width=lu, load_wait_w=lw, load_wait_a=lw)
        k = _lib.accumulate_kernel(ops.desc_for(a, w, L, mode, (ph, pw), **kw))
        seen[k] = seen.get(k, 0) + 1
        y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, (ph, pw), **kw).cpu().numpy()
        assert np.array_equal(y, oracle_lib.conv2d(a, w, L, mode, pad_h=ph, pad_w=pw, **kw)), (done, fam, mode, k, a.shape, w.shape)
        done += 1
    assert {"dense", "sorted_short", "sorted_taps", "sorted_im2col"} <= set(seen), seen
    assert _lib.device_error_count() == 0


def test_small_stream_lengths(cuda_device, oracle_lib):
    from geo_b200 import ops

    for L in (8, 16):
        for mode in ("1d_bin", "z_bin", "yz_bin", "full_or", "2d_bin", "full_bin"):
            a, w = _rand((2, 4, 6, 6), (6, 4, 3, 3), L)
            y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, (1, 1), z_unit=2).cpu().numpy()
            assert np.array_equal(y, oracle_lib.conv2d(a, w, L, mode, z_unit=2, pad_h=1, pad_w=1))


def test_golden_reference_cpu_kernel(cuda_device):
    from geo_b200 import ops

    g = np.load(os.path.join(GOLDEN, "ref_cpu_1d.npz"))
    for i in range(int(g["n"])):
        L, p0, p1 = (int(v) for v in g[f"c{i}_meta"])
        y = ops.sc_conv2d(torch.from_numpy(g[f"c{i}_a"]).to(cuda_device), torch.from_numpy(g[f"c{i}_w"]).to(cuda_device),
                          L, "1d_bin", (p1, p0))
        assert np.array_equal(y.cpu().numpy(), g[f"c{i}_y"]), f"case {i}"


def test_golden_reference_bit_serial(cuda_device):
    from geo_b200 import ops

    g = np.load(os.path.join(GOLDEN, "ref_legacy_L128.npz"))
    for i in range(int(g["n"])):
        L, p0, p1, mode = (int(v) for v in g[f"c{i}_meta"])
        y = ops.sc_conv2d(torch.from_numpy(g[f"c{i}_a"]).to(cuda_device), torch.from_numpy(g[f"c{i}_w"]).to(cuda_device),
                          L, MODE_NAMES[mode], (p1, p0))
        assert np.array_equal(y.cpu().numpy(), g[f"c{i}_y"]), f"case {i}"
    a, w = torch.from_numpy(g["lin_a"]), torch.from_numpy(g["lin_w"])
    y = ops.sc_linear(a.to(cuda_device), w.to(cuda_device), 128, z_unit=a.shape[1])
    assert np.array_equal(y.cpu().numpy(), g["lin_y"])


def test_golden_reference_bit_serial_2d_bin(cuda_device):
    """2d_bin through conv2d_generic (the reference's own call: forward='2d_bin') against the outputs of the
    reference's bit-serial simulation."""
    from geo_b200 import functional as sc_f

    g = np.load(os.path.join(GOLDEN, "ref_legacy_2d_L128.npz"))
    for i in range(int(g["n"])):
        L, p0, p1, mode = (int(v) for v in g[f"c{i}_meta"])
        a = torch.from_numpy(g[f"c{i}_a"]).to(cuda_device)
        w = torch.from_numpy(g[f"c{i}_w"]).to(cuda_device)
        y = sc_f.conv2d_generic(a, w, (p0, p1), (1, 1), bit_length=L, forward="2d_bin", generator="lfsr")
        assert np.array_equal((y * L).round().to(torch.int32).cpu().numpy(), g[f"c{i}_y"]), f"case {i}"


def test_golden_reference_bit_serial_full_bin(cuda_device):
    """full_bin through conv2d_generic and linear_generic (the reference's own calls) against the outputs of
    the reference's bit-serial simulation."""
    from geo_b200 import functional as sc_f

    g = np.load(os.path.join(GOLDEN, "ref_legacy_full_bin_L128.npz"))
    for i in range(int(g["n"])):
        L, p0, p1, mode = (int(v) for v in g[f"c{i}_meta"])
        a = torch.from_numpy(g[f"c{i}_a"]).to(cuda_device)
        w = torch.from_numpy(g[f"c{i}_w"]).to(cuda_device)
        y = sc_f.conv2d_generic(a, w, (p0, p1), (1, 1), bit_length=L, forward="full_bin", generator="lfsr")
        assert np.array_equal((y * L).round().to(torch.int32).cpu().numpy(), g[f"c{i}_y"]), f"case {i}"
    a, w = torch.from_numpy(g["lin_a"]).to(cuda_device), torch.from_numpy(g["lin_w"]).to(cuda_device)
    y = sc_f.linear_generic(a, w, bit_length=128, generator="lfsr", forward="full_bin")
    assert np.array_equal((y * 128).round().to(torch.int32).cpu().numpy(), g["lin_y"])


def test_golden_reference_cuda_kernels(cuda_device):
    from geo_b200 import ops

    path = os.path.join(GOLDEN, "ref_cuda_modes.npz")
    if not os.path.exists(path):
        pytest.skip("reference-CUDA golden vectors not generated yet")
    g = np.load(path)
    for i in range(int(g["n"])):
        L, mode, z, tw, lu, lww, lwa = (int(v) for v in g[f"c{i}_meta"])
        y = ops.sc_conv2d(torch.from_numpy(g[f"c{i}_a"]).to(cuda_device), torch.from_numpy(g[f"c{i}_w"]).to(cuda_device),
                          L, MODE_NAMES[mode], (0, 0), z_unit=z, total_width=tw, load_width=lu, load_wait_w=lww,
                          load_wait_a=lwa)
        assert np.array_equal(y.cpu().numpy(), g[f"c{i}_y"]), f"case {i} meta {g[f'c{i}_meta']}"


def test_linear_groups_of_16(cuda_device, oracle_lib):
    from geo_b200 import ops

    g = torch.Generator().manual_seed(3)
    a = q7(torch.rand(33, 160, generator=g))
    w = q7(torch.rand(45, 160, generator=g) * 2 - 1)
    for L in (32, 64, 128, 256):
        y = ops.sc_linear(a.to(cuda_device), w.to(cuda_device), L, z_unit=16).cpu().numpy()
        assert np.array_equal(y, oracle_lib.linear(a, w, L, z_unit=16))


def test_full_size_training_layer_properties(cuda_device, oracle_lib):
    """Second conv of the 4-layer CNN at batch 256 (padded 20x20 input, 32->32, 5x5, L=128,
    load 2/2).  Activation generators restart for every image and weight generators are shared
    by all output channels, so any (image, channel) slice of the full run must equal the oracle
    run on that slice alone; the full run must also be invariant under batch permutation."""
    from geo_b200 import ops

    g = torch.Generator().manual_seed(42)
    a = q7(torch.rand(256, 32, 16, 16, generator=g))
    w = q7((torch.rand(32, 32, 5, 5, generator=g) * 2 - 1) * 0.3)
    kw = dict(total_width=7, load_width=2, load_wait_w=2, load_wait_a=2)
    y = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), 128, "1d_bin", (2, 2), **kw)
    assert y.shape == (256, 32, 16, 16)
    for b, o in [(0, slice(0, 4)), (131, slice(13, 15)), (255, slice(30, 32))]:
        ref = oracle_lib.conv2d(a[b:b + 1], w[o], 128, "1d_bin", pad_h=2, pad_w=2, **kw)
        assert np.array_equal(y[b:b + 1, o].cpu().numpy(), ref)
    perm = torch.randperm(256, generator=g)
    y2 = ops.sc_conv2d(a[perm].to(cuda_device), w.to(cuda_device), 128, "1d_bin", (2, 2), **kw)
    assert torch.equal(y2.cpu(), y.cpu()[perm])
    assert int(y.abs().max()) <= 128 * 5


def test_reference_module_names_and_signatures(cuda_device, oracle_lib):
    """The pybind11 shims keep the reference's module and function names (sc_cuda.cpp:78-83)."""
    ext_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "geo_b200", "ext")
    sys.path.insert(0, ext_dir)
    saved = {n: sys.modules.pop(n, None) for n in ("sc_extension", "sc_extension_cuda")}
    try:
        import sc_extension
        import sc_extension_cuda
    finally:
        sys.path.remove(ext_dir)
        for n, m in saved.items():
            if m is not None:
                sys.modules[n] = m
    assert os.path.dirname(sc_extension.__file__) == ext_dir and os.path.dirname(sc_extension_cuda.__file__) == ext_dir
    a, w = _rand((2, 4, 8, 8), (6, 4, 3, 3), 9)
    ad, wd = a.to(cuda_device), w.to(cuda_device)
    ap = torch.nn.functional.pad(ad, (1, 1, 1, 1))
    y = sc_extension_cuda.conv2d_add_partial_variable_acc(ap, wd, 128, (0, 0), (1, 1), 7, 2, 2, False, 2)
    assert y.dtype == torch.int32 and y.is_cuda
    assert np.array_equal(y.cpu().numpy(), oracle_lib.conv2d(a, w, 128, "1d_bin", load_width=2, load_wait_w=2,
                                                             pad_h=1, pad_w=1))
    y = sc_extension_cuda.conv2d_add_partial_variable_acc(ap, wd, 64, (0, 0), (1, 1), 7, 2, 2, False, 0)
    assert np.array_equal(y.cpu().numpy(), oracle_lib.conv2d(a, w, 64, "z_bin", load_width=2, load_wait_w=2,
                                                             pad_h=1, pad_w=1))
    y = sc_extension_cuda.conv2d_add_yz_variable_acc(ap, wd, 128, (0, 0), (1, 1), 7, 2, 2, 3, False, 2)
    assert np.array_equal(y.cpu().numpy(), oracle_lib.conv2d(a, w, 128, "yz_bin", z_unit=2, load_width=2,
                                                             load_wait_w=2, load_wait_a=3, pad_h=1, pad_w=1))
    y = sc_extension_cuda.conv2d_or_acc(ad, wd, 128, (1, 1), (1, 1), False)   # padding done by the extension
    assert np.array_equal(y.cpu().numpy(), oracle_lib.conv2d(a, w, 128, "full_or", pad_h=1, pad_w=1))
    y = sc_extension.conv2d_add_partial_new(ad, wd, 32, (2, 0), (1, 1))        # pads the last dim by 2
    assert np.array_equal(y.cpu().numpy(), oracle_lib.conv2d(a, w, 32, "1d_bin", pad_h=0, pad_w=2))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        sc_extension.conv2d_add_partial_new(a, w, 32, (0, 0), (1, 1))
    with pytest.raises(RuntimeError, match="bit_length"):
        sc_extension_cuda.conv2d_or_acc(ad, wd, 100, (0, 0), (1, 1), False)


def _popcount(x):
    """Ones in every element of an int32/uint32 numpy array."""
    return np.unpackbits(np.ascontiguousarray(x).view(np.uint8)).reshape(x.shape + (32,)).sum(-1)


@pytest.mark.parametrize("L", [8, 32, 128, 256])
def test_accurate_generator_streams_hold_exactly_their_level(cuda_device, L):
    """GEO_SC_GEN_ACC (sampling without replacement, utils_functional.py:157-176): the stream of level V has
    exactly V ones, whatever the seed; a seed reproduces its streams and another seed gives others."""
    from geo_b200 import ops

    a, w = _rand((2, 5, 6, 7), (9, 5, 3, 2), 50 + L)
    for mode in ("1d_bin", "z_bin", "full_or"):
        d = ops.desc_for(a, w, L, mode, (1, 2), generator="acc", seed=7)
        asg = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d), d).cpu().numpy()   # [B,C,H,W,P]
        wsg = ops.weight_streams_canonical(ops.prepare_weights(w.to(cuda_device), d), d).cpu().numpy()     # [2,O,C,K2,K3,P]
        ap = np.pad(a.numpy(), ((0, 0), (0, 0), (1, 1), (2, 2)))
        va = np.ceil(np.clip(ap * L, 0, L - 1)).astype(np.int64)
        assert np.array_equal(_popcount(asg).sum(-1), va)
        vp = np.ceil(np.clip(w.numpy() * L, 0, L - 1)).astype(np.int64)
        vn = np.ceil(-np.clip(w.numpy() * L, 1 - L, 0)).astype(np.int64)
        assert np.array_equal(_popcount(wsg[0]).sum(-1), vp) and np.array_equal(_popcount(wsg[1]).sum(-1), vn)
        y1 = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, (1, 2), generator="acc", seed=7)
        y2 = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, (1, 2), generator="acc", seed=7)
        y3 = ops.sc_conv2d(a.to(cuda_device), w.to(cuda_device), L, mode, (1, 2), generator="acc", seed=8)
        assert torch.equal(y1, y2) and not torch.equal(y1, y3)


@pytest.mark.parametrize("generator", ["acc", "rand"])
def test_counter_based_generators_do_not_depend_on_the_stream_image_layout(cuda_device, generator):
    """The streams of the counter-based generators are a function of (seed, element, bit): the batch-innermost
    image of a 64-channel layer holds the same words as the batch-major image that another mode gets for the
    same activations."""
    from geo_b200 import _lib, ops

    a, w = _rand((7, 64, 5, 4), (32, 64, 3, 3), 4242)
    kw = dict(generator=generator, seed=5)
    d_batch = ops.desc_for(a, w, 128, "1d_bin", (1, 1), **kw)
    d_major = ops.desc_for(a, w, 128, "z_bin", (1, 1), **kw)
    assert _lib.act_stream_layout(d_batch)[0] and not _lib.act_stream_layout(d_major)[0]
    s1 = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d_batch), d_batch)
    s2 = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d_major), d_major)
    assert torch.equal(s1, s2)
    if generator == "acc":
        ap = np.pad(a.numpy(), ((0, 0), (0, 0), (1, 1), (1, 1)))
        assert np.array_equal(_popcount(s1.cpu().numpy()).sum(-1), np.ceil(np.clip(ap * 128, 0, 127)).astype(np.int64))


def test_random_generator_bits_are_independent_draws_against_shared_thresholds(cuda_device):
    """GEO_SC_GEN_RAND (utils_functional.py:92-102): a bit is one when the level exceeds a uniform integer below
    L, so the ones of a stream average level (not exactly, unlike 'acc'); the integers are shared like the
    LFSR generators: weights of different output channels with the same level get the same stream."""
    from geo_b200 import ops

    L = 128
    a = torch.full((1, 2, 64, 64), 40 / 128)
    w = torch.zeros(6, 2, 3, 3)
    w[:, 0] = 0.5                    # the same positive level for every output channel
    w[:, 1] = -0.25
    d = ops.desc_for(a, w, L, "1d_bin", (0, 0), generator="rand", seed=3)
    asg = ops.act_streams_canonical(ops.generate_act_streams(a.to(cuda_device), d), d).cpu().numpy()
    ones = _popcount(asg).sum(-1).astype(np.float64)          # 8192 streams of level 40
    assert abs(ones.mean() - 40) < 0.5 and 3.5 < ones.std() < 7.0          # binomial(128, 40/128): sigma 5.2
    wsg = ops.weight_streams_canonical(ops.prepare_weights(w.to(cuda_device), d), d).cpu().numpy()
    assert (wsg[0, :, 0] == wsg[0, :1, 0]).all() and (wsg[1, :, 1] == wsg[1, :1, 1]).all()   # shared over c_out
    assert not (wsg[0, 0, 0, 0] == wsg[0, 0, 0, 1]).all()                                    # but not over ky
    assert (wsg[1, :, 0] == 0).all() and (wsg[0, :, 1] == 0).all()


@pytest.mark.parametrize("generator", ["acc", "rand"])
def test_accurate_generator_statistics_match_reference_simulation(cuda_device, generator):
    """Against the reference's random generators only distributions can agree: mean of the outputs over
    200 seeds against the mean over 200 runs of the reference's bit-serial simulation (fixture), element by
    element within 5 standard errors and overall within 0.25 (acc) / 0.4 (rand) counts, about 6 standard
    errors of the grand mean; the spread of the outputs within 30 %."""
    from geo_b200 import functional as sc_f

    g = np.load(os.path.join(GOLDEN, f"ref_legacy_{generator}_stats.npz"))
    a, w = torch.from_numpy(g["a"]).to(cuda_device), torch.from_numpy(g["w"]).to(cuda_device)
    n = 200
    runs = torch.stack([sc_f.conv2d_generic(a.clone(), w, (1, 1), (1, 1), bit_length=128, forward="1d_bin",
                                            generator=generator, seed=1000 + i) * 128 for i in range(n)])
    mean = runs.mean(0).cpu().numpy()
    se = np.sqrt(g["std"] ** 2 / int(g["runs"]) + runs.std(0).cpu().numpy() ** 2 / n) + 1e-6
    assert np.all(np.abs(mean - g["mean"]) <= 5 * se + 0.5)
    assert abs(mean.mean() - g["mean"].mean()) <= (0.25 if generator == "acc" else 0.4)
    assert 0.7 <= runs.std(0).mean().item() / g["std"].mean() <= 1.3
