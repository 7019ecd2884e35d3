"""fp32 parity of the native guide kernels (forward exp(-y), weight and activation gradients) with
the PyTorch restatement of the reference's guide functions, run on the CPU in fp32.
Tolerance: 1e-5 relative to the largest magnitude of each gradient tensor."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


CASES = [
    # act, weight, (pad_h, pad_w), z_unit
    ((2, 3, 7, 6), (3, 3, 3, 2), (0, 0), 2),
    ((3, 5, 9, 8), (7, 5, 2, 4), (1, 0), 2),
    ((2, 8, 12, 12), (33, 8, 3, 3), (1, 1), 4),
    ((5, 4, 11, 13), (17, 4, 5, 5), (2, 2), 3),
    ((4, 32, 8, 8), (20, 32, 5, 5), (2, 2), 8),
    ((3, 16, 4, 4), (10, 16, 4, 4), (0, 0), 16),
    ((2, 40, 6, 6), (70, 40, 3, 3), (1, 1), 16),
    ((9, 24, 1, 1), (12, 24, 1, 1), (0, 0), 8),
    ((3, 128, 6, 6), (16, 128, 3, 3), (1, 1), 16),   # 128 input channels: widest activation-gradient tile
]


def _close(a, b, what):
    scale = b.abs().max().item() + 1e-30
    err = (a - b).abs().max().item()
    assert err <= RTOL * scale, f"{what}: max err {err:.3e} vs scale {scale:.3e} (rel {err / scale:.2e})"


@pytest.mark.parametrize("mode", ["1d_bin", "z_bin", "yz_bin", "full_or", "2d_bin", "full_bin"])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_guide_gradients_match_reference_guide(cuda_device, mode, case):
    from geo_b200 import ops
    from oracle import guide as oracle_guide

    ashape, wshape, pad, z = CASES[case]
    g = torch.Generator().manual_seed(17 * case + len(mode))
    a = q7(torch.rand(*ashape, generator=g))
    w = q7((torch.rand(*wshape, generator=g) * 2 - 1) * 0.5)
    w.view(-1)[::7] = 0.0          # exact zeros: clamp passes the gradient on both branches there
    desc = ops.desc_for(a, w, 128, mode, pad, z_unit=z)
    go = torch.randn(*ops.out_shape(desc), generator=g)
    ga_ref, gw_ref = oracle_guide.guide_grads(a, w, go, mode, pad[0], pad[1], z_unit=z)

    ad, wd = a.to(cuda_device), w.to(cuda_device)
    ga, gw = ops.guide_backward(ad, wd, go.to(cuda_device), desc)
    _close(gw.cpu(), gw_ref, f"{mode} grad_weight")
    _close(ga.cpu(), ga_ref, f"{mode} grad_act")


def test_guide_gradients_match_recorded_reference_functions(cuda_device):
    """The CUDA guide against gradients recorded from the reference's own guide functions
    (utils_functional.py:189-296, fixture tests/golden/ref_guide_grads.npz), every mode, through both entry
    points: the general one and the one for quantised inputs (tensor-core kernels alone)."""
    from test_oracle_golden import guide_fixture_cases

    from geo_b200 import ops

    n = 0
    for mode, pad_h, pad_w, z, a, w, go, ga_ref, gw_ref in guide_fixture_cases():
        desc = ops.desc_for(a, w, 128, mode, (pad_h, pad_w), z_unit=z)
        for quantized in (False, True):
            ga, gw = ops.guide_backward(a.to(cuda_device), w.to(cuda_device), go.to(cuda_device), desc,
                                        quantized=quantized)
            _close(gw.cpu(), gw_ref, f"{mode} grad_weight case {n} quantized={quantized}")
            _close(ga.cpu(), ga_ref, f"{mode} grad_act case {n} quantized={quantized}")
        n += 1
    assert n == 18


@pytest.mark.parametrize("mode", ["1d_bin", "full_or", "2d_bin", "full_bin"])
def test_guide_gradients_for_inputs_that_bf16_cannot_hold(cuda_device, mode):
    """Unquantised inputs: the tensor-core path must stand down (its exactness argument does not
    apply) and the fp32 FFMA kernels must produce the gradients."""
    from geo_b200 import ops
    from oracle import guide as oracle_guide

    g = torch.Generator().manual_seed(99)
    a = torch.rand(3, 16, 9, 9, generator=g)
    w = (torch.rand(40, 16, 3, 3, generator=g) * 2 - 1) * 0.3
    desc = ops.desc_for(a, w, 128, mode, (1, 1))
    go = torch.randn(*ops.out_shape(desc), generator=g)
    ga_ref, gw_ref = oracle_guide.guide_grads(a, w, go, mode, 1, 1)
    ga, gw = ops.guide_backward(a.to(cuda_device), w.to(cuda_device), go.to(cuda_device), desc)
    _close(gw.cpu(), gw_ref, f"{mode} grad_weight (fp32 inputs)")
    _close(ga.cpu(), ga_ref, f"{mode} grad_act (fp32 inputs)")
    # one inexact value among exact ones is enough to switch paths
    a2 = q7(a)
    a2[1, 3, 4, 4] = 0.123456
    w2 = q7(w)
    ga_ref, gw_ref = oracle_guide.guide_grads(a2, w2, go, mode, 1, 1)
    ga, gw = ops.guide_backward(a2.to(cuda_device), w2.to(cuda_device), go.to(cuda_device), desc)
    _close(gw.cpu(), gw_ref, f"{mode} grad_weight (one inexact value)")
    _close(ga.cpu(), ga_ref, f"{mode} grad_act (one inexact value)")


@pytest.mark.parametrize("mode", ["1d_bin", "z_bin", "yz_bin", "full_or", "2d_bin"])
def test_guide_backward_with_quantised_inputs_promise(cuda_device, mode):
    """geo_sc_guide_backward_quantized: same gradients as the general entry point (bit for bit) for
    inputs that keep the promise; NaN gradients, not silently wrong ones, for inputs that break it
    in the modes the tensor-core kernels serve."""
    from geo_b200 import ops

    g = torch.Generator().manual_seed(31)
    a = q7(torch.rand(4, 12, 10, 10, generator=g)).to(cuda_device)
    w = q7((torch.rand(24, 12, 3, 3, generator=g) * 2 - 1) * 0.4).to(cuda_device)
    desc = ops.desc_for(a, w, 128, mode, (1, 1), z_unit=4)
    go = torch.randn(*ops.out_shape(desc), generator=g).to(cuda_device)
    ga0, gw0 = ops.guide_backward(a, w, go, desc)
    ga1, gw1 = ops.guide_backward(a, w, go, desc, quantized=True)
    assert torch.equal(ga0, ga1) and torch.equal(gw0, gw1)
    _, gw2 = ops.guide_backward(a, w, go, desc, need_act=False, quantized=True)
    _close(gw2.cpu(), gw0.cpu(), f"{mode} grad_weight alone")   # may take the one-kernel route: other summation order
    bad = a.clone()
    bad[0, 0, 0, 0] = 0.123456
    ga3, gw3 = ops.guide_backward(bad, w, go, desc, quantized=True)
    if mode in ("1d_bin", "full_or", "2d_bin"):
        assert torch.isnan(ga3).all() and torch.isnan(gw3).all()
    else:
        ga4, gw4 = ops.guide_backward(bad, w, go, desc)
        assert torch.equal(ga3, ga4) and torch.equal(gw3, gw4)


FIRST_LAYER_CASES = [
    # act, weight, (pad_h, pad_w), mode -- groups of at most 64 padded members, weight gradient only
    ((5, 3, 12, 12), (32, 3, 5, 5), (2, 2), "1d_bin"),      # 5 taps x 8 channels -> 64 members
    ((3, 3, 9, 7), (20, 3, 3, 3), (1, 1), "1d_bin"),        # 32 members, odd image size (scalar gout loads)
    ((2, 12, 10, 10), (40, 12, 3, 3), (1, 1), "1d_bin"),    # two column tiles, 48 -> 64 members
    ((7, 8, 6, 6), (9, 8, 2, 2), (0, 0), "full_or"),        # one group of 4 taps x 8 channels
    ((40, 3, 16, 16), (32, 3, 5, 5), (2, 2), "1d_bin"),     # more position tiles than resident CTAs per group
    ((1, 5, 3, 3), (3, 5, 3, 3), (1, 1), "1d_bin"),         # a single, partly filled position tile
    ((4, 8, 8, 8), (16, 8, 3, 3), (1, 1), "2d_bin"),        # nine groups of one tap x 8 channels
    ((2, 40, 6, 6), (12, 40, 2, 3), (0, 1), "2d_bin"),      # 40 channels -> 64 members
    ((3, 4, 7, 8), (9, 4, 2, 2), (0, 0), "full_bin"),       # linear guide (no exp), 4 taps x 8 channels
]


@pytest.mark.parametrize("case", range(len(FIRST_LAYER_CASES)))
def test_weight_gradient_alone_short_groups(cuda_device, case):
    """Only grad_weight wanted and short groups (a network's first layer): forward and weight
    gradient run as one kernel; same tolerance against the reference guide."""
    from geo_b200 import ops
    from oracle import guide as oracle_guide

    ashape, wshape, pad, mode = FIRST_LAYER_CASES[case]
    g = torch.Generator().manual_seed(400 + case)
    a = q7(torch.rand(*ashape, generator=g))
    w = q7((torch.rand(*wshape, generator=g) * 2 - 1) * 0.5)
    w.view(-1)[::5] = 0.0
    desc = ops.desc_for(a, w, 128, mode, pad)
    go = torch.randn(*ops.out_shape(desc), generator=g)
    _, gw_ref = oracle_guide.guide_grads(a, w, go, mode, pad[0], pad[1])
    for quantized in (False, True):
        ga, gw = ops.guide_backward(a.to(cuda_device), w.to(cuda_device), go.to(cuda_device), desc, need_act=False,
                                    quantized=quantized)
        assert ga is None
        _close(gw.cpu(), gw_ref, f"case {case} grad_weight (quantized={quantized})")
    # run-to-run determinism
    _, gw2 = ops.guide_backward(a.to(cuda_device), w.to(cuda_device), go.to(cuda_device), desc, need_act=False,
                                quantized=True)
    assert torch.equal(gw, gw2)


def test_layer_autograd_matches_reference_semantics(cuda_device, oracle_lib):
    """conv2d_generic: value = SC counts / L (bit-exact), gradient = guide gradient."""
    from geo_b200 import functional as sc_f
    from oracle import guide as oracle_guide

    g = torch.Generator().manual_seed(5)
    a = q7(torch.rand(4, 6, 10, 10, generator=g))
    w = q7((torch.rand(12, 6, 5, 5, generator=g) * 2 - 1) * 0.4)
    for mode, kw in (("1d_bin", {}), ("yz_bin", {"z_unit": 2}), ("z_bin", {}), ("full_or", {}), ("2d_bin", {}),
                     ("full_bin", {})):
        ad = a.to(cuda_device).requires_grad_(True)
        wd = w.to(cuda_device).requires_grad_(True)
        out = sc_f.conv2d_generic(ad, wd, (2, 2), (1, 1), bit_length=128, forward=mode, generator="lfsr", load_unit=2,
                                  load_wait_w=2, load_wait_a=2, **kw)
        lu = 8 if mode in ("full_or", "2d_bin", "full_bin") else 2
        lw = 1 if mode in ("full_or", "2d_bin", "full_bin") else 2
        ref = oracle_lib.conv2d(a, w, 128, mode, pad_h=2, pad_w=2, load_width=lu, load_wait_w=lw, load_wait_a=lw,
                                z_unit=kw.get("z_unit", 1024))
        assert torch.equal(out.detach().cpu(), torch.from_numpy(ref).float() / 128)
        go = torch.randn(out.shape, generator=g)
        out.backward(go.to(cuda_device))
        ga_ref, gw_ref = oracle_guide.guide_grads(a, w, go, mode, 2, 2, z_unit=kw.get("z_unit", 1024))
        _close(wd.grad.cpu(), gw_ref, f"{mode} layer grad_weight")
        _close(ad.grad.cpu(), ga_ref, f"{mode} layer grad_act")


def test_training_layer_shapes_full_batch(cuda_device):
    """Second conv of the 4-layer CNN at batch 256: gradients against the same guide evaluated by
    PyTorch on the GPU with TF32 convolutions disabled."""
    from geo_b200 import ops
    from oracle import guide as oracle_guide

    g = torch.Generator().manual_seed(8)
    a = q7(torch.rand(256, 32, 16, 16, generator=g)).to(cuda_device)
    w = q7((torch.rand(32, 32, 5, 5, generator=g) * 2 - 1) * 0.1).to(cuda_device)
    go = torch.randn(256, 32, 16, 16, generator=g).to(cuda_device)
    desc = ops.desc_for(a, w, 128, "1d_bin", (2, 2))
    ga, gw = ops.guide_backward(a, w, go, desc)
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        ga_ref, gw_ref = oracle_guide.guide_grads(a, w, go, "1d_bin", 2, 2)
    finally:
        torch.backends.cudnn.allow_tf32 = old
    # 65536 positions are summed per weight: allow the summation-order error of fp32 itself
    scale = gw_ref.abs().max().item()
    assert (gw - gw_ref).abs().max().item() <= 5e-5 * scale
    assert (ga - ga_ref).abs().max().item() <= 1e-5 * ga_ref.abs().max().item()


WIDE_CASES = [
    # layers wide enough for the tcgen05 activation-gradient kernel (>= 128 input channels, image width a power of
    # two): act, weight, (pad_h, pad_w)
    ((4, 128, 8, 8), (32, 128, 3, 3), (1, 1)),        # two whole 8x8 images per 128-pixel tile
    ((3, 128, 8, 8), (40, 128, 3, 3), (1, 1)),        # odd batch: the last tile is half outside the batch
    ((2, 256, 16, 16), (64, 256, 3, 3), (1, 1)),      # half an image per tile, two channel tiles
    ((2, 128, 16, 16), (32, 128, 5, 5), (2, 2)),      # 5x5 taps
    ((9, 160, 4, 4), (48, 160, 3, 3), (1, 1)),        # eight 4x4 images per tile, channels padded to 256
    ((1, 128, 32, 32), (32, 128, 3, 3), (1, 1)),      # four rows of a 32-wide image per tile
    ((2, 128, 16, 16), (64, 128, 5, 5), (2, 2)),      # 128 columns: the forward product runs on tcgen05 too
    ((9, 192, 4, 4), (128, 192, 3, 3), (1, 1)),       # 4x4 images, 256 columns, three 64-channel blocks per tap
    ((5, 64, 2, 2), (64, 64, 3, 3), (1, 1)),          # 2x2 images, 32 per tile; forward on tcgen05, gradient not
    ((4, 256, 8, 8), (128, 256, 3, 3), (1, 1)),       # all three GEMMs on tcgen05; weight gradient: one image per stage
    ((16, 128, 2, 2), (64, 128, 3, 3), (1, 1)),       # weight gradient: sixteen 2x2 images per stage
]


@pytest.mark.parametrize("mode", ["1d_bin", "full_or", "2d_bin"])
@pytest.mark.parametrize("case", range(len(WIDE_CASES)))
def test_guide_gradients_of_wide_layers(cuda_device, mode, case):
    """Same check as above on shapes that take the tcgen05 / tensor-memory / TMA kernel for the activation
    gradient; none of its bounded barrier waits may have run out."""
    from geo_b200 import _lib, ops
    from oracle import guide as oracle_guide

    ashape, wshape, pad = WIDE_CASES[case]
    g = torch.Generator().manual_seed(900 + 13 * case + len(mode))
    a = q7(torch.rand(*ashape, generator=g))
    w = q7((torch.rand(*wshape, generator=g) * 2 - 1) * 0.25)
    w.view(-1)[::5] = 0.0
    desc = ops.desc_for(a, w, 128, mode, pad)
    go = torch.randn(*ops.out_shape(desc), generator=g)
    ga_ref, gw_ref = oracle_guide.guide_grads(a, w, go, mode, pad[0], pad[1])
    ga, gw = ops.guide_backward(a.to(cuda_device), w.to(cuda_device), go.to(cuda_device), desc, quantized=True)
    torch.cuda.synchronize()
    assert _lib.device_error_count() == 0
    _close(gw.cpu(), gw_ref, f"{mode} grad_weight")
    _close(ga.cpu(), ga_ref, f"{mode} grad_act")
