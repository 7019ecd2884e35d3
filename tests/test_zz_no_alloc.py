"""The workspace-free entry point (geo_sc_conv2d_forward_static).

It exists for callers that cannot allocate device memory when they call the library (a frozen
memory plan, an allocator-free steady state, a pointer-only plugin boundary): the stream scratch
is a fixed 64 MiB array inside the library.  Checked here through the C ABI against the ordinary
entry point, bit for bit, on two calls in a row whose scratch footprints differ, so that the
second call runs over the first call's leftovers.  Collected last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


def _static_forward(a, w, desc, out=None):
    from geo_b200 import _lib, ops

    if out is None:
        out = torch.full(ops.out_shape(desc), -12345, dtype=torch.int32, device=a.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check(_lib.lib().geo_sc_conv2d_forward_static(ctypes.byref(desc), a.data_ptr(), w.data_ptr(), out.data_ptr(),
                                                       stream), "geo_sc_conv2d_forward_static")
    return out


def test_static_scratch_entry_point_matches_workspace_entry_point(cuda_device):
    from geo_b200 import _lib, ops

    assert _lib.lib().geo_sc_static_scratch_bytes() == 64 << 20
    g = torch.Generator().manual_seed(2024)
    calls = [
        # first a larger problem (multi-CTA split path, 128-bit streams, progressive loading) ...
        ((24, 16, 14, 14), (40, 16, 3, 3), (1, 1), 128, "1d_bin", dict(total_width=7, load_width=2, load_wait_w=2)),
        # ... then a smaller one with another mode and stream length, over the leftovers
        ((3, 6, 9, 7), (5, 6, 3, 2), (0, 1), 64, "yz_bin", dict(z_unit=2)),
        # long groups (160 members): the ordinary entry point takes its sign-sorted kernel here, this one stays
        # on the dense kernel; 8 x 12 x 12 positions leave a ragged last position tile
        ((8, 32, 12, 12), (64, 32, 5, 5), (2, 2), 128, "1d_bin", dict(total_width=7, load_width=2, load_wait_w=2)),
        # the counter-based "accurate" generator with a fixed seed
        ((4, 8, 10, 10), (12, 8, 3, 3), (1, 1), 64, "1d_bin", dict(generator="acc", seed=11)),
        # 64 input channels: the stream image is batch-innermost (batch padded 6 -> 8); this entry point's dense
        # kernel reads it through the same offsets
        ((6, 64, 6, 6), (16, 64, 3, 3), (1, 1), 64, "1d_bin", dict(total_width=7, load_width=2, load_wait_w=2)),
        # a linear layer (batch-innermost image as well)
        ((9, 48, 1, 1), (20, 48, 1, 1), (0, 0), 128, "yz_bin", dict(z_unit=16)),
    ]
    for ashape, wshape, pad, L, mode, kw in calls:
        a = q7(torch.rand(*ashape, generator=g)).to(cuda_device)
        w = q7(torch.rand(*wshape, generator=g) * 2 - 1).to(cuda_device)
        desc = ops.desc_for(a, w, L, mode, pad, **kw)
        expect = ops.sc_conv2d(a, w, L, mode, pad, **kw)
        got = _static_forward(a, w, desc)
        torch.cuda.synchronize()
        assert torch.equal(got, expect), f"{mode} L={L}: static-scratch result differs"


def test_static_scratch_call_leaves_device_memory_untouched(cuda_device):
    """A warm call neither takes nor returns device memory: the free-memory figure of the driver is the same
    before and after (inputs and output are allocated beforehand)."""
    from geo_b200 import ops

    g = torch.Generator().manual_seed(7)
    a = q7(torch.rand(16, 8, 12, 12, generator=g)).to(cuda_device)
    w = q7(torch.rand(16, 8, 3, 3, generator=g) * 2 - 1).to(cuda_device)
    desc = ops.desc_for(a, w, 128, "1d_bin", (1, 1))
    out = torch.empty(ops.out_shape(desc), dtype=torch.int32, device=cuda_device)
    _static_forward(a, w, desc, out)          # first call on the device: address look-up, table upload
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    for _ in range(3):
        _static_forward(a, w, desc, out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert free_after == free_before
    assert torch.equal(out, ops.sc_conv2d(a, w, 128, "1d_bin", (1, 1)))


def test_static_scratch_rejects_oversized_problems(cuda_device):
    from geo_b200 import _lib

    # 512 x 64 x 66 x 66 padded pixels x 8 packs = 4.6 GB of activation streams
    desc = _lib.make_desc(512, 64, 64, 64, 64, 3, 3, 256, "1d_bin", pad_h=1, pad_w=1)
    dummy = torch.zeros(16, device=cuda_device)
    out = torch.zeros(16, dtype=torch.int32, device=cuda_device)
    rc = _lib.lib().geo_sc_conv2d_forward_static(ctypes.byref(desc), dummy.data_ptr(), dummy.data_ptr(), out.data_ptr(),
                                                 None)
    assert rc == -7
    assert b"built-in scratch holds" in _lib.lib().geo_sc_last_error()
