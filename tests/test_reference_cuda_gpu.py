"""Live comparison with the reference's own CUDA kernels (built unmodified for sm_100a into
oracle/_ref/cuda).  Skipped where that build is absent."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


@pytest.fixture(scope="module")
def ref_cuda(cuda_device):
    from oracle import ref_loader

    m = ref_loader.ref_sc_extension_cuda()
    if m is None:
        pytest.skip("reference CUDA extension not built")
    return m


# Shapes keep k_w <= c_in (z_bin seed table) and c_in % z_unit == 0 (yz_bin pack stride): outside
# those the reference reads memory it did not write.
@pytest.mark.parametrize("L,lu,lw", [(128, 2, 2), (64, 8, 1), (256, 1, 3), (32, 2, 2)])
def test_three_modes_against_reference_kernels(cuda_device, ref_cuda, L, lu, lw):
    from geo_b200 import ops

    g = torch.Generator().manual_seed(L + lu)
    a = q7(torch.rand(5, 8, 14, 14, generator=g)).to(cuda_device)
    w = q7(torch.rand(24, 8, 5, 5, generator=g) * 2 - 1).to(cuda_device)
    ref = ref_cuda.conv2d_add_partial_variable_acc(a, w, L, (0, 0), (1, 1), 7, lu, lw, False, 2)
    torch.cuda.synchronize()
    mine = ops.sc_conv2d(a, w, L, "1d_bin", total_width=7, load_width=lu, load_wait_w=lw)
    assert ref.abs().sum() > 0 and torch.equal(ref, mine)
    ref = ref_cuda.conv2d_add_partial_variable_acc(a, w, L, (0, 0), (1, 1), 7, lu, lw, False, 0)
    torch.cuda.synchronize()
    mine = ops.sc_conv2d(a, w, L, "z_bin", total_width=7, load_width=lu, load_wait_w=lw)
    assert ref.abs().sum() > 0 and torch.equal(ref, mine)
    ref = ref_cuda.conv2d_add_yz_variable_acc(a, w, L, (0, 0), (1, 1), 7, lu, lw, lw + 1, False, 4)
    torch.cuda.synchronize()
    mine = ops.sc_conv2d(a, w, L, "yz_bin", z_unit=4, total_width=7, load_width=lu, load_wait_w=lw,
                         load_wait_a=lw + 1)
    assert ref.abs().sum() > 0 and torch.equal(ref, mine)
