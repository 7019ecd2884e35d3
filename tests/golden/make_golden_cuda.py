"""Generate golden vectors from the reference's own CUDA kernels (needs a GPU).

The reference extension (torch_c/sc-extension/sc_cuda.cpp + sc_cuda_kernel.cu) is built
unmodified for sm_100a by ``oracle/build_ref.py`` into ``oracle/_ref/cuda``.  This script
runs its three deterministic entry points

    conv2d_add_partial_variable_acc(..., dim=2)   1d_bin   (sc_cuda.cpp:47-63)
    conv2d_add_partial_variable_acc(..., dim=0)   z_bin
    conv2d_add_yz_variable_acc(...)               yz_bin   (sc_cuda.cpp:34-45)

with and without progressive loading on small inputs and stores inputs and outputs in
``<out_dir>/ref_cuda_modes.npz`` (default: next to this script).  Shapes avoid the two
configurations in which the reference reads or strides outside what it wrote: z_bin needs
k_w <= c_in (seed array of c_in*k_h entries indexed by ky*k_w+kx, sc_cuda_kernel.cu:322-324)
and yz_bin needs c_in divisible by z_unit (pack stride, sc_cuda_kernel.cu:251).

    python tests/golden/make_golden_cuda.py [out_dir]
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref_loader  # noqa: E402

MODE_1D, MODE_Z, MODE_YZ = 0, 1, 2


def q7(x):
    return (x * 128).round().clamp(-127, 127) / 128


def run_ref(ext, a, w, L, mode, z, tw, lu, lww, lwa):
    if mode == MODE_YZ:
        y = ext.conv2d_add_yz_variable_acc(a, w, L, (0, 0), (1, 1), tw, lu, lww, lwa, False, z)
    else:
        y = ext.conv2d_add_partial_variable_acc(a, w, L, (0, 0), (1, 1), tw, lu, lww, False, 0 if mode == MODE_Z else 2)
    torch.cuda.synchronize()
    return y


def cases():
    plans = [(7, 2, 2, 2), (7, 8, 1, 1), (7, 1, 3, 3), (7, 3, 5, 2)]
    out = []
    for L in (8, 16, 32, 64, 128, 256):
        for pi, (tw, lu, lww, lwa) in enumerate(plans):
            if L < 32 and pi > 1:
                continue
            for mode in (MODE_1D, MODE_Z, MODE_YZ):
                if mode != MODE_YZ:
                    lwa = lww
                out.append(dict(L=L, mode=mode, z=2, tw=tw, lu=lu, lww=lww, lwa=lwa, a=(2, 4, 7, 6), w=(5, 4, 3, 2)))
    # tile edges of a register-tiled kernel: 33 output channels, 100 positions per image
    for mode in (MODE_1D, MODE_Z, MODE_YZ):
        out.append(dict(L=128, mode=mode, z=4, tw=7, lu=2, lww=2, lwa=2, a=(3, 8, 12, 12), w=(33, 8, 3, 3)))
        out.append(dict(L=64, mode=mode, z=8, tw=7, lu=2, lww=2, lwa=2, a=(2, 16, 6, 6), w=(10, 16, 4, 4)))
    return out


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out_dir, exist_ok=True)
    ext = ref_loader.ref_sc_extension_cuda()
    assert ext is not None, "oracle/_ref/cuda/ref_sc_extension_cuda.so missing (run oracle/build_ref.py)"
    dev = torch.device("cuda:0")
    torch.manual_seed(777)
    res = {}
    cs = cases()
    for i, c in enumerate(cs):
        a = q7(torch.rand(*c["a"]))
        w = q7(torch.rand(*c["w"]) * 2 - 1)
        y = run_ref(ext, a.to(dev), w.to(dev), c["L"], c["mode"], c["z"], c["tw"], c["lu"], c["lww"], c["lwa"])
        y2 = run_ref(ext, a.to(dev), w.to(dev), c["L"], c["mode"], c["z"], c["tw"], c["lu"], c["lww"], c["lwa"])
        assert torch.equal(y, y2), f"reference kernel not deterministic on case {i}"
        assert y.abs().sum().item() > 0, f"reference kernel returned all zeros on case {i}"
        res[f"c{i}_a"] = a.numpy()
        res[f"c{i}_w"] = w.numpy()
        res[f"c{i}_meta"] = np.array([c["L"], c["mode"], c["z"], c["tw"], c["lu"], c["lww"], c["lwa"]], np.int32)
        res[f"c{i}_y"] = y.cpu().numpy().astype(np.int32)
    res["n"] = np.array(len(cs))
    path = os.path.join(out_dir, "ref_cuda_modes.npz")
    np.savez_compressed(path, **res)
    print("wrote", path, "cases", len(cs))


if __name__ == "__main__":
    main()
