"""CPU-only checks of the native library's host side: it loads, exports every symbol the
header declares, validates descriptors, and its table-driven stream generator reproduces the
bit-serial oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from geo_b200 import _lib

    L = _lib.lib()
    header = open(os.path.join(ROOT, "include", "geo_sc.h")).read()
    names = set(re.findall(r"\b(geo_sc_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 15
    for n in sorted(names):
        assert hasattr(L, n), f"{n} declared in geo_sc.h but not exported"
    assert L.geo_sc_version() == 1


def test_descriptor_validation_codes():
    from geo_b200 import _lib

    def rc(**kw):
        base = dict(batch=1, c_in=3, h_in=8, w_in=8, c_out=4, k_h=3, k_w=3, bit_length=128)
        base.update(kw)
        d = _lib.make_desc(**base)
        out = ctypes.c_size_t(0)
        return _lib.lib().geo_sc_conv2d_workspace_bytes(ctypes.byref(d), ctypes.byref(out)), out.value

    assert rc()[0] == 0 and rc()[1] > 0
    assert rc(bit_length=100)[0] == -2       # the reference leaves its LFSR pointer uninitialised here
    assert rc(bit_length=512)[0] == -2
    assert rc(c_in=0)[0] == -3
    assert rc(k_h=9)[0] == -3                # filter larger than the image
    assert rc(k_h=9, pad_h=1)[0] == 0
    assert rc(mode=7)[0] == -4
    assert rc(load_width=0)[0] == -5
    assert rc(load_wait_w=0)[0] == -5
    assert rc(batch=1 << 20, h_in=512, w_in=512)[0] == -6
    assert rc(mode="yz_bin", z_unit=0)[0] == -3
    assert b"bit_length" in _lib.lib().geo_sc_last_error() or True
    with pytest.raises(_lib.GeoScError):
        _lib.size_query("geo_sc_conv2d_workspace_bytes", _lib.make_desc(1, 1, 1, 1, 1, 1, 1, 7))


def test_group_geometry_per_mode():
    from geo_b200 import _lib

    d = lambda mode, **kw: _lib.make_desc(2, 12, 9, 9, 40, 3, 5, 64, mode, **kw)  # noqa: E731
    assert _lib.group_geometry(d("1d_bin")) == (5, 36, 64, 64)
    assert _lib.group_geometry(d("z_bin")) == (12, 15, 64, 64)
    assert _lib.group_geometry(d("yz_bin", z_unit=4)) == (15, 12, 64, 64)
    assert _lib.group_geometry(d("yz_bin", z_unit=5)) == (15, 15, 64, 64)     # ragged last channel group
    assert _lib.group_geometry(d("yz_bin", z_unit=100)) == (5, 36, 64, 64)    # z clamps to c_in
    assert _lib.group_geometry(d("full_or")) == (1, 180, 64, 64)
    assert _lib.group_geometry(d("2d_bin")) == (15, 12, 64, 64)              # groups = filter taps, members = channels
    assert _lib.group_geometry(d("full_bin")) == (180, 1, 64, 64)            # every filter element its own group
    # which accumulate kernel a descriptor gets: long groups (>= 64 padded members) the sign-sorted one, short
    # groups the per-chunk sorted one (both one logic op per weight), tiny launches and full_bin neither
    big = lambda mode: _lib.make_desc(8, 32, 16, 16, 32, 5, 5, 128, mode, pad_h=2, pad_w=2)  # noqa: E731
    assert _lib.is_sign_sorted(big("1d_bin")) and _lib.is_sign_sorted(big("full_or"))
    assert _lib.is_sign_sorted(big("z_bin")) and _lib.is_sign_sorted(big("2d_bin"))
    assert not _lib.is_sign_sorted(big("full_bin"))
    assert not _lib.is_sign_sorted(d("1d_bin"))                               # 70 positions: dense kernel
    assert [_lib.accumulate_kernel(big(m)) for m in ("1d_bin", "z_bin", "2d_bin", "full_bin")] == \
        ["sorted_rows", "sorted_short", "sorted_short", "full_bin"]
    assert _lib.accumulate_kernel(d("1d_bin")) == "dense"
    wide = lambda mode, b=64: _lib.make_desc(b, 128, 8, 8, 128, 3, 3, 128, mode, pad_h=1, pad_w=1)  # noqa: E731
    assert [_lib.accumulate_kernel(wide(m)) for m in ("1d_bin", "full_or", "2d_bin", "z_bin")] == \
        ["sorted_taps", "sorted_taps", "sorted_taps", "sorted_short"]          # >= 64 channels: tap tiles
    assert _lib.act_stream_layout(wide("1d_bin", 30)) == (True, 32) and _lib.act_stream_layout(wide("z_bin"))[0] is False
    tiny = _lib.make_desc(3, 128, 4, 4, 128, 3, 3, 128, "1d_bin", pad_h=1, pad_w=1)
    assert _lib.accumulate_kernel(tiny) == "dense"                             # fewer than the 64 runs of four images of a tile
    lin = lambda b: _lib.make_desc(b, 64, 1, 1, 32, 1, 1, 128, "yz_bin", z_unit=16)  # noqa: E731
    assert _lib.accumulate_kernel(lin(256)) == "sorted_short"                 # batch-innermost image, 16-byte copies
    assert _lib.accumulate_kernel(lin(255)) == "sorted_short"                 # the image pads the batch to 256
    assert _lib.act_stream_layout(lin(255)) == (True, 256) and _lib.act_stream_layout(big("1d_bin"))[0] is False
    assert _lib.group_geometry(_lib.make_desc(1, 3, 8, 8, 10, 3, 3, 32))[2:] == (16, 16)
    assert _lib.group_geometry(_lib.make_desc(1, 3, 8, 8, 32, 3, 3, 32))[2:] == (32, 32)


@pytest.mark.parametrize("L", [8, 16, 32, 64, 128, 256])
def test_table_driven_streams_match_bit_serial_oracle(oracle_lib, L):
    from geo_b200 import _lib

    plans = [(7, 8, 1), (7, 2, 2), (7, 1, 3), (7, 3, 5), (7, 1, 9), (7, 2, 40), (5, 2, 2), (0, 1, 1), (15, 4, 3)]
    for tw, lu, lw in plans:
        Wd = 2 * L + 9
        rng = np.random.default_rng(L + lu)
        vals = rng.integers(0, L, size=Wd)
        a = (vals / L).astype(np.float32).reshape(1, 1, 1, Wd)
        ora = oracle_lib.act_streams(a, L, "1d_bin", total_width=tw, load_width=lu, load_wait_a=lw)[0, 0, 0]
        w = (vals / L).astype(np.float32).reshape(1, Wd, 1, 1)
        w[0, ::2] *= -1
        ow = oracle_lib.weight_streams(w, L, "1d_bin", total_width=tw, load_width=lu, load_wait_w=lw)
        for x in range(Wd):
            v = int(vals[x])
            assert _lib.host_stream(L, v, 0, x, tw, lu, lw) == list(ora[x])
            neg = x % 2 == 0
            assert _lib.host_stream(L, 0 if neg else v, 67, x, tw, lu, lw) == list(ow[0, 0, x, 0, 0])
            assert _lib.host_stream(L, v if neg else 0, 37, x, tw, lu, lw) == list(ow[1, 0, x, 0, 0])


def test_ops_refuse_cpu_tensors():
    import torch

    from geo_b200 import ops

    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.sc_conv2d(torch.zeros(1, 1, 4, 4), torch.zeros(1, 1, 3, 3), 32)
