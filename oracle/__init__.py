"""CPU oracle for the SC hot path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs
of ``bench.py`` import this package, and only as the checker (or as the timed CPU
baseline).  The product (``geo_b200``) never does.

Contents
--------
* ``sc_oracle.c`` -- plain-C restatement of the reference's SC forward, built by
  :func:`build` with gcc into ``oracle/_build/libsc_oracle.so`` and bound here
  with ctypes (:func:`conv2d`, :func:`act_streams`, :func:`weight_streams`).
* ``guide.py`` -- fp32 PyTorch restatement of the reference's float "guide"
  forward whose autograd is the training backward.
* ``build_ref.py`` / ``ref_loader.py`` -- build and load the reference's own
  extension sources, unmodified, into ``oracle/_ref``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# where the reference's source tree is mounted, when it is (build of oracle/_ref, fixture generation)
# GEO_REFERENCE_ROOT, else a checkout named "reference" beside this repository
REFERENCE_ROOT = os.environ.get("GEO_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
BUILD_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(BUILD_DIR, "libsc_oracle.so")

MODE_1D, MODE_Z, MODE_YZ, MODE_FULL_OR, MODE_2D, MODE_FULL_BIN = 0, 1, 2, 3, 4, 5
MODES = {"1d_bin": MODE_1D, "z_bin": MODE_Z, "yz_bin": MODE_YZ, "full_or": MODE_FULL_OR, "2d_bin": MODE_2D,
         "full_bin": MODE_FULL_BIN}

_lib = None


def build(force: bool = False) -> str:
    """Compile ``sc_oracle.c`` with gcc (OpenMP linked by name, see build_ref.py)."""
    src = os.path.join(HERE, "sc_oracle.c")
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= os.path.getmtime(src):
        return LIB_PATH
    os.makedirs(BUILD_DIR, exist_ok=True)
    obj = os.path.join(BUILD_DIR, "sc_oracle.o")
    subprocess.run(["gcc", "-O2", "-fPIC", "-fopenmp", "-c", src, "-o", obj], check=True)
    subprocess.run(["gcc", "-shared", obj, "-o", LIB_PATH, "-L/usr/lib/gcc/x86_64-linux-gnu/13", "-lgomp", "-lm"],
                   check=True)
    os.remove(obj)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = ctypes.CDLL(LIB_PATH)
        i = ctypes.c_int
        fp = ctypes.c_void_p
        L.geo_oracle_lfsr_step.argtypes = [i, i]
        L.geo_oracle_lfsr_step.restype = i
        for n in ("geo_oracle_quant_act", "geo_oracle_quant_wpos", "geo_oracle_quant_wneg"):
            getattr(L, n).argtypes = [ctypes.c_float, i]
            getattr(L, n).restype = i
        L.geo_oracle_act_streams.argtypes = [fp, i, i, i, i, i, i, i, i, i, i, fp]
        L.geo_oracle_weight_streams.argtypes = [fp, i, i, i, i, i, i, i, i, i, i, fp]
        L.geo_oracle_accumulate.argtypes = [fp, fp, i, i, i, i, i, i, i, i, i, i, fp]
        L.geo_oracle_conv2d.argtypes = [fp, fp] + [i] * 14 + [fp]
        _lib = L
    return _lib


def _f32(x):
    if hasattr(x, "detach"):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(x, dtype=np.float32)


def _mode(mode):
    return MODES[mode] if isinstance(mode, str) else int(mode)


def lfsr_step(v: int, nbits: int) -> int:
    return lib().geo_oracle_lfsr_step(int(v), int(nbits))


def act_streams(act, L, mode="1d_bin", z_unit=1 << 20, total_width=7, load_width=8, load_wait_a=1):
    """Packed activation streams, uint32 [B][C][H][W][P]; ``act`` is already padded."""
    a = _f32(act)
    B, C, H, W = a.shape
    P = (L + 31) // 32
    out = np.zeros((B, C, H, W, P), np.uint32)
    rc = lib().geo_oracle_act_streams(a.ctypes.data, B, C, H, W, L, _mode(mode), z_unit, total_width, load_width,
                                      load_wait_a, out.ctypes.data)
    if rc:
        raise ValueError(f"oracle act_streams failed rc={rc}")
    return out


def weight_streams(w, L, mode="1d_bin", z_unit=1 << 20, total_width=7, load_width=8, load_wait_w=1):
    """Packed weight streams, uint32 [2][O][C][K2][K3][P] (plane 0 positive, 1 negative)."""
    w_ = _f32(w)
    O, C, K2, K3 = w_.shape
    P = (L + 31) // 32
    out = np.zeros((2, O, C, K2, K3, P), np.uint32)
    rc = lib().geo_oracle_weight_streams(w_.ctypes.data, O, C, K2, K3, L, _mode(mode), z_unit, total_width,
                                         load_width, load_wait_w, out.ctypes.data)
    if rc:
        raise ValueError(f"oracle weight_streams failed rc={rc}")
    return out


def pad_act(act, pad_h=0, pad_w=0):
    a = _f32(act)
    if pad_h or pad_w:
        a = np.pad(a, ((0, 0), (0, 0), (pad_h, pad_h), (pad_w, pad_w)))
    return a


def conv2d(act, w, L, mode="1d_bin", z_unit=1 << 20, total_width=7, load_width=8, load_wait_w=1, load_wait_a=None,
           pad_h=0, pad_w=0):
    """SC conv2d forward, int32 [B][O][Ho][Wo].  ``pad_h``/``pad_w`` zero-pad dims 2/3 first."""
    if load_wait_a is None:
        load_wait_a = load_wait_w
    a = pad_act(act, pad_h, pad_w)
    w_ = _f32(w)
    B, C, H, W = a.shape
    O, C2, K2, K3 = w_.shape
    assert C == C2
    out = np.zeros((B, O, H - K2 + 1, W - K3 + 1), np.int32)
    rc = lib().geo_oracle_conv2d(a.ctypes.data, w_.ctypes.data, B, C, H, W, O, K2, K3, L, _mode(mode), z_unit,
                                 total_width, load_width, load_wait_w, load_wait_a, out.ctypes.data)
    if rc:
        raise ValueError(f"oracle conv2d failed rc={rc}")
    return out


def linear(act, w, L, z_unit=16, total_width=7, load_width=8, load_wait_w=1, load_wait_a=None):
    """SC linear = yz_bin conv on a 1x1 image: OR inside groups of ``z_unit`` inputs,
    binary accumulation across groups.  act [B][F], w [O][F] -> int32 [B][O]."""
    a = _f32(act)
    w_ = _f32(w)
    out = conv2d(a[:, :, None, None], w_[:, :, None, None], L, "yz_bin", z_unit, total_width, load_width,
                 load_wait_w, load_wait_a)
    return out[:, :, 0, 0]
