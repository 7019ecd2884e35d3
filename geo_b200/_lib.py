"""ctypes binding of ``libgeo_sc.so`` (the C ABI declared in ``include/geo_sc.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libgeo_sc.so")

MODE_1D, MODE_Z, MODE_YZ, MODE_FULL_OR, MODE_2D, MODE_FULL_BIN = 0, 1, 2, 3, 4, 5
MODES = {"1d_bin": MODE_1D, "z_bin": MODE_Z, "yz_bin": MODE_YZ, "full_or": MODE_FULL_OR, "2d_bin": MODE_2D,
         "full_bin": MODE_FULL_BIN}


class GeoScError(RuntimeError):
    def __init__(self, status, what, detail):
        self.status = status
        super().__init__(f"{what}: status {status} ({detail})")


class ConvDesc(ctypes.Structure):
    """Mirror of ``geo_sc_conv_desc``."""

    _fields_ = [(n, ctypes.c_int32) for n in (
        "batch", "c_in", "h_in", "w_in", "pad_h", "pad_w", "c_out", "k_h", "k_w", "bit_length", "mode", "z_unit",
        "total_width", "load_width", "load_wait_w", "load_wait_a", "generator")] + [("seed", ctypes.c_uint32)]


GENERATORS = {"lfsr": 0, "acc": 1, "rand": 2}


_lib = None


def lib():
    """Load ``libgeo_sc.so`` (built by ``python -m geo_b200.build``) and declare its prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python -m geo_b200.build` (there is no fallback path)")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    dp = ctypes.POINTER(ConvDesc)
    szp = ctypes.POINTER(ctypes.c_size_t)
    L.geo_sc_version.restype = i32
    L.geo_sc_status_string.restype = ctypes.c_char_p
    L.geo_sc_status_string.argtypes = [i32]
    L.geo_sc_last_error.restype = ctypes.c_char_p
    L.geo_sc_init.restype = i32
    L.geo_sc_device_error_count.argtypes = [ctypes.POINTER(i32)]
    L.geo_sc_device_error_count.restype = i32
    for n in ("geo_sc_conv2d_workspace_bytes", "geo_sc_weight_prep_bytes", "geo_sc_act_stream_bytes"):
        getattr(L, n).argtypes = [dp, szp]
        getattr(L, n).restype = i32
    L.geo_sc_conv2d_forward.argtypes = [dp, vp, vp, vp, vp, sz, vp]
    L.geo_sc_linear_forward.argtypes = [dp, vp, vp, vp, vp, sz, vp]
    L.geo_sc_prepare_weights.argtypes = [dp, vp, vp, sz, vp]
    L.geo_sc_generate_act_streams.argtypes = [dp, vp, vp, sz, vp]
    L.geo_sc_accumulate.argtypes = [dp, vp, vp, vp, vp]
    i32p = ctypes.POINTER(ctypes.c_int32)
    L.geo_sc_group_geometry.argtypes = [dp, i32p, i32p, i32p, i32p, i32p]
    L.geo_sc_host_stream.argtypes = [i32] * 7 + [vp]
    L.geo_sc_static_scratch_bytes.restype = ctypes.c_size_t
    L.geo_sc_conv2d_forward_static.argtypes = [dp, vp, vp, vp, vp]
    L.geo_sc_conv2d_forward_static.restype = i32
    f32 = ctypes.c_float
    L.geo_sc_bn_fixed_scratch_bytes.argtypes = [i32, i32, szp]
    L.geo_sc_bn_fixed_forward.argtypes = [i32, i32, i32, i32, f32, f32] + [vp] * 10 + [sz, vp]
    L.geo_sc_bn_fixed_backward.argtypes = [i32, i32, i32, i32] + [vp] * 9 + [sz, vp]
    L.geo_sc_accumulate_is_sign_sorted.argtypes = [dp, ctypes.POINTER(i32)]
    L.geo_sc_accumulate_kernel.argtypes = [dp, ctypes.POINTER(i32)]
    L.geo_sc_act_stream_layout.argtypes = [dp, ctypes.POINTER(i32), ctypes.POINTER(i32)]
    L.geo_sc_quantize.argtypes = [vp, vp, sz, i32, vp]
    L.geo_sc_counts_to_float.argtypes = [vp, vp, sz, i32, vp]
    L.geo_sc_bn_pool_act_forward.argtypes = [i32, i32, i32, i32, i32, f32, f32] + [vp] * 12 + [sz, vp]
    L.geo_sc_bn_pool_act_backward.argtypes = [i32, i32, i32, i32, i32] + [vp] * 11 + [sz, vp]
    L.geo_sc_epilogue_forward.argtypes = [dp, i32, i32, i32, f32, f32] + [vp] * 12 + [sz, vp, sz, vp]
    L.geo_sc_epilogue_backward.argtypes = [i32] * 6 + [vp] * 10 + [vp, sz, vp]
    L.geo_sc_epilogue_forward.restype = i32
    L.geo_sc_epilogue_backward.restype = i32
    L.geo_sc_pool_act_forward.argtypes = [i32, i32, i32, vp, vp, vp]
    L.geo_sc_pool_act_backward.argtypes = [i32, i32, i32, vp, vp, vp, vp]
    L.geo_sc_guide_backward_bytes.argtypes = [dp, szp]
    L.geo_sc_guide_backward.argtypes = [dp, vp, vp, vp, vp, vp, vp, sz, vp]
    L.geo_sc_guide_backward_quantized.argtypes = [dp, vp, vp, vp, vp, vp, vp, sz, vp]
    L.geo_sc_measure_lop3_peak.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    for n in ("geo_sc_conv2d_forward", "geo_sc_linear_forward", "geo_sc_prepare_weights",
              "geo_sc_generate_act_streams", "geo_sc_accumulate", "geo_sc_group_geometry", "geo_sc_host_stream",
              "geo_sc_measure_lop3_peak", "geo_sc_guide_backward_bytes", "geo_sc_guide_backward",
              "geo_sc_guide_backward_quantized", "geo_sc_quantize", "geo_sc_counts_to_float", "geo_sc_accumulate_is_sign_sorted", "geo_sc_accumulate_kernel", "geo_sc_act_stream_layout", "geo_sc_bn_pool_act_forward", "geo_sc_bn_pool_act_backward",
              "geo_sc_bn_fixed_scratch_bytes",
              "geo_sc_bn_fixed_forward", "geo_sc_bn_fixed_backward", "geo_sc_pool_act_forward",
              "geo_sc_pool_act_backward"):
        getattr(L, n).restype = i32
    _lib = L
    return L


def check(status, what):
    if status != 0:
        L = lib()
        detail = L.geo_sc_last_error().decode() or L.geo_sc_status_string(status).decode()
        raise GeoScError(status, what, detail)


def make_desc(batch, c_in, h_in, w_in, c_out, k_h, k_w, bit_length, mode="1d_bin", pad_h=0, pad_w=0, z_unit=1 << 20,
              total_width=7, load_width=8, load_wait_w=1, load_wait_a=None, generator="lfsr", seed=0):
    if load_wait_a is None:
        load_wait_a = load_wait_w
    m = MODES[mode] if isinstance(mode, str) else int(mode)
    gen = GENERATORS[generator] if isinstance(generator, str) else int(generator)
    return ConvDesc(batch, c_in, h_in, w_in, pad_h, pad_w, c_out, k_h, k_w, bit_length, m, min(int(z_unit), 1 << 30),
                    total_width, load_width, load_wait_w, load_wait_a, gen, int(seed) & 0xFFFFFFFF)


def size_query(fn_name, desc):
    out = ctypes.c_size_t(0)
    check(getattr(lib(), fn_name)(ctypes.byref(desc), ctypes.byref(out)), fn_name)
    return out.value


def group_geometry(desc):
    """(groups, members, c_out tile, padded c_out) of the prepared-weight layout."""
    return group_geometry_full(desc)[:2] + group_geometry_full(desc)[3:]


def group_geometry_full(desc):
    """(groups, members, members as laid out (padded to 16), c_out tile, padded c_out)."""
    g, k, kp, nt, op = (ctypes.c_int32(0) for _ in range(5))
    check(lib().geo_sc_group_geometry(ctypes.byref(desc), ctypes.byref(g), ctypes.byref(k), ctypes.byref(kp),
                                      ctypes.byref(nt), ctypes.byref(op)), "geo_sc_group_geometry")
    return g.value, k.value, kp.value, nt.value, op.value


KERNEL_NAMES = ("dense", "sorted_im2col", "sorted_rows", "sorted_short", "full_bin", "sorted_taps")


def accumulate_kernel(desc):
    """Name of the accumulation kernel this descriptor gets (one of KERNEL_NAMES)."""
    k = ctypes.c_int32(0)
    check(lib().geo_sc_accumulate_kernel(ctypes.byref(desc), ctypes.byref(k)), "geo_sc_accumulate_kernel")
    return KERNEL_NAMES[k.value]


def act_stream_layout(desc):
    """(batch_innermost, batch extent) of the activation-stream image of this descriptor."""
    bf, bp = ctypes.c_int32(0), ctypes.c_int32(0)
    check(lib().geo_sc_act_stream_layout(ctypes.byref(desc), ctypes.byref(bf), ctypes.byref(bp)), "geo_sc_act_stream_layout")
    return bool(bf.value), bp.value


def is_sign_sorted(desc):
    """True if the accumulation of this descriptor runs on the sign-sorted kernel."""
    yes = ctypes.c_int32(0)
    check(lib().geo_sc_accumulate_is_sign_sorted(ctypes.byref(desc), ctypes.byref(yes)), "geo_sc_accumulate_is_sign_sorted")
    return bool(yes.value)


def device_error_count():
    """Bounded hardware-barrier waits that ran out on the current device since the library was loaded."""
    n = ctypes.c_int32(0)
    check(lib().geo_sc_device_error_count(ctypes.byref(n)), "geo_sc_device_error_count")
    return n.value


def host_stream(bit_length, value, seed_base, seed_index, total_width=7, load_width=8, load_wait=1):
    """Packed stream words of one integer level, computed on the CPU with the kernels' own tables."""
    P = (bit_length + 31) // 32
    buf = (ctypes.c_uint32 * P)()
    check(lib().geo_sc_host_stream(bit_length, value, seed_base, seed_index, total_width, load_width, load_wait,
                                   ctypes.cast(buf, ctypes.c_void_p)), "geo_sc_host_stream")
    return list(buf)
