// Python module `sc_extension_cuda`: the reference's GPU extension API (sc_cuda.cpp:78-83),
// same function names, positional arguments and return type (int32 CUDA tensor), served by
// libgeo_sc.so.  This file has no kernels; it is a binding over the C ABI.
#include <atomic>

#include "sc_torch_shim.h"

using geo_shim::sc_conv2d;

// sc_cuda.cpp:47-63.  dim == 0 -> z-dimension binary accumulation, anything else -> y-dimension.
// `stride` is accepted and ignored (as in the reference); `im2col` selected between two
// reference kernels with identical results for dim != 0 and is ignored.
static at::Tensor conv2d_add_partial_variable_acc(at::Tensor input, at::Tensor weight, int64_t bit_length,
                                                  at::IntArrayRef padding, at::IntArrayRef stride, int64_t total_width,
                                                  int64_t load_width, int64_t load_wait, bool im2col, int64_t dim) {
    (void)stride;
    TORCH_CHECK(!(dim == 0 && im2col),
                "z_bin with im2col=True seeds activations per (c,ky) after im2col in the reference "
                "(sc_cuda_kernel.cu:1500-1624); that variant is not provided");
    return sc_conv2d(input, weight, bit_length, padding, dim == 0 ? GEO_SC_MODE_Z : GEO_SC_MODE_1D, 1, total_width,
                     load_width, load_wait, load_wait);
}

// sc_cuda.cpp:34-45.
static at::Tensor conv2d_add_yz_variable_acc(at::Tensor input, at::Tensor weight, int64_t bit_length,
                                             at::IntArrayRef padding, at::IntArrayRef stride, int64_t total_width,
                                             int64_t load_width, int64_t load_wait_w, int64_t load_wait_a, bool im2col,
                                             int64_t z_unit) {
    (void)stride;
    (void)im2col;
    return sc_conv2d(input, weight, bit_length, padding, GEO_SC_MODE_YZ, z_unit, total_width, load_width, load_wait_w,
                     load_wait_a);
}

// sc_cuda.cpp:65-76.  y-dimension accumulation with the "accurate" generator (sampling without
// replacement, every stream holds exactly as many ones as its level).  The reference draws from cuRAND
// states that its thread blocks share and race on (sc_cuda_kernel.cu:517), so its output is not
// reproducible even against itself.  Served here by the counter-based accurate generator
// (GEO_SC_GEN_ACC); every call takes the next seed of a process-wide counter, as a random generator
// would move on.
static at::Tensor conv2d_add_partial_acc_acc(at::Tensor input, at::Tensor weight, int64_t bit_length,
                                             at::IntArrayRef padding, at::IntArrayRef stride, bool share, int64_t dim) {
    (void)stride;
    (void)share;
    (void)dim;
    static std::atomic<uint32_t> calls{0};
    return sc_conv2d(input, weight, bit_length, padding, GEO_SC_MODE_1D, 1, 7, 8, 1, 1, GEO_SC_GEN_ACC, ++calls);
}

// sc_cuda.cpp:21-32.  Full OR accumulation.  The reference uses cuRAND here as well (same
// race, sc_cuda_kernel.cu:1315); served by the LFSR generator with the seed layout of the
// reference's bit-serial simulation (utils_functional.py:562-570).
static at::Tensor conv2d_or_acc(at::Tensor input, at::Tensor weight, int64_t bit_length, at::IntArrayRef padding,
                                at::IntArrayRef stride, bool im2col) {
    (void)stride;
    (void)im2col;
    return sc_conv2d(input, weight, bit_length, padding, GEO_SC_MODE_FULL_OR, 1, 7, 8, 1, 1);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("conv2d_add_partial_variable_acc", &conv2d_add_partial_variable_acc,
          "SC forward conv2d partial (y or z dimension) bin add variable load lfsr generator");
    m.def("conv2d_add_yz_variable_acc", &conv2d_add_yz_variable_acc,
          "SC forward conv2d partial (yz dimension) bin add variable load lfsr generator");
    m.def("conv2d_add_partial_acc_acc", &conv2d_add_partial_acc_acc,
          "SC forward conv2d partial bin add, accurate generator (counter-based, reproducible)");
    m.def("conv2d_or_acc", &conv2d_or_acc, "SC forward conv2d or add (deterministic generator)");
}
