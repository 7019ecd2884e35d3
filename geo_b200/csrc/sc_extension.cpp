// Python module `sc_extension`: the name of the reference's CPU extension (sc.cpp:474-476),
// which utils_functional.py imports unconditionally.  This build has no CPU compute path:
// the function runs CUDA tensors through libgeo_sc.so (y-dimension binary accumulation, LFSR,
// no progressive loading -- what sc.cpp:292-472 computes) and refuses CPU tensors loudly.
#include "sc_torch_shim.h"

static at::Tensor conv2d_add_partial_new(at::Tensor input, at::Tensor weight, int64_t bit_length,
                                         at::IntArrayRef padding, at::IntArrayRef stride) {
    (void)stride;
    return geo_shim::sc_conv2d(input, weight, bit_length, padding, GEO_SC_MODE_1D, 1, 7, 8, 1, 1);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("conv2d_add_partial_new", &conv2d_add_partial_new, "SC forward conv2d partial bin add (CUDA tensors only)");
}
