// Shared helper of the two pybind11 shims: turns torch tensors into a geo_sc_conv_desc plus raw
// device pointers, calls the C ABI on torch's current stream with a workspace from torch's
// caching allocator, and turns a non-zero status into a Python exception.
#pragma once

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "geo_sc.h"

namespace geo_shim {

inline at::Tensor sc_conv2d(const at::Tensor &input, const at::Tensor &weight, int64_t bit_length,
                            at::IntArrayRef padding, int mode, int64_t z_unit, int64_t total_width,
                            int64_t load_width, int64_t load_wait_w, int64_t load_wait_a,
                            int generator = GEO_SC_GEN_LFSR, uint32_t seed = 0) {
    TORCH_CHECK(input.is_cuda() && weight.is_cuda(),
                "geo_b200 SC kernels run on CUDA tensors only (there is no CPU path in this build)");
    TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "expected NCHW input and OIHW weight");
    TORCH_CHECK(input.size(1) == weight.size(1), "channel mismatch between input and weight");
    TORCH_CHECK(padding.size() == 2, "padding must have two entries");
    c10::cuda::CUDAGuard guard(input.device());
    at::Tensor a = input.to(at::kFloat).contiguous();
    at::Tensor w = weight.to(input.device(), at::kFloat).contiguous();

    geo_sc_conv_desc d = {};
    d.generator = generator;
    d.seed = seed;
    d.batch = (int32_t)a.size(0); d.c_in = (int32_t)a.size(1); d.h_in = (int32_t)a.size(2); d.w_in = (int32_t)a.size(3);
    // F::pad(input, {p0, p0, p1, p1}) pads the last dimension by p0 and dimension 2 by p1.
    d.pad_w = (int32_t)padding[0]; d.pad_h = (int32_t)padding[1];
    d.c_out = (int32_t)w.size(0); d.k_h = (int32_t)w.size(2); d.k_w = (int32_t)w.size(3);
    d.bit_length = (int32_t)bit_length;
    d.mode = mode;
    d.z_unit = (int32_t)std::min<int64_t>(std::max<int64_t>(z_unit, 0), 1 << 30);
    d.total_width = (int32_t)total_width; d.load_width = (int32_t)load_width;
    d.load_wait_w = (int32_t)load_wait_w; d.load_wait_a = (int32_t)load_wait_a;

    size_t bytes = 0;
    int rc = geo_sc_conv2d_workspace_bytes(&d, &bytes);
    TORCH_CHECK(rc == 0, "geo_sc: ", geo_sc_status_string(rc), ": ", geo_sc_last_error());
    const int64_t Ho = d.h_in + 2 * d.pad_h - d.k_h + 1, Wo = d.w_in + 2 * d.pad_w - d.k_w + 1;
    at::Tensor ws = at::empty({(int64_t)bytes}, a.options().dtype(at::kByte));
    at::Tensor out = at::empty({d.batch, d.c_out, Ho, Wo}, a.options().dtype(at::kInt));
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(a.device().index()).stream();
    rc = geo_sc_conv2d_forward(&d, a.data_ptr<float>(), w.data_ptr<float>(), out.data_ptr<int32_t>(), ws.data_ptr(),
                               bytes, (void *)stream);
    TORCH_CHECK(rc == 0, "geo_sc: ", geo_sc_status_string(rc), ": ", geo_sc_last_error());
    return out;
}

}  // namespace geo_shim
