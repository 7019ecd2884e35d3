// The layers between SC convolutions as native kernels: quantised batch normalisation (below),
// 2x2 average pooling + hardtanh, the fixed-point rounding of activations and weights
// (utils_functional.py:33-39) and the hand-off from bit counts to the layer's float value
// (further down, each with its own note).
//
// Quantised batch normalisation ("BatchNorm*_fixed", utils_class.py:37-93).
//
// The reference computes it with F.batch_norm (for the autograd graph), separate mean / var
// reductions, a dozen small element-wise ops for the 7-bit folded scale and shift
// (quantize_shift, utils_functional.py:41-57) and a final x * w_q + b_q that replaces the value.
// Here: two deterministic reduction passes (mean, then squared deviations), one single-CTA
// kernel that folds, quantises and updates the running statistics, and one apply pass.  The
// backward pass is the ordinary batch-norm gradient with respect to the *unquantised*
// normalisation, which is what the reference's graph differentiates:
//     dgamma = sum g * xhat,  dbeta = sum g,  dx = gamma * invstd * (g - dbeta/N - xhat * dgamma/N)
// (in evaluation mode dx = gamma * invstd * g).  Layout: x [B][C][HW] (HW = 1 for the 1d variant).
#include "sc_common.h"
#include "sc_pool.h"

namespace geo {

namespace {

constexpr int BN_THREADS = 256;

struct BnDims {
    int B, C, HW, S;  // S = batch slices per channel in the reduction passes
};

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = 0.f;
    if (threadIdx.x < 32) {
        r = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    }
    return r;  // valid in thread 0
}

// mode 0: sum(x)   mode 1: sum((x - mean)^2)   -> partial[c][s]
// VEC: rows of HW floats are read as float4 (HW % 4 == 0, 16-byte aligned base).
template <int MODE, bool VEC>
__global__ void __launch_bounds__(BN_THREADS) bn_reduce_kernel(BnDims d, XSource xs,
                                                               const float *__restrict__ mean,
                                                               float *__restrict__ partial) {
    const float *x = (const float *)xs.p;   // scalar path: fp32 only
    __shared__ float red[32];
    const int c = blockIdx.x, s = blockIdx.y;
    const int b0 = (int)((long long)d.B * s / d.S), b1 = (int)((long long)d.B * (s + 1) / d.S);
    const float mu = MODE == 1 ? mean[c] : 0.f;
    float acc = 0.f;
    if (VEC) {
        const unsigned q = (unsigned)d.HW >> 2, n = (unsigned)(b1 - b0) * q;
        float a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (unsigned i = threadIdx.x; i < n; i += BN_THREADS) {
            const unsigned b = b0 + i / q, p = i % q;
            const float4 v = load_x4(xs, (((size_t)b * d.C + c) * d.HW >> 2) + p);
            if (MODE == 0) { acc += v.x; a1 += v.y; a2 += v.z; a3 += v.w; }
            else {
                acc = fmaf(v.x - mu, v.x - mu, acc); a1 = fmaf(v.y - mu, v.y - mu, a1);
                a2 = fmaf(v.z - mu, v.z - mu, a2); a3 = fmaf(v.w - mu, v.w - mu, a3);
            }
        }
        acc = (acc + a1) + (a2 + a3);
    } else {
        const unsigned n = (unsigned)(b1 - b0) * (unsigned)d.HW;
        for (unsigned i = threadIdx.x; i < n; i += BN_THREADS) {
            const unsigned b = b0 + i / (unsigned)d.HW, p = i % (unsigned)d.HW;
            const float v = x[((size_t)b * d.C + c) * d.HW + p];
            if (MODE == 0) acc += v;
            else acc = fmaf(v - mu, v - mu, acc);
        }
    }
    const float tot = block_sum(acc, red);
    if (threadIdx.x == 0) partial[c * d.S + s] = tot;
}

__global__ void __launch_bounds__(BN_THREADS) bn_mean_kernel(BnDims d, const float *__restrict__ partial,
                                                             float *__restrict__ mean) {
    const float inv_n = 1.0f / ((float)d.B * (float)d.HW);
    for (int c = blockIdx.x * BN_THREADS + threadIdx.x; c < d.C; c += gridDim.x * BN_THREADS) {
        float s = 0.f;
        for (int i = 0; i < d.S; i++) s += partial[c * d.S + i];
        mean[c] = s * inv_n;
    }
}

// Single CTA: variance, invstd, running statistics, folded scale/shift and their 7-bit
// quantisation under one power-of-two range (quantize_shift).
__global__ void __launch_bounds__(BN_THREADS) bn_fold_kernel(BnDims d, int training, float eps, float momentum,
                                                             const float *__restrict__ partial2, float *mean,
                                                             float *invstd, const float *__restrict__ weight,
                                                             const float *__restrict__ bias, float *running_mean,
                                                             float *running_var, float *wq, float *bq, float *scale_out) {
    __shared__ float red[32];
    __shared__ float s_scale;
    const float n = (float)d.B * (float)d.HW;
    // pass A: per-channel statistics and the unquantised folded scale; sum of scales for the range
    float local = 0.f;
    for (int c = threadIdx.x; c < d.C; c += BN_THREADS) {
        float mu, var;
        if (training) {
            float s = 0.f;
            for (int i = 0; i < d.S; i++) s += partial2[c * d.S + i];
            var = s / n;
            mu = mean[c];
            if (running_mean) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mu;
            if (running_var) running_var[c] = (1.f - momentum) * running_var[c] + momentum * (n > 1.f ? s / (n - 1.f) : var);
        } else {
            mu = running_mean[c];
            var = running_var[c];
            mean[c] = mu;
        }
        const float sd = sqrtf(var + eps);
        invstd[c] = 1.0f / sd;
        const float w = weight ? weight[c] : 1.0f;
        const float wn = w / sd;
        wq[c] = wn;  // unquantised for now
        local += wn;
    }
    const float tot = block_sum(local, red);
    if (threadIdx.x == 0) {
        // scale = 2 ** ceil(log2(mean(w_n) * 3))
        const float m3 = tot / (float)d.C * 3.0f;
        s_scale = exp2f(ceilf(log2f(m3)));
        scale_out[0] = s_scale;
    }
    __syncthreads();
    const float scale = s_scale;
    for (int c = threadIdx.x; c < d.C; c += BN_THREADS) {
        const float w = weight ? weight[c] : 1.0f;
        const float b = bias ? bias[c] : 0.0f;
        const float sd = 1.0f / invstd[c];
        const float wn = wq[c];
        const float bn = b - mean[c] * w / sd;
        const float qw = fminf(fmaxf(rintf(wn / scale * 128.0f), -127.0f), 127.0f) / 128.0f * scale;
        const float qb = fminf(fmaxf(rintf(bn / scale * 128.0f), -127.0f), 127.0f) / 128.0f * scale;
        wq[c] = qw;
        bq[c] = qb;
    }
}

template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS) bn_apply_kernel(BnDims d, const float *__restrict__ x,
                                                              const float *__restrict__ wq, const float *__restrict__ bq,
                                                              float *__restrict__ out) {
    const unsigned stride = gridDim.x * BN_THREADS;
    if (VEC) {
        const unsigned q = (unsigned)d.HW >> 2, total = (unsigned)d.B * d.C * q;
        for (unsigned i = blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += stride) {
            const unsigned c = (i / q) % (unsigned)d.C;
            const float w = wq[c], b = bq[c];
            const float4 v = __ldg((const float4 *)x + i);
            ((float4 *)out)[i] = make_float4(v.x * w + b, v.y * w + b, v.z * w + b, v.w * w + b);
        }
    } else {
        const unsigned total = (unsigned)d.B * d.C * d.HW;
        for (unsigned i = blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += stride) {
            const unsigned c = (i / (unsigned)d.HW) % (unsigned)d.C;
            out[i] = x[i] * wq[c] + bq[c];
        }
    }
}

// backward pass 1: partial sums of g and g * xhat
template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_reduce_kernel(BnDims d, const float *__restrict__ x,
                                                                   const float *__restrict__ g,
                                                                   const float *__restrict__ mean,
                                                                   const float *__restrict__ invstd,
                                                                   float *__restrict__ partial) {
    __shared__ float red[32];
    const int c = blockIdx.x, s = blockIdx.y;
    const int b0 = (int)((long long)d.B * s / d.S), b1 = (int)((long long)d.B * (s + 1) / d.S);
    const float mu = mean[c], is = invstd[c];
    float sg = 0.f, sgx = 0.f;
    if (VEC) {
        const unsigned q = (unsigned)d.HW >> 2, n = (unsigned)(b1 - b0) * q;
        float sg1 = 0.f, sgx1 = 0.f;
        for (unsigned i = threadIdx.x; i < n; i += BN_THREADS) {
            const unsigned b = b0 + i / q, p = i % q;
            const size_t row = ((size_t)b * d.C + c) * d.HW;
            const float4 gv = __ldg((const float4 *)(g + row) + p);
            const float4 xv = __ldg((const float4 *)(x + row) + p);
            sg += gv.x + gv.y; sg1 += gv.z + gv.w;
            sgx = fmaf(gv.x, (xv.x - mu) * is, sgx); sgx1 = fmaf(gv.y, (xv.y - mu) * is, sgx1);
            sgx = fmaf(gv.z, (xv.z - mu) * is, sgx); sgx1 = fmaf(gv.w, (xv.w - mu) * is, sgx1);
        }
        sg += sg1; sgx += sgx1;
    } else {
        const unsigned n = (unsigned)(b1 - b0) * (unsigned)d.HW;
        for (unsigned i = threadIdx.x; i < n; i += BN_THREADS) {
            const unsigned b = b0 + i / (unsigned)d.HW, p = i % (unsigned)d.HW;
            const size_t idx = ((size_t)b * d.C + c) * d.HW + p;
            const float gv = g[idx];
            sg += gv;
            sgx = fmaf(gv, (x[idx] - mu) * is, sgx);
        }
    }
    const float t0 = block_sum(sg, red);
    const float t1 = block_sum(sgx, red);
    if (threadIdx.x == 0) {
        partial[(c * d.S + s) * 2 + 0] = t0;
        partial[(c * d.S + s) * 2 + 1] = t1;
    }
}

__global__ void __launch_bounds__(BN_THREADS) bn_bwd_final_kernel(BnDims d, const float *__restrict__ partial,
                                                                  float *__restrict__ sums, float *grad_weight,
                                                                  float *grad_bias) {
    for (int c = blockIdx.x * BN_THREADS + threadIdx.x; c < d.C; c += gridDim.x * BN_THREADS) {
        float a = 0.f, b = 0.f;
        for (int i = 0; i < d.S; i++) {
            a += partial[(c * d.S + i) * 2 + 0];
            b += partial[(c * d.S + i) * 2 + 1];
        }
        sums[c * 2 + 0] = a;
        sums[c * 2 + 1] = b;
        if (grad_bias) grad_bias[c] = a;
        if (grad_weight) grad_weight[c] = b;
    }
}

template <bool VEC>
__global__ void __launch_bounds__(BN_THREADS) bn_bwd_apply_kernel(BnDims d, int training, const float *__restrict__ x,
                                                                  const float *__restrict__ g,
                                                                  const float *__restrict__ mean,
                                                                  const float *__restrict__ invstd,
                                                                  const float *__restrict__ weight,
                                                                  const float *__restrict__ sums,
                                                                  float *__restrict__ gx) {
    const float inv_n = 1.0f / ((float)d.B * (float)d.HW);
    const unsigned stride = gridDim.x * BN_THREADS;
    const unsigned q = VEC ? (unsigned)d.HW >> 2 : (unsigned)d.HW, total = (unsigned)d.B * d.C * q;
    for (unsigned i = blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += stride) {
        const unsigned c = (i / q) % (unsigned)d.C;
        const float w = weight ? weight[c] : 1.0f;
        const float is = invstd[c];
        const float k = w * is;
        // gx = w * is * (g - sum_g / N - xhat * sum_gx / N), same association per element
        const float a = training ? sums[c * 2] * inv_n : 0.f, bb = training ? sums[c * 2 + 1] * inv_n : 0.f;
        const float mu = mean[c];
        if (VEC) {
            const float4 gv = __ldg((const float4 *)g + i);
            float4 r;
            if (training) {
                const float4 xv = __ldg((const float4 *)x + i);
                r.x = k * (gv.x - a - (xv.x - mu) * is * bb);
                r.y = k * (gv.y - a - (xv.y - mu) * is * bb);
                r.z = k * (gv.z - a - (xv.z - mu) * is * bb);
                r.w = k * (gv.w - a - (xv.w - mu) * is * bb);
            } else {
                r = make_float4(k * gv.x, k * gv.y, k * gv.z, k * gv.w);
            }
            ((float4 *)gx)[i] = r;
        } else {
            gx[i] = training ? k * (g[i] - a - (x[i] - mu) * is * bb) : k * g[i];
        }
    }
}

// ---- batch norm + 2x2 average pool + hardtanh(0, 1) in one pass per direction -----------------------
// out = clamp(mean over the 2x2 window of (x * w_q + b_q), 0, 1).  A thread owns two horizontally
// adjacent windows = one float4 of each of the two input rows (even H, W % 4 == 0).  The backward pass
// recomputes the pooled value from x to decide whether the hardtanh passes the gradient, spreads it
// over the window (factor 1/4) and applies the batch-norm gradient to it -- the composition of the two
// separate backward passes without ever storing the normalised tensor or its gradient.
// Window rows: r = (b * C + c) * (H/2) + oy, input rows 2r and 2r + 1.
struct PoolWin {
    float4 t, b;       // the two input rows
    float v0, v1;      // pooled values before the clamp
};
__device__ __forceinline__ PoolWin load_windows(const XSource &xs, unsigned r, unsigned j, unsigned W, float w, float bq) {
    PoolWin p;
    p.t = load_x4(xs, ((size_t)(2 * r) * W >> 2) + j);
    p.b = load_x4(xs, ((size_t)(2 * r + 1) * W >> 2) + j);
    // same expressions as bn_apply_kernel and pool_act_fwd_kernel, so the value equals their composition
    p.v0 = pooled_value(p.t.x, p.t.y, p.b.x, p.b.y, w, bq);
    p.v1 = pooled_value(p.t.z, p.t.w, p.b.z, p.b.w, w, bq);
    return p;
}

__global__ void __launch_bounds__(BN_THREADS) bn_pool_apply_kernel(unsigned rows, unsigned W, unsigned Ho, unsigned C,
                                                                   XSource x,
                                                                   const float *__restrict__ wq,
                                                                   const float *__restrict__ bq, float *__restrict__ out) {
    const unsigned q = W >> 2, total = rows * q;
    for (unsigned i = blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += gridDim.x * BN_THREADS) {
        const unsigned r = i / q, j = i % q, c = (r / Ho) % C;
        const PoolWin p = load_windows(x, r, j, W, wq[c], bq[c]);
        ((float2 *)(out + (size_t)r * (W >> 1)))[j] = make_float2(fminf(fmaxf(p.v0, 0.0f), 1.0f), fminf(fmaxf(p.v1, 0.0f), 1.0f));
    }
}

// partial sums of gy and gy * xhat, gy = gradient reaching the batch-norm output
__global__ void __launch_bounds__(BN_THREADS) bn_pool_bwd_reduce_kernel(BnDims d, unsigned W, unsigned Ho,
                                                                        XSource x,
                                                                        const float *__restrict__ g,
                                                                        const float *__restrict__ mean,
                                                                        const float *__restrict__ invstd,
                                                                        const float *__restrict__ wq,
                                                                        const float *__restrict__ bq,
                                                                        float *__restrict__ partial) {
    __shared__ float red[32];
    const int c = blockIdx.x, s = blockIdx.y;
    const int b0 = (int)((long long)d.B * s / d.S), b1 = (int)((long long)d.B * (s + 1) / d.S);
    const float mu = mean[c], is = invstd[c], w = wq[c], bqc = bq[c];
    const unsigned q = W >> 2, per_img = Ho * q, n = (unsigned)(b1 - b0) * per_img;
    float sg = 0.f, sgx = 0.f;
    for (unsigned i = threadIdx.x; i < n; i += BN_THREADS) {
        const unsigned b = b0 + i / per_img, rem = i % per_img;
        const unsigned r = (b * d.C + c) * Ho + rem / q, j = rem % q;
        const PoolWin p = load_windows(x, r, j, W, w, bqc);
        const float2 gv = __ldg((const float2 *)(g + (size_t)r * (W >> 1)) + j);
        const float g0 = p.v0 > 0.0f && p.v0 < 1.0f ? gv.x * 0.25f : 0.0f;
        const float g1 = p.v1 > 0.0f && p.v1 < 1.0f ? gv.y * 0.25f : 0.0f;
        sg += 4.0f * g0 + 4.0f * g1;
        sgx = fmaf(g0, ((p.t.x - mu) + (p.t.y - mu) + (p.b.x - mu) + (p.b.y - mu)) * is, sgx);
        sgx = fmaf(g1, ((p.t.z - mu) + (p.t.w - mu) + (p.b.z - mu) + (p.b.w - mu)) * is, sgx);
    }
    const float t0 = block_sum(sg, red);
    const float t1 = block_sum(sgx, red);
    if (threadIdx.x == 0) {
        partial[(c * d.S + s) * 2 + 0] = t0;
        partial[(c * d.S + s) * 2 + 1] = t1;
    }
}

__global__ void __launch_bounds__(BN_THREADS) bn_pool_bwd_apply_kernel(BnDims d, unsigned rows, unsigned W, unsigned Ho,
                                                                       int training, XSource x,
                                                                       const float *__restrict__ g,
                                                                       const float *__restrict__ mean,
                                                                       const float *__restrict__ invstd,
                                                                       const float *__restrict__ weight,
                                                                       const float *__restrict__ sums,
                                                                       const float *__restrict__ wq,
                                                                       const float *__restrict__ bq,
                                                                       float *__restrict__ gx) {
    const float inv_n = 1.0f / ((float)d.B * (float)d.HW);
    const unsigned q = W >> 2, total = rows * q;
    for (unsigned i = blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += gridDim.x * BN_THREADS) {
        const unsigned r = i / q, j = i % q, c = (r / Ho) % (unsigned)d.C;
        const PoolWin p = load_windows(x, r, j, W, wq[c], bq[c]);
        const float2 gv = __ldg((const float2 *)(g + (size_t)r * (W >> 1)) + j);
        const float g0 = p.v0 > 0.0f && p.v0 < 1.0f ? gv.x * 0.25f : 0.0f;
        const float g1 = p.v1 > 0.0f && p.v1 < 1.0f ? gv.y * 0.25f : 0.0f;
        const float is = invstd[c], k = (weight ? weight[c] : 1.0f) * is, mu = mean[c];
        const float a = training ? sums[c * 2] * inv_n : 0.f, bb = training ? sums[c * 2 + 1] * inv_n : 0.f;
        float4 o0, o1;
        if (training) {
            o0 = make_float4(k * (g0 - a - (p.t.x - mu) * is * bb), k * (g0 - a - (p.t.y - mu) * is * bb),
                             k * (g1 - a - (p.t.z - mu) * is * bb), k * (g1 - a - (p.t.w - mu) * is * bb));
            o1 = make_float4(k * (g0 - a - (p.b.x - mu) * is * bb), k * (g0 - a - (p.b.y - mu) * is * bb),
                             k * (g1 - a - (p.b.z - mu) * is * bb), k * (g1 - a - (p.b.w - mu) * is * bb));
        } else {
            o0 = make_float4(k * g0, k * g0, k * g1, k * g1);
            o1 = o0;
        }
        ((float4 *)(gx + (size_t)(2 * r) * W))[j] = o0;
        ((float4 *)(gx + (size_t)(2 * r + 1) * W))[j] = o1;
    }
}

int bn_slices(int B, int C) {
    int S = (sm_count() * 4 + C - 1) / C;
    if (S > B) S = B;
    if (S < 1) S = 1;
    if (S > 64) S = 64;
    return S;
}

int bn_grid(long long total) {
    long long b = (total + BN_THREADS - 1) / BN_THREADS;
    return (int)(b < sm_count() * 8 ? (b > 0 ? b : 1) : sm_count() * 8);
}

}  // namespace

}  // namespace geo

using namespace geo;

extern "C" {

int geo_sc_bn_fixed_scratch_bytes(int batch, int channels, size_t *bytes) {
    if (batch < 1 || channels < 1) return fail(GEO_SC_ERR_SHAPE, "batch %d channels %d", batch, channels);
    if (!bytes) return fail(GEO_SC_ERR_NULL, "bytes is NULL");
    *bytes = align_up((size_t)channels * 64 * 2 * sizeof(float), 256) + align_up((size_t)channels * 4 * sizeof(float), 256);
    return GEO_SC_OK;
}

int geo_sc_bn_fixed_forward(int batch, int channels, int spatial, int training, float eps, float momentum,
                            const float *x, const float *weight, const float *bias, float *running_mean,
                            float *running_var, float *out, float *save_mean, float *save_invstd, float *scale_out,
                            void *scratch, size_t scratch_bytes, void *stream) {
    if (batch < 1 || channels < 1 || spatial < 1) return fail(GEO_SC_ERR_SHAPE, "batch %d channels %d spatial %d", batch, channels, spatial);
    if (!x || !out || !save_mean || !save_invstd || !scale_out || !scratch) return fail(GEO_SC_ERR_NULL, "a required pointer is NULL");
    if (!training && (!running_mean || !running_var)) return fail(GEO_SC_ERR_NULL, "evaluation mode needs running statistics");
    if ((long long)batch * channels * spatial > (1LL << 31) - 1) return fail(GEO_SC_ERR_TOO_LARGE, "tensor too large");
    size_t need = 0;
    geo_sc_bn_fixed_scratch_bytes(batch, channels, &need);
    if (scratch_bytes < need || ((uintptr_t)scratch & 255)) return fail(GEO_SC_ERR_WORKSPACE, "bn scratch holds %zu bytes, %zu needed", scratch_bytes, need);
    cudaStream_t s = (cudaStream_t)stream;
    BnDims d = {batch, channels, spatial, bn_slices(batch, channels)};
    float *partial = (float *)scratch;
    float *wq = (float *)((char *)scratch + align_up((size_t)channels * 64 * 2 * sizeof(float), 256));
    float *bq = wq + channels;
    const bool vec = spatial % 4 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
    if (training) {
        const XSource xs = {x, 1.0f, 0};
        if (vec) bn_reduce_kernel<0, true><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, xs, nullptr, partial);
        else bn_reduce_kernel<0, false><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, xs, nullptr, partial);
        bn_mean_kernel<<<(channels + BN_THREADS - 1) / BN_THREADS, BN_THREADS, 0, s>>>(d, partial, save_mean);
        if (vec) bn_reduce_kernel<1, true><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, xs, save_mean, partial);
        else bn_reduce_kernel<1, false><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, xs, save_mean, partial);
    }
    bn_fold_kernel<<<1, BN_THREADS, 0, s>>>(d, training, eps, momentum, partial, save_mean, save_invstd, weight, bias,
                                            running_mean, running_var, wq, bq, scale_out);
    if (vec) bn_apply_kernel<true><<<bn_grid((long long)batch * channels * spatial / 4), BN_THREADS, 0, s>>>(d, x, wq, bq, out);
    else bn_apply_kernel<false><<<bn_grid((long long)batch * channels * spatial), BN_THREADS, 0, s>>>(d, x, wq, bq, out);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int geo_sc_bn_fixed_backward(int batch, int channels, int spatial, int training, const float *x, const float *grad_out,
                             const float *weight, const float *save_mean, const float *save_invstd, float *grad_x,
                             float *grad_weight, float *grad_bias, void *scratch, size_t scratch_bytes, void *stream) {
    if (batch < 1 || channels < 1 || spatial < 1) return fail(GEO_SC_ERR_SHAPE, "batch %d channels %d spatial %d", batch, channels, spatial);
    if (!x || !grad_out || !save_mean || !save_invstd || !grad_x || !scratch) return fail(GEO_SC_ERR_NULL, "a required pointer is NULL");
    size_t need = 0;
    geo_sc_bn_fixed_scratch_bytes(batch, channels, &need);
    if (scratch_bytes < need || ((uintptr_t)scratch & 255)) return fail(GEO_SC_ERR_WORKSPACE, "bn scratch holds %zu bytes, %zu needed", scratch_bytes, need);
    cudaStream_t s = (cudaStream_t)stream;
    BnDims d = {batch, channels, spatial, bn_slices(batch, channels)};
    float *partial = (float *)scratch;
    float *sums = (float *)((char *)scratch + align_up((size_t)channels * 64 * 2 * sizeof(float), 256));
    if ((long long)batch * channels * spatial > (1LL << 31) - 1) return fail(GEO_SC_ERR_TOO_LARGE, "tensor too large");
    const bool vec = spatial % 4 == 0 && (((uintptr_t)x | (uintptr_t)grad_out | (uintptr_t)grad_x) & 15) == 0;
    if (vec) bn_bwd_reduce_kernel<true><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, x, grad_out, save_mean, save_invstd, partial);
    else bn_bwd_reduce_kernel<false><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, x, grad_out, save_mean, save_invstd, partial);
    bn_bwd_final_kernel<<<(channels + BN_THREADS - 1) / BN_THREADS, BN_THREADS, 0, s>>>(d, partial, sums, grad_weight, grad_bias);
    if (vec)
        bn_bwd_apply_kernel<true><<<bn_grid((long long)batch * channels * spatial / 4), BN_THREADS, 0, s>>>(
            d, training, x, grad_out, save_mean, save_invstd, weight, sums, grad_x);
    else
        bn_bwd_apply_kernel<false><<<bn_grid((long long)batch * channels * spatial), BN_THREADS, 0, s>>>(
            d, training, x, grad_out, save_mean, save_invstd, weight, sums, grad_x);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}


static int bn_pool_check(int batch, int channels, int height, int width, const void *a, const void *b, const void *c) {
    if (batch < 1 || channels < 1 || height < 2 || width < 4 || height % 2 || width % 4)
        return fail(GEO_SC_ERR_SHAPE, "the fused form needs an even height and a width that is a multiple of 4 (got %dx%d)", height, width);
    if ((long long)batch * channels * height * width > (1LL << 31) - 1) return fail(GEO_SC_ERR_TOO_LARGE, "tensor too large");
    if ((((uintptr_t)a | (uintptr_t)c) & 15) || ((uintptr_t)b & 7)) return fail(GEO_SC_ERR_SHAPE, "x / grad_x need 16-byte, pooled tensors 8-byte alignment");
    return GEO_SC_OK;
}

// Statistics and folded scale / shift of the pooled forms; x as fp32 or as bit counts.
static int bn_pool_stats(int batch, int channels, int height, int width, int training, float eps, float momentum, XSource xs,
                         const float *weight, const float *bias, float *running_mean, float *running_var, float *save_mean,
                         float *save_invstd, float *save_wq, float *save_bq, float *scale_out, void *scratch,
                         size_t scratch_bytes, cudaStream_t s) {
    if (!xs.p || !save_mean || !save_invstd || !save_wq || !save_bq || !scale_out || !scratch) return fail(GEO_SC_ERR_NULL, "a required pointer is NULL");
    if (!training && (!running_mean || !running_var)) return fail(GEO_SC_ERR_NULL, "evaluation mode needs running statistics");
    size_t need = 0;
    geo_sc_bn_fixed_scratch_bytes(batch, channels, &need);
    if (scratch_bytes < need || ((uintptr_t)scratch & 255)) return fail(GEO_SC_ERR_WORKSPACE, "bn scratch holds %zu bytes, %zu needed", scratch_bytes, need);
    BnDims d = {batch, channels, height * width, bn_slices(batch, channels)};
    float *partial = (float *)scratch;
    if (training) {
        bn_reduce_kernel<0, true><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, xs, nullptr, partial);
        bn_mean_kernel<<<(channels + BN_THREADS - 1) / BN_THREADS, BN_THREADS, 0, s>>>(d, partial, save_mean);
        bn_reduce_kernel<1, true><<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, xs, save_mean, partial);
    }
    bn_fold_kernel<<<1, BN_THREADS, 0, s>>>(d, training, eps, momentum, partial, save_mean, save_invstd, weight, bias,
                                            running_mean, running_var, save_wq, save_bq, scale_out);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

static int bn_pool_backward(int batch, int channels, int height, int width, int training, XSource xs, const float *grad_out,
                            const float *weight, const float *save_mean, const float *save_invstd, const float *save_wq,
                            const float *save_bq, float *grad_x, float *grad_weight, float *grad_bias, void *scratch,
                            size_t scratch_bytes, cudaStream_t s) {
    if (!xs.p || !grad_out || !save_mean || !save_invstd || !save_wq || !save_bq || !grad_x || !scratch) return fail(GEO_SC_ERR_NULL, "a required pointer is NULL");
    int rc = bn_pool_check(batch, channels, height, width, xs.p, grad_out, grad_x);
    if (rc) return rc;
    size_t need = 0;
    geo_sc_bn_fixed_scratch_bytes(batch, channels, &need);
    if (scratch_bytes < need || ((uintptr_t)scratch & 255)) return fail(GEO_SC_ERR_WORKSPACE, "bn scratch holds %zu bytes, %zu needed", scratch_bytes, need);
    BnDims d = {batch, channels, height * width, bn_slices(batch, channels)};
    float *partial = (float *)scratch;
    float *sums = (float *)((char *)scratch + align_up((size_t)channels * 64 * 2 * sizeof(float), 256));
    const unsigned W = (unsigned)width, Ho = (unsigned)(height / 2);
    bn_pool_bwd_reduce_kernel<<<dim3(channels, d.S), BN_THREADS, 0, s>>>(d, W, Ho, xs, grad_out, save_mean, save_invstd, save_wq, save_bq, partial);
    bn_bwd_final_kernel<<<(channels + BN_THREADS - 1) / BN_THREADS, BN_THREADS, 0, s>>>(d, partial, sums, grad_weight, grad_bias);
    const unsigned rows = (unsigned)batch * channels * Ho;
    bn_pool_bwd_apply_kernel<<<bn_grid((long long)rows * (width / 4)), BN_THREADS, 0, s>>>(d, rows, W, Ho, training, xs, grad_out, save_mean,
                                                                                      save_invstd, weight, sums, save_wq, save_bq, grad_x);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int geo_sc_bn_pool_act_forward(int batch, int channels, int height, int width, int training, float eps, float momentum,
                               const float *x, const float *weight, const float *bias, float *running_mean,
                               float *running_var, float *out, float *save_mean, float *save_invstd, float *save_wq,
                               float *save_bq, float *scale_out, void *scratch, size_t scratch_bytes, void *stream) {
    if (!out) return fail(GEO_SC_ERR_NULL, "out is NULL");
    int rc = bn_pool_check(batch, channels, height, width, x, out, x);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const XSource xs = {x, 1.0f, 0};
    rc = bn_pool_stats(batch, channels, height, width, training, eps, momentum, xs, weight, bias, running_mean, running_var,
                       save_mean, save_invstd, save_wq, save_bq, scale_out, scratch, scratch_bytes, s);
    if (rc) return rc;
    const unsigned rows = (unsigned)batch * channels * (height / 2);
    bn_pool_apply_kernel<<<bn_grid((long long)rows * (width / 4)), BN_THREADS, 0, s>>>(rows, (unsigned)width, (unsigned)(height / 2),
                                                                                  (unsigned)channels, xs, save_wq, save_bq, out);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int geo_sc_bn_pool_act_backward(int batch, int channels, int height, int width, int training, const float *x,
                                const float *grad_out, const float *weight, const float *save_mean,
                                const float *save_invstd, const float *save_wq, const float *save_bq, float *grad_x,
                                float *grad_weight, float *grad_bias, void *scratch, size_t scratch_bytes, void *stream) {
    const XSource xs = {x, 1.0f, 0};
    return bn_pool_backward(batch, channels, height, width, training, xs, grad_out, weight, save_mean, save_invstd, save_wq,
                            save_bq, grad_x, grad_weight, grad_bias, scratch, scratch_bytes, (cudaStream_t)stream);
}

int geo_sc_epilogue_forward(const geo_sc_conv_desc *next_desc, int in_bit_length, int prec, int training, float eps,
                            float momentum, const int32_t *counts, const float *weight, const float *bias,
                            float *running_mean, float *running_var, float *act_out, float *save_mean, float *save_invstd,
                            float *save_wq, float *save_bq, float *scale_out, void *astream, size_t astream_bytes,
                            void *scratch, size_t scratch_bytes, void *stream) {
    Geometry g;
    int rc = make_geometry(next_desc, &g);
    if (rc) return rc;
    if (in_bit_length < 1 || (in_bit_length & (in_bit_length - 1))) return fail(GEO_SC_ERR_BIT_LENGTH, "bit length %d of the counts is not a power of two", in_bit_length);
    if (prec < 0 || prec > 23) return fail(GEO_SC_ERR_SHAPE, "prec %d outside 0..23", prec);
    if (g.generator != GEO_SC_GEN_LFSR) return fail(GEO_SC_ERR_UNSUPPORTED, "the fused epilogue generates LFSR streams only");
    if (!act_out || !astream) return fail(GEO_SC_ERR_NULL, "act_out or astream is NULL");
    const int height = 2 * g.H, width = 2 * g.W;
    if ((rc = bn_pool_check(g.B, g.C, height, width, counts, act_out, counts))) return rc;
    const size_t need = align_up(g.act_stream_words * 4, 256);
    if (astream_bytes < need || ((uintptr_t)astream & 255)) return fail(GEO_SC_ERR_WORKSPACE, "activation-stream buffer holds %zu bytes, %zu needed (256-byte aligned)", astream_bytes, need);
    cudaStream_t s = (cudaStream_t)stream;
    const XSource xs = {counts, 1.0f / (float)in_bit_length, 1};
    rc = bn_pool_stats(g.B, g.C, height, width, training, eps, momentum, xs, weight, bias, running_mean, running_var, save_mean,
                       save_invstd, save_wq, save_bq, scale_out, scratch, scratch_bytes, s);
    if (rc) return rc;
    return launch_epilogue_streams(g, xs, save_wq, save_bq, prec, act_out, (uint32_t *)astream, s);
}

int geo_sc_epilogue_backward(int batch, int channels, int height, int width, int in_bit_length, int training,
                             const int32_t *counts, const float *grad_out, const float *weight, const float *save_mean,
                             const float *save_invstd, const float *save_wq, const float *save_bq, float *grad_x,
                             float *grad_weight, float *grad_bias, void *scratch, size_t scratch_bytes, void *stream) {
    if (in_bit_length < 1 || (in_bit_length & (in_bit_length - 1))) return fail(GEO_SC_ERR_BIT_LENGTH, "bit length %d of the counts is not a power of two", in_bit_length);
    const XSource xs = {counts, 1.0f / (float)in_bit_length, 1};
    return bn_pool_backward(batch, channels, height, width, training, xs, grad_out, weight, save_mean, save_invstd, save_wq,
                            save_bq, grad_x, grad_weight, grad_bias, scratch, scratch_bytes, (cudaStream_t)stream);
}

}  // extern "C"

// ---- 2x2 average pooling followed by hardtanh(0, 1) ------------------------------------------------
// The activation between SC layers (network.py:168-184: x = tanh(pool(x)) with nn.AvgPool2d(2) and
// nn.Hardtanh(0, 1)) as one pass in each direction.  Backward: the gradient passes where the pooled
// value lies strictly inside (0, 1) and is spread evenly over the 2x2 window.
namespace geo {
namespace {

__global__ void __launch_bounds__(256) pool_act_fwd_kernel(int planes, int H, int W, const float *__restrict__ x,
                                                           float *__restrict__ y) {
    const int Ho = H / 2, Wo = W / 2;
    const long long total = (long long)planes * Ho * Wo;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int ox = (int)(i % Wo), oy = (int)((i / Wo) % Ho);
        const long long p = i / ((long long)Wo * Ho);
        const float *s = x + (p * H + 2 * oy) * W + 2 * ox;
        // same association as at::avg_pool2d: sum the window, then divide by its size
        const float v = (s[0] + s[1] + s[W] + s[W + 1]) / 4.0f;
        y[i] = fminf(fmaxf(v, 0.0f), 1.0f);
    }
}

__global__ void __launch_bounds__(256) pool_act_bwd_kernel(int planes, int H, int W, const float *__restrict__ x,
                                                           const float *__restrict__ gy, float *__restrict__ gx) {
    const long long total = (long long)planes * H * W;
    const int Ho = H / 2, Wo = W / 2;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int xx = (int)(i % W), yy = (int)((i / W) % H);
        const long long p = i / ((long long)W * H);
        const int oy = yy >> 1, ox = xx >> 1;
        float g = 0.0f;
        if (oy < Ho && ox < Wo) {   // a trailing odd row / column is not covered by any window
            const float *s = x + (p * H + 2 * oy) * W + 2 * ox;
            const float v = (s[0] + s[1] + s[W] + s[W + 1]) / 4.0f;
            if (v > 0.0f && v < 1.0f) g = gy[(p * Ho + oy) * Wo + ox] * 0.25f;
        }
        gx[i] = g;
    }
}

// Vector forms for even H and W % 4 == 0: a thread owns two horizontally adjacent windows, i.e. one
// float4 of each of the two input rows.  Rows of windows: r = plane * (H/2) + oy, input rows 2r, 2r+1.
__global__ void __launch_bounds__(256) pool_act_fwd_vec_kernel(unsigned rows, unsigned W, const float *__restrict__ x,
                                                               float *__restrict__ y) {
    const unsigned q = W >> 2, total = rows * q;
    for (unsigned i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
        const unsigned r = i / q, j = i % q;
        const float4 t = __ldg((const float4 *)(x + (size_t)(2 * r) * W) + j);
        const float4 b = __ldg((const float4 *)(x + (size_t)(2 * r + 1) * W) + j);
        const float v0 = (t.x + t.y + b.x + b.y) / 4.0f, v1 = (t.z + t.w + b.z + b.w) / 4.0f;
        ((float2 *)(y + (size_t)r * (W >> 1)))[j] = make_float2(fminf(fmaxf(v0, 0.0f), 1.0f), fminf(fmaxf(v1, 0.0f), 1.0f));
    }
}

__global__ void __launch_bounds__(256) pool_act_bwd_vec_kernel(unsigned rows, unsigned W, const float *__restrict__ x,
                                                               const float *__restrict__ gy, float *__restrict__ gx) {
    const unsigned q = W >> 2, total = rows * q;
    for (unsigned i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
        const unsigned r = i / q, j = i % q;
        const float4 t = __ldg((const float4 *)(x + (size_t)(2 * r) * W) + j);
        const float4 b = __ldg((const float4 *)(x + (size_t)(2 * r + 1) * W) + j);
        const float2 g = __ldg((const float2 *)(gy + (size_t)r * (W >> 1)) + j);
        const float v0 = (t.x + t.y + b.x + b.y) / 4.0f, v1 = (t.z + t.w + b.z + b.w) / 4.0f;
        const float g0 = v0 > 0.0f && v0 < 1.0f ? g.x * 0.25f : 0.0f;
        const float g1 = v1 > 0.0f && v1 < 1.0f ? g.y * 0.25f : 0.0f;
        const float4 o = make_float4(g0, g0, g1, g1);
        ((float4 *)(gx + (size_t)(2 * r) * W))[j] = o;
        ((float4 *)(gx + (size_t)(2 * r + 1) * W))[j] = o;
    }
}

// SC bit counts -> the layer's value counts / bit_length (exact: bit_length is a power of two)
template <bool VEC>
__global__ void __launch_bounds__(256) counts_to_float_kernel(const int32_t *__restrict__ c, float *__restrict__ y, size_t n,
                                                              float inv) {
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        if (VEC) {
            const int4 v = __ldg((const int4 *)c + i);
            ((float4 *)y)[i] = make_float4((float)v.x * inv, (float)v.y * inv, (float)v.z * inv, (float)v.w * inv);
        } else {
            y[i] = (float)c[i] * inv;
        }
    }
}

__global__ void __launch_bounds__(256) quantize_vec_kernel(const float4 *x, float4 *y, unsigned n4, float levels, float inv) {
    for (unsigned i = blockIdx.x * 256 + threadIdx.x; i < n4; i += gridDim.x * 256) {
        const float4 v = x[i];
        float4 r;
        const float lo = 1.0f - levels, hi = levels - 1.0f;
        r.x = v.x != v.x ? v.x : fminf(fmaxf(rintf(v.x * levels), lo), hi) * inv;
        r.y = v.y != v.y ? v.y : fminf(fmaxf(rintf(v.y * levels), lo), hi) * inv;
        r.z = v.z != v.z ? v.z : fminf(fmaxf(rintf(v.z * levels), lo), hi) * inv;
        r.w = v.w != v.w ? v.w : fminf(fmaxf(rintf(v.w * levels), lo), hi) * inv;
        y[i] = r;
    }
}

}  // namespace
}  // namespace geo

namespace geo {
namespace {
// y = clamp(rint(x * 2^prec), -(2^prec - 1), 2^prec - 1) / 2^prec; NaN stays NaN
__global__ void __launch_bounds__(256) quantize_kernel(const float *x, float *y, long long n, float levels, float inv) {
    const long long stride = (long long)gridDim.x * 256;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const float v = x[i];
        const float q = fminf(fmaxf(rintf(v * levels), 1.0f - levels), levels - 1.0f) * inv;
        y[i] = v != v ? v : q;
    }
}
}  // namespace
}  // namespace geo

extern "C" {

int geo_sc_quantize(const float *x, float *y, size_t n, int prec, void *stream) {
    if (prec < 0 || prec > 23) return fail(GEO_SC_ERR_SHAPE, "prec %d outside 0..23", prec);
    if (n == 0) return GEO_SC_OK;
    if (!x || !y) return fail(GEO_SC_ERR_NULL, "x or y is NULL");
    const float levels = (float)(1 << prec);
    if (n % 4 == 0 && n / 4 < (1ULL << 32) && (((uintptr_t)x | (uintptr_t)y) & 15) == 0)
        quantize_vec_kernel<<<bn_grid((long long)(n / 4)), 256, 0, (cudaStream_t)stream>>>((const float4 *)x, (float4 *)y,
                                                                                       (unsigned)(n / 4), levels, 1.0f / levels);
    else
        quantize_kernel<<<bn_grid((long long)n), 256, 0, (cudaStream_t)stream>>>(x, y, (long long)n, levels, 1.0f / levels);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int geo_sc_counts_to_float(const int32_t *counts, float *out, size_t n, int bit_length, void *stream) {
    if (bit_length < 1 || (bit_length & (bit_length - 1))) return fail(GEO_SC_ERR_BIT_LENGTH, "bit_length %d is not a power of two", bit_length);
    if (n == 0) return GEO_SC_OK;
    if (!counts || !out) return fail(GEO_SC_ERR_NULL, "counts or out is NULL");
    const float inv = 1.0f / (float)bit_length;
    const bool vec = n % 4 == 0 && n / 4 < (1ULL << 32) && (((uintptr_t)counts | (uintptr_t)out) & 15) == 0;
    if (vec) counts_to_float_kernel<true><<<bn_grid((long long)(n / 4)), 256, 0, (cudaStream_t)stream>>>(counts, out, n / 4, inv);
    else counts_to_float_kernel<false><<<bn_grid((long long)n), 256, 0, (cudaStream_t)stream>>>(counts, out, n, inv);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int geo_sc_pool_act_forward(int planes, int height, int width, const float *x, float *y, void *stream) {
    if (planes < 1 || height < 2 || width < 2) return fail(GEO_SC_ERR_SHAPE, "planes %d height %d width %d", planes, height, width);
    if (!x || !y) return fail(GEO_SC_ERR_NULL, "x or y is NULL");
    const long long total = (long long)planes * (height / 2) * (width / 2);
    if (height % 2 == 0 && width % 4 == 0 && (long long)planes * height * width < (1LL << 32) &&
        (((uintptr_t)x & 15) | ((uintptr_t)y & 7)) == 0)
        pool_act_fwd_vec_kernel<<<bn_grid(total / 2), 256, 0, (cudaStream_t)stream>>>((unsigned)(planes * (height / 2)),
                                                                                 (unsigned)width, x, y);
    else
        pool_act_fwd_kernel<<<bn_grid(total), 256, 0, (cudaStream_t)stream>>>(planes, height, width, x, y);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int geo_sc_pool_act_backward(int planes, int height, int width, const float *x, const float *grad_y, float *grad_x,
                             void *stream) {
    if (planes < 1 || height < 2 || width < 2) return fail(GEO_SC_ERR_SHAPE, "planes %d height %d width %d", planes, height, width);
    if (!x || !grad_y || !grad_x) return fail(GEO_SC_ERR_NULL, "x, grad_y or grad_x is NULL");
    const long long total = (long long)planes * height * width;
    if (height % 2 == 0 && width % 4 == 0 && total < (1LL << 32) &&
        ((((uintptr_t)x | (uintptr_t)grad_x) & 15) | ((uintptr_t)grad_y & 7)) == 0)
        pool_act_bwd_vec_kernel<<<bn_grid(total / 8), 256, 0, (cudaStream_t)stream>>>((unsigned)(planes * (height / 2)),
                                                                                 (unsigned)width, x, grad_y, grad_x);
    else
        pool_act_bwd_kernel<<<bn_grid(total), 256, 0, (cudaStream_t)stream>>>(planes, height, width, x, grad_y, grad_x);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

}  // extern "C"
