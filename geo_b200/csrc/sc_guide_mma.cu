// Tensor-core path of the float guide (see sc_guide.cu for the mathematics).
//
// Activations and weights that went through the layers' 7-bit quantisation (utils_class.py:32-33)
// are multiples of 1/128 below 1 in magnitude, hence exactly representable in bf16, and products of
// two such values are exact in fp32.  For such inputs the guide's convolutions can run on the
// tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulation) without changing the result
// beyond the order of the fp32 additions.  Whether the inputs qualify is decided on the device:
// the preparation kernels raise a flag when they meet a value that bf16 cannot hold, and the
// tensor-core kernels and the FFMA kernels of sc_guide.cu each return at once when the flag says
// the other family is in charge -- no host synchronisation, so the sequence can live in a CUDA graph.
//
// Tensor-core accumulation rounds toward zero; to keep that bias out of long sums, the MMA
// accumulators are flushed into ordinary fp32 registers (round-to-nearest adds) every few steps.
//
// Kernels: preparation (NHWC bf16 activations, weights per group), mma_forward_kernel
// (D = gout * exp(-y) as three bf16 terms), mma_wgrad_kernel + mma_wgrad_reduce_kernel, mma_dgrad_kernel,
// and mma_fused_wgrad_kernel, which does forward and weight gradient in one pass without storing D
// when no activation gradient is wanted and the groups are short (a network's first layer).
//
// Layouts: activations NHWC bf16 [B][Hp][Wp][Cp] (Cp = c_in rounded up to 8, zero filled), so that
// the members of a filter tap are 16-byte chunks; weights [group][2*c_out_padded][Kp] with the
// member index k' = tap * Cp + c contiguous.  Only the modes whose groups are whole filter taps
// over all channels use this path (1d_bin: the taps of one filter column; 2d_bin: one tap; full_or: all taps).
#include <cuda_bf16.h>

#include <algorithm>

#include "sc_common.h"
#include "sc_guide_mma.h"
#include "sc_guide_tc.h"

namespace geo {

namespace {

__device__ __forceinline__ void cp16z(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp4z(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cpa_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Filter coordinates of tap `tap` of group g: 1d_bin groups are filter columns (taps = rows), 2d_bin
// groups are single taps, full_or has one group with all taps.
__device__ __forceinline__ void tap_coords(const MmaDims &d, int g, int tap, int *ky, int *kx) {
    if (d.mode == GEO_SC_MODE_1D) { *ky = tap; *kx = g; }
    else if (d.mode == GEO_SC_MODE_2D) { *ky = g / d.K3; *kx = g % d.K3; }
    else { *ky = tap / d.K3; *kx = tap % d.K3; }
}

// Byte offset of 16-byte chunk `chunk` (0..3) of row `row` in a tile whose rows are 64 bytes
// (32 bf16); the XOR keeps the 8 rows of an ldmatrix 8x8 block in 8 different bank groups.
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
}

// ---- preparation --------------------------------------------------------------------------------
// NCHW fp32 -> padded NHWC bf16, raising *inexact if a value is not representable in bf16.
// One thread per pixel and group of 8 channels: eight plane reads (consecutive threads = consecutive
// channel groups, then consecutive x, so a warp reads whole 32-byte sectors) and one 16-byte store.
__global__ void __launch_bounds__(256) mma_prep_act_kernel(MmaDims d, const float *__restrict__ act,
                                                           __nv_bfloat16 *__restrict__ out, int *inexact) {
    const unsigned cg = (unsigned)d.Cp >> 3;
    const unsigned total = (unsigned)d.B * d.Hp * d.Wp * cg;    // < 2^31: the padded tensor is indexed by int
    const size_t hw = (size_t)d.H * d.W;
    bool bad = false;
    for (unsigned i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
        const unsigned c0 = (i % cg) * 8;
        unsigned r = i / cg;
        const int x = (int)(r % (unsigned)d.Wp); r /= (unsigned)d.Wp;
        const int y = (int)(r % (unsigned)d.Hp);
        const int b = (int)(r / (unsigned)d.Hp);
        const int yi = y - d.ph, xi = x - d.pw;
        const bool in = yi >= 0 && yi < d.H && xi >= 0 && xi < d.W;
        const float *src = act + ((size_t)b * d.C + c0) * hw + (in ? (size_t)yi * d.W + xi : 0);
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float v0 = in && (int)c0 + 2 * j < d.C ? __ldg(src + (size_t)(2 * j) * hw) : 0.0f;
            const float v1 = in && (int)c0 + 2 * j + 1 < d.C ? __ldg(src + (size_t)(2 * j + 1) * hw) : 0.0f;
            const __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
            pk[j] = *(const uint32_t *)&h;
            bad |= (__uint_as_float(pk[j] << 16) != v0) | (__uint_as_float(pk[j] & 0xffff0000u) != v1);
        }
        ((uint4 *)out)[i] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
    if (bad) atomicOr(inexact, 1);
}

// Wb[g][n2][Kp] bf16, n2 = pol * Opad + o, k' = tap * Cp + c (taps of group g in order), zero padded.
__global__ void __launch_bounds__(256) mma_prep_weight_kernel(MmaDims d, const float *__restrict__ w,
                                                              __nv_bfloat16 *__restrict__ wb, int *inexact) {
    const long long total = (long long)d.G * d.N2 * d.Kp;
    bool bad = false;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int kp = (int)(i % d.Kp);
        const int n2 = (int)((i / d.Kp) % d.N2), g = (int)(i / ((long long)d.Kp * d.N2));
        const int tap = kp / d.Cp, c = kp % d.Cp;
        const int pol = n2 / d.Opad, o = n2 % d.Opad;
        float v = 0.0f;
        if (tap < d.taps && c < d.C && o < d.O) {
            int ky, kx;
            tap_coords(d, g, tap, &ky, &kx);
            const float x = w[(((size_t)o * d.C + c) * d.K2 + ky) * d.K3 + kx];
            v = pol == 0 ? fminf(fmaxf(x, 0.0f), 100.0f) : -fminf(fmaxf(x, -100.0f), 0.0f);
        }
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        bad |= (__bfloat162float(h) != v);
        wb[i] = h;
    }
    if (bad) atomicOr(inexact, 1);
}

// ---- D = gout * exp(-conv) on the tensor cores -------------------------------------------------------
// CTA: 128 positions x 64 columns (polarity, channel), 4 warps of 32 positions each.
constexpr int MK = 32;        // members per stage (two k16 steps)
constexpr int MSTAGE = 4;
constexpr int MFLUSH = 8;     // k16 steps between flushes of the MMA accumulators

// Output: Dh[plane][g][m][n2] bf16, plane = term of the 3-way split of D = gout * exp(-y).
// MI = m16 tiles per warp: 2 (4 warps) or 1 (8 warps, half the accumulators per thread).
template <int MI>
__global__ void __launch_bounds__(256 / MI) mma_forward_kernel(MmaDims d, const __nv_bfloat16 *__restrict__ apad,
                                                               const __nv_bfloat16 *__restrict__ wb,
                                                               const float *__restrict__ gout,
                                                               __nv_bfloat16 *__restrict__ Dh, int vec_ok,
                                                               const int *inexact) {
    if (*inexact) return;   // the FFMA kernels handle inputs that bf16 cannot hold
    constexpr int NTH = 256 / MI, AROWS = 512 / NTH, BROWS = 256 / NTH, RSTEP = NTH / 4;
    constexpr int A_BYTES = 128 * 64, B_BYTES = 64 * 64, ST_BYTES = A_BYTES + B_BYTES;
    constexpr int GS = 132;   // floats per staged gout row (128 positions + 4: the epilogue's reads hit 32 banks)
    extern __shared__ __align__(128) unsigned char msm[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int m0 = blockIdx.x * 128, n0 = blockIdx.y * 64, g = blockIdx.z;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(msm);

    // gather assignment: thread t copies chunk (t & 3) of rows (t >> 2) + RSTEP * i
    const int gchunk = t & 3;
    long long rbase[AROWS];
#pragma unroll
    for (int i = 0; i < AROWS; i++) {
        int m = m0 + (t >> 2) + RSTEP * i;
        if (m >= d.M) m = d.M - 1;
        const int b = m / d.HoWo, rem = m % d.HoWo;
        const int oy = rem / d.Wo, ox = rem % d.Wo;
        rbase[i] = (((long long)b * d.Hp + oy) * d.Wp + ox) * d.Cp;
    }
    const int nchunks = d.linear ? 0 : d.Kp / MK;   // linear guide: y = 0, D = gout
    int ld = 0;
    auto issue = [&]() {
        if (ld < nchunks) {
            const uint32_t a_s = sbase + (uint32_t)(ld % MSTAGE) * ST_BYTES, b_s = a_s + A_BYTES;
            const int kp = ld * MK + gchunk * 8;     // first member of this thread's chunk
            const int tap = kp / d.Cp, c = kp % d.Cp;
            const bool kv = tap < d.taps;
            int ky, kx;
            tap_coords(d, g, tap, &ky, &kx);
            const long long koff = kv ? ((long long)ky * d.Wp + kx) * d.Cp + c : 0;
#pragma unroll
            for (int i = 0; i < AROWS; i++) {
                const int row = (t >> 2) + RSTEP * i;
                cp16z(a_s + swz(row, gchunk), apad + rbase[i] + koff, kv);
            }
            // weights: 64 rows (columns n) x 4 chunks
#pragma unroll
            for (int i = 0; i < BROWS; i++) {
                const int row = (t >> 2) + RSTEP * i;
                const __nv_bfloat16 *src = wb + ((size_t)g * d.N2 + n0 + row) * d.Kp + ld * MK + gchunk * 8;
                cp16z(b_s + swz(row, gchunk), src, true);
            }
            ld++;
        }
        cpa_commit();
    };
    // gout of the tile, [column][position], rides in the first cp.async group and is read by the epilogue
    const uint32_t g_s = sbase + MSTAGE * ST_BYTES;
    const float *g_p = (const float *)(msm + MSTAGE * ST_BYTES);
    if (vec_ok) {   // 16-byte copies of 4 positions (HoWo % 4 == 0, so they stay inside one image)
        const int m4 = m0 + (t & 31) * 4;
        const bool mv = m4 < d.M;
        const int mm = mv ? m4 : 0;
        const float *src = gout + (size_t)(mm / d.HoWo) * d.O * d.HoWo + mm % d.HoWo;
#pragma unroll
        for (int j = 0; j < 64 * 32 / NTH; j++) {
            const int col = (t >> 5) + (NTH / 32) * j;
            const int o = (n0 + col) % d.Opad;
            const bool v = mv && o < d.O;
            cp16z(g_s + (uint32_t)(col * GS + (t & 31) * 4) * 4, src + (size_t)(v ? o : 0) * d.HoWo, v);
        }
    } else {
        for (int i = t; i < 64 * 128; i += NTH) {
            const int col = i >> 7, m = m0 + (i & 127);
            const int o = (n0 + col) % d.Opad;
            const bool v = m < d.M && o < d.O;
            const int mm = v ? m : 0;
            cp4z(g_s + (uint32_t)(col * GS + (i & 127)) * 4,
                 gout + ((size_t)(mm / d.HoWo) * d.O + (v ? o : 0)) * d.HoWo + mm % d.HoWo, v);
        }
    }
#pragma unroll
    for (int s = 0; s < MSTAGE - 1; s++) issue();

    float acc[MI][8][4], sum[MI][8][4];
#pragma unroll
    for (int mi = 0; mi < MI; mi++)
#pragma unroll
        for (int ni = 0; ni < 8; ni++)
#pragma unroll
            for (int q = 0; q < 4; q++) { acc[mi][ni][q] = 0.f; sum[mi][ni][q] = 0.f; }

    int since_flush = 0;
    for (int s = 0; s < nchunks; s++) {
        cpa_wait<MSTAGE - 2>();
        __syncthreads();
        issue();
        const uint32_t a_s = sbase + (uint32_t)(s % MSTAGE) * ST_BYTES, b_s = a_s + A_BYTES;
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            uint32_t af[MI][4];
#pragma unroll
            for (int mi = 0; mi < MI; mi++) {
                // matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
                const int row = warp * (16 * MI) + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldsm_x4(af[mi], a_s + swz(row, ks * 2 + (lane >> 4)));
            }
#pragma unroll
            for (int np = 0; np < 4; np++) {
                // two n8 tiles per ldmatrix: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                uint32_t bf[4];
                const int row = np * 16 + (lane & 7) + (lane >> 4) * 8;
                ldsm_x4(bf, b_s + swz(row, ks * 2 + ((lane >> 3) & 1)));
#pragma unroll
                for (int mi = 0; mi < MI; mi++) {
                    mma_bf16(acc[mi][np * 2 + 0], af[mi], bf[0], bf[1]);
                    mma_bf16(acc[mi][np * 2 + 1], af[mi], bf[2], bf[3]);
                }
            }
        }
        since_flush += 2;
        if (since_flush >= MFLUSH || s == nchunks - 1) {
            since_flush = 0;
#pragma unroll
            for (int mi = 0; mi < MI; mi++)
#pragma unroll
                for (int ni = 0; ni < 8; ni++)
#pragma unroll
                    for (int q = 0; q < 4; q++) { sum[mi][ni][q] += acc[mi][ni][q]; acc[mi][ni][q] = 0.f; }
        }
    }
    cpa_wait<0>();
    __syncthreads();   // the staged gout tile is complete and visible even when the member loop was empty

    // epilogue: accumulator (mi, ni, q): row = lane/4 + 8*(q>>1), column = ni*8 + (lane%4)*2 + (q&1)
#pragma unroll
    for (int mi = 0; mi < MI; mi++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
            const int mrow = warp * (16 * MI) + mi * 16 + (lane >> 2) + hr * 8;
            const int m = m0 + mrow;
            if (m >= d.M) continue;
            const size_t plane = (size_t)d.G * d.M * d.N2;
            __nv_bfloat16 *row = Dh + ((size_t)g * d.M + m) * d.N2 + n0;
#pragma unroll
            for (int ni = 0; ni < 8; ni++) {
                const int col = ni * 8 + (lane & 3) * 2;
                const float v0 = g_p[col * GS + mrow] * expf(-sum[mi][ni][hr * 2 + 0]);
                const float v1 = g_p[(col + 1) * GS + mrow] * expf(-sum[mi][ni][hr * 2 + 1]);
                // three-term bf16 split of both values at once (cvt.rn.bf16x2.f32)
                __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                const uint32_t p0 = *(uint32_t *)&h;
                const float r0 = v0 - __uint_as_float(p0 << 16), r1 = v1 - __uint_as_float(p0 & 0xffff0000u);
                h = __floats2bfloat162_rn(r0, r1);
                const uint32_t p1 = *(uint32_t *)&h;
                const float s0 = r0 - __uint_as_float(p1 << 16), s1 = r1 - __uint_as_float(p1 & 0xffff0000u);
                h = __floats2bfloat162_rn(s0, s1);
                *(uint32_t *)(row + col) = p0;
                *(uint32_t *)(row + plane + col) = p1;
                *(__nv_bfloat162 *)(row + 2 * plane + col) = h;
            }
        }
}

// ---- weight gradient on the tensor cores ----------------------------------------------------------------
// partial[slice][g][k'][n2] = sum over the slice's positions of a[m, k'] * D[m, n2] (three split terms).
// CTA: 64 members x 64 columns, 2 warps of 32 members each; a stage holds 32 positions.
constexpr int WP = 32;        // positions per stage
constexpr int WSTG = 3;

__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// rows of 128 bytes (64 bf16), 8 chunks of 16 bytes
__device__ __forceinline__ uint32_t swz128(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__global__ void __launch_bounds__(64) mma_wgrad_kernel(MmaDims d, const __nv_bfloat16 *__restrict__ apad,
                                                       const __nv_bfloat16 *__restrict__ Dh, float *__restrict__ partial,
                                                       int slice_len, const int *inexact) {
    if (*inexact) return;
    constexpr int A_BYTES = WP * 128, D_BYTES = WP * 128, ST_BYTES = A_BYTES + 3 * D_BYTES;
    extern __shared__ __align__(128) unsigned char wsm2[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int ntiles = d.N2 / 64;
    const int g = blockIdx.z / ntiles, n0 = (blockIdx.z % ntiles) * 64;
    const int k0 = blockIdx.y * 64;
    const int mbeg = blockIdx.x * slice_len, mend = min(d.M, mbeg + slice_len);
    const int nst = (mend - mbeg + WP - 1) / WP;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(wsm2);
    const size_t plane = (size_t)d.G * d.M * d.N2;

    // this thread's chunk of members: tap and channel are fixed for the whole kernel
    const int gchunk = t & 7;
    const int kp = k0 + gchunk * 8;
    const int tap = kp / d.Cp, cch = kp % d.Cp;
    const bool kvalid = tap < d.taps;
    int ky, kx;
    tap_coords(d, g, tap, &ky, &kx);
    const long long koff = kvalid ? ((long long)ky * d.Wp + kx) * d.Cp + cch : 0;

    int ld = 0;
    auto issue = [&]() {
        if (ld < nst) {
            const uint32_t a_s = sbase + (uint32_t)(ld % WSTG) * ST_BYTES, d_s = a_s + A_BYTES;
            const int mc = mbeg + ld * WP;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = (t >> 3) + 8 * i;
                const int m = mc + row;
                const bool v = m < mend;
                const int mm = v ? m : mbeg;
                const int b = mm / d.HoWo, rem = mm % d.HoWo;
                const long long rb = (((long long)b * d.Hp + rem / d.Wo) * d.Wp + rem % d.Wo) * d.Cp;
                cp16z(a_s + swz128(row, gchunk), apad + rb + koff, v && kvalid);
                const __nv_bfloat16 *src = Dh + ((size_t)g * d.M + mm) * d.N2 + n0 + gchunk * 8;
#pragma unroll
                for (int p = 0; p < 3; p++) cp16z(d_s + p * D_BYTES + swz128(row, gchunk), src + p * plane, v);
            }
            ld++;
        }
        cpa_commit();
    };
#pragma unroll
    for (int s = 0; s < WSTG - 1; s++) issue();

    float acc[2][8][4], sum[2][8][4];
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int ni = 0; ni < 8; ni++)
#pragma unroll
            for (int q = 0; q < 4; q++) { acc[mi][ni][q] = 0.f; sum[mi][ni][q] = 0.f; }

    int since_flush = 0;
    for (int s = 0; s < nst; s++) {
        cpa_wait<WSTG - 2>();
        __syncthreads();
        issue();
        const uint32_t a_s = sbase + (uint32_t)(s % WSTG) * ST_BYTES, d_s = a_s + A_BYTES;
#pragma unroll
        for (int ps = 0; ps < 2; ps++) {   // two runs of 16 positions
            const int p0 = ps * 16;
            uint32_t af[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; mi++) {
                // transposed 8x8 blocks: (m 0-7, k' 0-7), (m 0-7, k' 8-15), (m 8-15, k' 0-7), (m 8-15, k' 8-15)
                const int row = p0 + (lane & 7) + (lane >> 4) * 8;
                const int chunk = warp * 4 + mi * 2 + ((lane >> 3) & 1);
                ldsm_x4_t(af[mi], a_s + swz128(row, chunk));
            }
#pragma unroll
            for (int p = 0; p < 3; p++) {
#pragma unroll
                for (int np = 0; np < 4; np++) {
                    // (m 0-7, n tile 2np), (m 8-15, n tile 2np), (m 0-7, n tile 2np+1), (m 8-15, n tile 2np+1)
                    uint32_t bf[4];
                    const int row = p0 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldsm_x4_t(bf, d_s + p * D_BYTES + swz128(row, np * 2 + (lane >> 4)));
#pragma unroll
                    for (int mi = 0; mi < 2; mi++) {
                        mma_bf16(acc[mi][np * 2 + 0], af[mi], bf[0], bf[1]);
                        mma_bf16(acc[mi][np * 2 + 1], af[mi], bf[2], bf[3]);
                    }
                }
            }
        }
        since_flush += 2;
        if (since_flush >= MFLUSH || s == nst - 1) {
            since_flush = 0;
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
#pragma unroll
                for (int ni = 0; ni < 8; ni++)
#pragma unroll
                    for (int q = 0; q < 4; q++) { sum[mi][ni][q] += acc[mi][ni][q]; acc[mi][ni][q] = 0.f; }
        }
    }
    cpa_wait<0>();
    float *dst = partial + ((size_t)blockIdx.x * d.G + g) * d.Kp * d.N2;
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
            const int k = k0 + warp * 32 + mi * 16 + (lane >> 2) + hr * 8;
            if (k >= d.Kp) continue;
#pragma unroll
            for (int ni = 0; ni < 8; ni++) {
                const int n2 = n0 + ni * 8 + (lane & 3) * 2;
                *(float2 *)(dst + (size_t)k * d.N2 + n2) = make_float2(sum[mi][ni][hr * 2], sum[mi][ni][hr * 2 + 1]);
            }
        }
}

// grad_w[o][c][ky][kx] = [w>=0] * sum_s partial[s][g][k'][o] + [w<=0] * sum_s partial[s][g][k'][Opad+o]
// A warp handles 32 consecutive outputs (lane = output, so that the reads are coalesced along o); SW
// warps share them, taking the slices s = sub, sub + SW, ..., and are combined in a fixed order.
template <int SW>
__global__ void __launch_bounds__(256) mma_wgrad_reduce_kernel(MmaDims d, int S, const float *__restrict__ partial,
                                                               const float *__restrict__ w, float *__restrict__ gw,
                                                               const int *inexact) {
    if (*inexact) return;
    __shared__ float red[2][8][32];
    constexpr int GROUPS = 8 / SW;                        // sets of 32 outputs per block and pass
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = warp % SW, grp = warp / SW;
    const long long total = (long long)d.G * d.taps * d.C * d.O;
    const long long per_pass = (long long)gridDim.x * GROUPS * 32;
    const size_t stride = (size_t)d.G * d.Kp * d.N2;
    for (long long pass0 = 0; pass0 < total; pass0 += per_pass) {
        const long long i = pass0 + ((long long)blockIdx.x * GROUPS + grp) * 32 + lane;
        float sp = 0.f, sn = 0.f;
        size_t wi = 0;
        if (i < total) {
            const int o = (int)(i % d.O);
            long long r = i / d.O;
            const int c = (int)(r % d.C); r /= d.C;
            const int tap = (int)(r % d.taps), g = (int)(r / d.taps);
            int ky, kx;
            tap_coords(d, g, tap, &ky, &kx);
            const float *p = partial + ((size_t)g * d.Kp + tap * d.Cp + c) * d.N2 + o;
#pragma unroll 4
            for (int s = sub; s < S; s += SW) {
                sp += p[s * stride];
                sn += p[s * stride + d.Opad];
            }
            wi = (((size_t)o * d.C + c) * d.K2 + ky) * d.K3 + kx;
        }
        if (SW > 1) {
            red[0][warp][lane] = sp;
            red[1][warp][lane] = sn;
            __syncthreads();
            if (sub == 0) {
#pragma unroll
                for (int k = 1; k < SW; k++) { sp += red[0][warp + k][lane]; sn += red[1][warp + k][lane]; }
            }
        }
        if (sub == 0 && i < total) {
            const float wv = w[wi];
            gw[wi] = (wv >= 0.f && wv <= 100.f ? sp : 0.f) + (wv <= 0.f && wv >= -100.f ? sn : 0.f);
        }
        if (SW > 1) __syncthreads();
    }
}

void launch_wgrad_reduce(const MmaDims &d, int S, const float *partial, const float *w, float *gw, const int *flag,
                         cudaStream_t s) {
    const long long sets = ((long long)d.G * d.taps * d.C * d.O + 31) / 32;
    const int sw = S <= 4 ? 1 : (S <= 16 ? 2 : (S <= 64 ? 4 : 8));
    const int blocks = (int)std::min<long long>((sets * sw + 7) / 8, sm_count() * 16);
    switch (sw) {
    case 1: mma_wgrad_reduce_kernel<1><<<blocks, 256, 0, s>>>(d, S, partial, w, gw, flag); break;
    case 2: mma_wgrad_reduce_kernel<2><<<blocks, 256, 0, s>>>(d, S, partial, w, gw, flag); break;
    case 4: mma_wgrad_reduce_kernel<4><<<blocks, 256, 0, s>>>(d, S, partial, w, gw, flag); break;
    default: mma_wgrad_reduce_kernel<8><<<blocks, 256, 0, s>>>(d, S, partial, w, gw, flag); break;
    }
}

// ---- forward and weight gradient in one kernel (no activation gradient wanted, short groups) ---------
// When a group has at most 64 padded members and only grad_weight is asked for (the first layer of a
// network), D never leaves the registers.  The forward product is computed transposed,
// y^T = Wb . a^T, with the columns n2 as MMA rows and the positions as MMA columns, so that the
// accumulator fragments of D^T = gout * exp(-y^T), split into three bf16 terms, are exactly the A
// fragments of gw^T[n2][k'] += D^T[n2][m] . a[m][k'].
// CTA: 8 warps on tiles of 128 positions x 64 columns; warp = 16 columns (warp & 3) x 64 positions
// (warp >> 2); a CTA walks a contiguous range of position tiles and writes two slices of partial sums.
constexpr int GSTRIDE = 136;   // floats per staged gout row: 128 positions + 8, so that 8 rows x 32 bytes tile the banks

template <int KS>
__device__ __forceinline__ uint32_t swz_rows(int row, int chunk) {
    return KS == 4 ? swz128(row, chunk) : swz(row, chunk);
}

template <int KS, int OROWS>
struct FusedCfg {
    static constexpr int STAGES = OROWS == 32 ? 3 : 2;
    static constexpr int A_BYTES = 128 * KS * 32, G_BYTES = OROWS * GSTRIDE * 4, ST_BYTES = A_BYTES + G_BYTES;
    static constexpr int W_BYTES = 64 * KS * 32;
    static constexpr size_t SMEM = (size_t)STAGES * ST_BYTES + W_BYTES;
};

// KS: k16 steps over the padded members of a group (Kp = 16 * KS, 2 or 4).  OROWS: distinct gout rows
// behind a 64-column tile: 32 when c_out <= 32 (both polarities of the same channels), else 64.
template <int KS, int OROWS>
__global__ void __launch_bounds__(256, 2) mma_fused_wgrad_kernel(MmaDims d, const __nv_bfloat16 *__restrict__ apad,
                                                                  const __nv_bfloat16 *__restrict__ wb,
                                                                  const float *__restrict__ gout,
                                                                  float *__restrict__ partial, int tiles_per_cta,
                                                                  int vec_ok, const int *inexact) {
    if (*inexact) return;
    using Cfg = FusedCfg<KS, OROWS>;
    constexpr int CPR = KS * 2;                             // 16-byte chunks per activation row
    constexpr int RPT = 128 * CPR / 256;                    // activation rows a thread gathers per stage
    constexpr int RSTEP = 256 / CPR;
    constexpr int FSTG = Cfg::STAGES;
    extern __shared__ __align__(128) unsigned char fsm[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int wn = warp & 3, wp = warp >> 2;
    const int gq = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.y * 64, g = blockIdx.z;
    const int ntiles = (d.M + 127) / 128;
    const int tbeg = min(ntiles, (int)blockIdx.x * tiles_per_cta), tend = min(ntiles, tbeg + tiles_per_cta);
    const int nt = tend - tbeg;
    const int kpairs = (d.taps * d.Cp + 15) / 16;           // k16 steps that hold real members
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(fsm);
    const uint32_t w_s = sbase + FSTG * Cfg::ST_BYTES;

    // activation gather: thread t copies chunk t % CPR (one tap, 8 channels) of rows t / CPR + RSTEP * i
    const int gchunk = t % CPR;
    const int kp = gchunk * 8;
    const int tap = kp / d.Cp, cch = kp % d.Cp;
    const bool kvalid = tap < d.taps;
    int ky, kx;
    tap_coords(d, g, tap, &ky, &kx);
    const long long koff = kvalid ? ((long long)ky * d.Wp + kx) * d.Cp + cch : 0;

    int ld = 0;
    auto issue = [&]() {
        if (ld < nt) {
            const uint32_t a_s = sbase + (uint32_t)(ld % FSTG) * Cfg::ST_BYTES, g_s = a_s + Cfg::A_BYTES;
            const int mc = (tbeg + ld) * 128;
#pragma unroll
            for (int i = 0; i < RPT; i++) {
                const int row = t / CPR + RSTEP * i;
                const int m = mc + row;
                const bool v = m < d.M;
                const int mm = v ? m : 0;
                const int b = mm / d.HoWo, rem = mm % d.HoWo;
                const long long rb = (((long long)b * d.Hp + rem / d.Wo) * d.Wp + rem % d.Wo) * d.Cp;
                cp16z(a_s + swz_rows<KS>(row, gchunk), apad + rb + koff, v && kvalid);
            }
            // gout: rows = channels behind the column tile, 4 positions (t & 31) per copy
            const int m4 = mc + (t & 31) * 4;
            if (vec_ok) {
                const bool v = m4 < d.M;
                const int mm = v ? m4 : 0;
                const int b = mm / d.HoWo, rem = mm % d.HoWo;
#pragma unroll
                for (int i = 0; i < OROWS / 8; i++) {
                    const int r = (t >> 5) + 8 * i;
                    const int o = (n0 + r) % d.Opad;
                    const bool ov = v && o < d.O;
                    cp16z(g_s + (uint32_t)(r * GSTRIDE + (t & 31) * 4) * 4,
                          gout + ((size_t)b * d.O + (ov ? o : 0)) * d.HoWo + rem, ov);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int m = m4 + e;
                    const bool v = m < d.M;
                    const int mm = v ? m : 0;
                    const int b = mm / d.HoWo, rem = mm % d.HoWo;
#pragma unroll
                    for (int i = 0; i < OROWS / 8; i++) {
                        const int r = (t >> 5) + 8 * i;
                        const int o = (n0 + r) % d.Opad;
                        const bool ov = v && o < d.O;
                        cp4z(g_s + (uint32_t)(r * GSTRIDE + (t & 31) * 4 + e) * 4,
                             gout + ((size_t)b * d.O + (ov ? o : 0)) * d.HoWo + rem, ov);
                    }
                }
            }
            ld++;
        }
        cpa_commit();
    };
    // the group's weights (64 columns x Kp members) travel with the first stage
#pragma unroll
    for (int i = 0; i < 64 * CPR / 256; i++) {
        const int row = t / CPR + RSTEP * i;
        cp16z(w_s + swz_rows<KS>(row, gchunk), wb + ((size_t)g * d.N2 + n0 + row) * d.Kp + gchunk * 8, true);
    }
#pragma unroll
    for (int s = 0; s < FSTG - 1; s++) issue();
    cpa_wait<FSTG - 2>();
    __syncthreads();
    uint32_t wf[KS][4];   // A fragments of the forward product: this warp's 16 columns, all members
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const int row = wn * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldsm_x4(wf[ks], w_s + swz_rows<KS>(row, ks * 2 + (lane >> 4)));
    }

    float gacc[2 * KS][4], gsum[2 * KS][4];
#pragma unroll
    for (int j = 0; j < 2 * KS; j++)
#pragma unroll
        for (int q = 0; q < 4; q++) { gacc[j][q] = 0.f; gsum[j][q] = 0.f; }

    // staged gout rows of this thread's two columns (n2 = n0 + wn*16 + gq and + 8)
    uint32_t grow[2];
#pragma unroll
    for (int hr = 0; hr < 2; hr++) grow[hr] = (uint32_t)(((wn * 16 + gq + hr * 8) % OROWS) * GSTRIDE + wp * 64 + 2 * tq) * 4;

    for (int s = 0; s < nt; s++) {
        cpa_wait<FSTG - 2>();
        __syncthreads();
        issue();
        const uint32_t a_s = sbase + (uint32_t)(s % FSTG) * Cfg::ST_BYTES;
        const unsigned char *g_p = fsm + (size_t)(s % FSTG) * Cfg::ST_BYTES + Cfg::A_BYTES;
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {   // 16 positions = one k16 step of the weight-gradient product
            // forward: acc[jj] = y^T for columns (gq, gq+8) and positions wp*64 + kk*16 + jj*8 + 2*tq, +1
            float acc[2][4];
#pragma unroll
            for (int jj = 0; jj < 2; jj++)
#pragma unroll
                for (int q = 0; q < 4; q++) acc[jj][q] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                if (ks < kpairs && !d.linear) {
                    uint32_t bf[4];
                    const int row = wp * 64 + kk * 16 + (lane & 7) + (lane >> 4) * 8;
                    ldsm_x4(bf, a_s + swz_rows<KS>(row, ks * 2 + ((lane >> 3) & 1)));
                    mma_bf16(acc[0], wf[ks], bf[0], bf[1]);
                    mma_bf16(acc[1], wf[ks], bf[2], bf[3]);
                }
            }
            uint32_t af[3][4];
#pragma unroll
            for (int jj = 0; jj < 2; jj++)
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {
                    const float2 go = *(const float2 *)(g_p + grow[hr] + (kk * 16 + jj * 8) * 4);
                    const float v0 = go.x * expf(-acc[jj][hr * 2 + 0]);
                    const float v1 = go.y * expf(-acc[jj][hr * 2 + 1]);
                    // three-term bf16 split of both values at once
                    __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                    const uint32_t p0 = *(uint32_t *)&h;
                    const float r0 = v0 - __uint_as_float(p0 << 16), r1 = v1 - __uint_as_float(p0 & 0xffff0000u);
                    h = __floats2bfloat162_rn(r0, r1);
                    const uint32_t p1 = *(uint32_t *)&h;
                    const float s0 = r0 - __uint_as_float(p1 << 16), s1 = r1 - __uint_as_float(p1 & 0xffff0000u);
                    h = __floats2bfloat162_rn(s0, s1);
                    const uint32_t p2 = *(uint32_t *)&h;
                    af[0][jj * 2 + hr] = p0; af[1][jj * 2 + hr] = p1; af[2][jj * 2 + hr] = p2;
                }
#pragma unroll
            for (int np = 0; np < KS; np++) {
                if (np < kpairs) {
                    // transposed blocks: (m 0-7, k' tile 2np), (m 8-15, k' tile 2np), (m 0-7, tile 2np+1), (m 8-15, tile 2np+1)
                    uint32_t bt[4];
                    const int row = wp * 64 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldsm_x4_t(bt, a_s + swz_rows<KS>(row, np * 2 + (lane >> 4)));
#pragma unroll
                    for (int p = 0; p < 3; p++) {
                        mma_bf16(gacc[np * 2 + 0], af[p], bt[0], bt[1]);
                        mma_bf16(gacc[np * 2 + 1], af[p], bt[2], bt[3]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 2 * KS; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) { gsum[j][q] += gacc[j][q]; gacc[j][q] = 0.f; }
    }
    cpa_wait<0>();
    // gsum[j][q]: column n2 = n0 + wn*16 + gq + 8*(q>>1), member k' = j*8 + 2*tq + (q&1)
    float *dst = partial + ((size_t)(blockIdx.x * 2 + wp) * d.G + g) * d.Kp * d.N2;
#pragma unroll
    for (int j = 0; j < 2 * KS; j++)
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int n2 = n0 + wn * 16 + gq + 8 * (q >> 1), k = j * 8 + 2 * tq + (q & 1);
            dst[(size_t)k * d.N2 + n2] = gsum[j][q];
        }
}

// ---- activation gradient on the tensor cores ---------------------------------------------------------------
// grad_a[pix][c] = sum over taps and columns n2 of D[g(tap)][pos(pix, tap)][n2] * Wd[c][tap*N2 + n2]
// Wd[c][r] bf16: +w+ for the positive columns, -(w-) for the negative ones, zero padded to Cn channels.
__global__ void __launch_bounds__(256) mma_prep_wd_kernel(MmaDims d, int Cn, const float *__restrict__ w,
                                                          __nv_bfloat16 *__restrict__ wd) {
    const int R = d.K2 * d.K3 * d.N2;
    const long long total = (long long)Cn * R;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int r = (int)(i % R), c = (int)(i / R);
        const int n2 = r % d.N2, tap = r / d.N2, ky = tap / d.K3, kx = tap % d.K3;
        const int pol = n2 / d.Opad, o = n2 % d.Opad;
        float v = 0.0f;
        if (c < d.C && o < d.O) {
            const float x = w[(((size_t)o * d.C + c) * d.K2 + ky) * d.K3 + kx];
            v = pol == 0 ? fminf(fmaxf(x, 0.0f), 100.0f) : fminf(fmaxf(x, -100.0f), 0.0f);
        }
        wd[i] = __float2bfloat16_rn(v);
    }
}


// NWC warps along the channels: a CTA of 4 * NWC warps covers 128 pixels x 32 * NWC channels, so that one
// staged D tile serves NWC times as many channels.
// DSTG: stages of the cp.async ring (2 lets four CTAs share an SM; 3 when there are too few CTAs for that).
template <int NWC, int DSTG>
__global__ void __launch_bounds__(128 * NWC) mma_dgrad_kernel(MmaDims d, int Cn, const __nv_bfloat16 *__restrict__ Dh,
                                                              const __nv_bfloat16 *__restrict__ wd,
                                                              float *__restrict__ ga, const int *inexact) {
    if (*inexact) return;
    constexpr int NTH = 128 * NWC;
    constexpr int A_BYTES = 128 * 64, B_BYTES = 32 * NWC * 64, ST_BYTES = 3 * A_BYTES + B_BYTES;
    constexpr int AROWS = 512 / NTH, RSTEP = NTH / 4;   // D rows a thread gathers per plane and stage
    extern __shared__ __align__(128) unsigned char dsm2[];
    const int t = threadIdx.x, lane = t & 31, warp = (t >> 5) & 3, wc = t >> 7;
    const int p0 = blockIdx.x * 128, c0 = blockIdx.y * (32 * NWC) + wc * 32;
    const int HW = d.H * d.W, Min = d.B * HW;
    const int R = d.K2 * d.K3 * d.N2;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dsm2);
    const size_t plane = (size_t)d.G * d.M * d.N2;

    const int gchunk = t & 3;
    int pb[AROWS], py[AROWS], px[AROWS];
#pragma unroll
    for (int i = 0; i < AROWS; i++) {
        int pix = p0 + (t >> 2) + RSTEP * i;
        const bool v = pix < Min;
        if (!v) pix = 0;
        const int b = pix / HW, rem = pix % HW;
        pb[i] = v ? b : -1;
        py[i] = rem / d.W + d.ph;
        px[i] = rem % d.W + d.pw;
    }
    const int spt = d.N2 / 32;             // stages per tap
    const int nst = d.K2 * d.K3 * spt;
    int ld = 0;
    auto issue = [&]() {
        if (ld < nst) {
            const uint32_t a_s = sbase + (uint32_t)(ld % DSTG) * ST_BYTES, b_s = a_s + 3 * A_BYTES;
            const int tap = ld / spt, n2 = (ld % spt) * 32 + gchunk * 8;
            const int ky = tap / d.K3, kx = tap % d.K3;
            const int g = d.mode == GEO_SC_MODE_1D ? kx : (d.mode == GEO_SC_MODE_2D ? tap : 0);
#pragma unroll
            for (int i = 0; i < AROWS; i++) {
                const int row = (t >> 2) + RSTEP * i;
                const int oy = py[i] - ky, ox = px[i] - kx;
                const bool v = pb[i] >= 0 && oy >= 0 && oy < d.Ho && ox >= 0 && ox < d.Wo;
                const size_t m = v ? (size_t)pb[i] * d.HoWo + oy * d.Wo + ox : 0;
                const __nv_bfloat16 *src = Dh + ((size_t)g * d.M + m) * d.N2 + n2;
#pragma unroll
                for (int p = 0; p < 3; p++) cp16z(a_s + p * A_BYTES + swz(row, gchunk), src + p * plane, v);
            }
            {   // weights: 32 * NWC rows (channels) x 4 chunks, one copy per thread
                const int row = t >> 2;
                const __nv_bfloat16 *src = wd + (size_t)(blockIdx.y * (32 * NWC) + row) * R + (size_t)ld * 32 + gchunk * 8;
                cp16z(b_s + swz(row, gchunk), src, true);
            }
            ld++;
        }
        cpa_commit();
    };
#pragma unroll
    for (int s = 0; s < DSTG - 1; s++) issue();

    float acc[2][4][4], sum[2][4][4];
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int ni = 0; ni < 4; ni++)
#pragma unroll
            for (int q = 0; q < 4; q++) { acc[mi][ni][q] = 0.f; sum[mi][ni][q] = 0.f; }

    int since_flush = 0;
    for (int s = 0; s < nst; s++) {
        cpa_wait<DSTG - 2>();
        __syncthreads();
        issue();
        const uint32_t a_s = sbase + (uint32_t)(s % DSTG) * ST_BYTES, b_s = a_s + 3 * A_BYTES;
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            uint32_t bf[2][4];
#pragma unroll
            for (int np = 0; np < 2; np++) {
                const int row = wc * 32 + np * 16 + (lane & 7) + (lane >> 4) * 8;
                ldsm_x4(bf[np], b_s + swz(row, ks * 2 + ((lane >> 3) & 1)));
            }
#pragma unroll
            for (int p = 0; p < 3; p++)
#pragma unroll
                for (int mi = 0; mi < 2; mi++) {
                    uint32_t af[4];
                    const int row = warp * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    ldsm_x4(af, a_s + p * A_BYTES + swz(row, ks * 2 + (lane >> 4)));
#pragma unroll
                    for (int np = 0; np < 2; np++) {
                        mma_bf16(acc[mi][np * 2 + 0], af, bf[np][0], bf[np][1]);
                        mma_bf16(acc[mi][np * 2 + 1], af, bf[np][2], bf[np][3]);
                    }
                }
        }
        since_flush += 2;
        if (since_flush >= MFLUSH || s == nst - 1) {
            since_flush = 0;
#pragma unroll
            for (int mi = 0; mi < 2; mi++)
#pragma unroll
                for (int ni = 0; ni < 4; ni++)
#pragma unroll
                    for (int q = 0; q < 4; q++) { sum[mi][ni][q] += acc[mi][ni][q]; acc[mi][ni][q] = 0.f; }
        }
    }
    cpa_wait<0>();
#pragma unroll
    for (int mi = 0; mi < 2; mi++)
#pragma unroll
        for (int hr = 0; hr < 2; hr++) {
            const int pix = p0 + warp * 32 + mi * 16 + (lane >> 2) + hr * 8;
            if (pix >= Min) continue;
            const int b = pix / HW, rem = pix % HW;
#pragma unroll
            for (int ni = 0; ni < 4; ni++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int c = c0 + ni * 8 + (lane & 3) * 2 + e;
                    if (c < d.C) ga[((size_t)b * d.C + c) * HW + rem] = sum[mi][ni][hr * 2 + e];
                }
        }
}

int grid1(long long total) {
    long long b = (total + 255) / 256;
    return (int)(b < sm_count() * 16 ? (b > 0 ? b : 1) : sm_count() * 16);
}

}  // namespace

bool mma_eligible(const Geometry &g) {
    // groups made of whole filter taps over all channels
    return g.mode == GEO_SC_MODE_1D || g.mode == GEO_SC_MODE_FULL_OR || g.mode == GEO_SC_MODE_2D;
}

MmaDims mma_dims(const Geometry &g) {
    MmaDims d;
    d.B = g.B; d.C = g.C; d.H = g.H; d.W = g.W; d.ph = g.pad_h; d.pw = g.pad_w; d.Hp = g.Hp; d.Wp = g.Wp;
    d.O = g.O; d.K2 = g.K2; d.K3 = g.K3; d.Ho = g.Ho; d.Wo = g.Wo; d.HoWo = g.Ho * g.Wo;
    // the guide's own channel padding: column tiles are 64 wide = 32 channels x 2 polarities
    d.mode = g.mode; d.G = g.G; d.Opad = (g.O + 31) / 32 * 32; d.N2 = 2 * d.Opad; d.M = (int)g.M;
    d.Cp = (g.C + 7) / 8 * 8;
    d.taps = g.mode == GEO_SC_MODE_1D ? g.K2 : (g.mode == GEO_SC_MODE_2D ? 1 : g.K2 * g.K3);
    d.Kp = (d.taps * d.Cp + MK - 1) / MK * MK;
    d.linear = g.guide_linear;
    return d;
}

namespace {

struct MmaPlan {
    size_t flag_bytes, apad_bytes, wb_bytes, dh_bytes, wd_bytes, partial_bytes;
    int S, slice_len, Cn;
    int fused_ctas, fused_tiles;   // one-kernel forward + weight gradient: CTAs per (group, column tile), tiles per CTA
    size_t total() const { return flag_bytes + apad_bytes + wb_bytes + dh_bytes + wd_bytes + partial_bytes; }
};

MmaPlan mma_plan(const MmaDims &d) {
    MmaPlan p;
    p.flag_bytes = 256;
    p.apad_bytes = align_up((size_t)d.B * d.Hp * d.Wp * d.Cp * 2, 256);
    p.wb_bytes = align_up((size_t)d.G * d.N2 * d.Kp * 2, 256);
    p.dh_bytes = align_up((size_t)3 * d.G * d.M * d.N2 * 2, 256);
    // channel rows of Wd: zero padded to the tile of the activation-gradient kernel (128 for the tcgen05 kernel of wide layers)
    p.Cn = d.C >= 128 ? (d.C + 127) / 128 * 128 : (d.C + 31) / 32 * 32;
    p.wd_bytes = align_up((size_t)p.Cn * d.K2 * d.K3 * d.N2 * 2, 256);
    const long long tiles = (long long)d.G * ((d.Kp + 63) / 64) * (d.N2 / 64);
    long long S = (long long)sm_count() * 8 / tiles;   // at most two full waves of four resident CTAs per SM, no third
    // slices are whole stages of the weight-gradient kernel: 32 positions (mma.sync), 64 for wide layers (tcgen05)
    const int wpos = d.Cp % 128 == 0 && d.N2 % 128 == 0 ? 64 : WP;
    const long long maxS = (d.M + wpos - 1) / wpos;
    if (S > maxS) S = maxS;
    if (S < 1) S = 1;
    long long len = (d.M + S - 1) / S;
    len = (len + wpos - 1) / wpos * wpos;
    p.slice_len = (int)len;
    p.S = (int)((d.M + len - 1) / len);
    // the fused kernel: two resident CTAs per SM, each writing two slices
    const long long mt = (d.M + 127) / 128;
    long long X = (long long)sm_count() * 2 / ((long long)d.G * (d.N2 / 64));
    if (X < 1) X = 1;
    if (X > mt) X = mt;
    p.fused_tiles = (int)((mt + X - 1) / X);
    p.fused_ctas = (int)((mt + p.fused_tiles - 1) / p.fused_tiles);
    const int smax = d.Kp <= 64 && 2 * p.fused_ctas > p.S ? 2 * p.fused_ctas : p.S;
    p.partial_bytes = align_up((size_t)smax * d.G * d.Kp * d.N2 * 4, 256);
    return p;
}

template <typename Kern>
int opt_in_smem(Kern kern, size_t bytes, bool *done) {
    static std::mutex m;   // host threads may launch concurrently: the flags are read and written under it
    std::lock_guard<std::mutex> lock(m);
    int dev = 0;
    GEO_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !done[dev]) {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        if (dev >= 0 && dev < 64) done[dev] = true;
    }
    return GEO_SC_OK;
}

}  // namespace

size_t mma_scratch_bytes(const Geometry &g) {
    if (!mma_eligible(g)) return 0;
    return mma_plan(mma_dims(g)).total();
}

template <int KS, int OROWS>
int launch_fused(const MmaDims &d, dim3 grid, const __nv_bfloat16 *apad, const __nv_bfloat16 *wb, const float *gout,
                 float *partial, int tiles, int vec_ok, const int *flag, cudaStream_t s) {
    static bool done[64] = {};
    int rc = opt_in_smem(mma_fused_wgrad_kernel<KS, OROWS>, FusedCfg<KS, OROWS>::SMEM, done);
    if (rc) return rc;
    mma_fused_wgrad_kernel<KS, OROWS><<<grid, 256, FusedCfg<KS, OROWS>::SMEM, s>>>(d, apad, wb, gout, partial, tiles,
                                                                                  vec_ok, flag);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

template <int NWC, int DSTG>
int launch_dgrad_staged(const MmaDims &d, int Cn, const __nv_bfloat16 *Dh, const __nv_bfloat16 *wd, float *grad_act,
                        const int *flag, cudaStream_t s) {
    constexpr size_t smem = (size_t)DSTG * (3 * 128 * 64 + 32 * NWC * 64);
    static bool done[64] = {};
    int rc = opt_in_smem(mma_dgrad_kernel<NWC, DSTG>, smem, done);
    if (rc) return rc;
    dim3 grid((d.B * d.H * d.W + 127) / 128, Cn / (32 * NWC));
    mma_dgrad_kernel<NWC, DSTG><<<grid, 128 * NWC, smem, s>>>(d, Cn, Dh, wd, grad_act, flag);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

template <int NWC>
int launch_dgrad(const MmaDims &d, int Cn, const __nv_bfloat16 *Dh, const __nv_bfloat16 *wd, float *grad_act,
                 const int *flag, cudaStream_t s) {
    const long long ctas = (((long long)d.B * d.H * d.W + 127) / 128) * (Cn / (32 * NWC));
    return ctas >= sm_count() * 2 ? launch_dgrad_staged<NWC, 2>(d, Cn, Dh, wd, grad_act, flag, s)
                           : launch_dgrad_staged<NWC, 3>(d, Cn, Dh, wd, grad_act, flag, s);
}

// Whole backward pass on the tensor cores; every kernel returns at once if an input turned out
// not to be bf16-exact (*flag_out != 0 after the preparation kernels), in which case the caller's
// FFMA kernels, which test the same flag the other way round, do the work.
int launch_mma_backward(const Geometry &g, const float *act, const float *weight, const float *gout, float *grad_act,
                        float *grad_weight, void *scratch, int **flag_out, cudaStream_t s) {
    const MmaDims d = mma_dims(g);
    const MmaPlan p = mma_plan(d);
    char *base = (char *)scratch;
    int *flag = (int *)base;
    __nv_bfloat16 *apad = (__nv_bfloat16 *)(base + p.flag_bytes);
    __nv_bfloat16 *wb = (__nv_bfloat16 *)(base + p.flag_bytes + p.apad_bytes);
    __nv_bfloat16 *Dh = (__nv_bfloat16 *)(base + p.flag_bytes + p.apad_bytes + p.wb_bytes);
    __nv_bfloat16 *wd = (__nv_bfloat16 *)(base + p.flag_bytes + p.apad_bytes + p.wb_bytes + p.dh_bytes);
    float *partial = (float *)(base + p.flag_bytes + p.apad_bytes + p.wb_bytes + p.dh_bytes + p.wd_bytes);
    *flag_out = flag;
    GEO_CUDA_CHECK(cudaMemsetAsync(flag, 0, sizeof(int), s));
    mma_prep_act_kernel<<<grid1((long long)d.B * d.Hp * d.Wp * (d.Cp / 8)), 256, 0, s>>>(d, act, apad, flag);
    mma_prep_weight_kernel<<<grid1((long long)d.G * d.N2 * d.Kp), 256, 0, s>>>(d, weight, wb, flag);
    GEO_CUDA_CHECK(cudaGetLastError());
    if (grad_weight && !grad_act && d.Kp <= 64) {
        // forward and weight gradient in one kernel, D stays in registers
        const int vec_ok = d.HoWo % 4 == 0 && ((uintptr_t)gout & 15) == 0;   // 16-byte copies of 4 positions
        dim3 grid(p.fused_ctas, d.N2 / 64, d.G);
        int rc;
        if (d.Kp == 64) {
            rc = d.Opad == 32 ? launch_fused<4, 32>(d, grid, apad, wb, gout, partial, p.fused_tiles, vec_ok, flag, s)
                              : launch_fused<4, 64>(d, grid, apad, wb, gout, partial, p.fused_tiles, vec_ok, flag, s);
        } else {
            rc = d.Opad == 32 ? launch_fused<2, 32>(d, grid, apad, wb, gout, partial, p.fused_tiles, vec_ok, flag, s)
                              : launch_fused<2, 64>(d, grid, apad, wb, gout, partial, p.fused_tiles, vec_ok, flag, s);
        }
        if (rc) return rc;
        launch_wgrad_reduce(d, 2 * p.fused_ctas, partial, weight, grad_weight, flag, s);
        GEO_CUDA_CHECK(cudaGetLastError());
        return GEO_SC_OK;
    }
    TcTile ftile;
    if (tc_forward_plan(d, &ftile)) {   // wide layers: tcgen05.mma, tensor-memory accumulators, TMA tiles (sc_guide_tc.cu)
        int rc = launch_tc_forward(d, apad, wb, gout, Dh, flag, s);
        if (rc) return rc;
    } else {
        constexpr size_t smem = (size_t)MSTAGE * (128 * 64 + 64 * 64) + 64 * 132 * 4;
        static bool done[64] = {};
        int rc = opt_in_smem(mma_forward_kernel<1>, smem, done);
        if (rc) return rc;
        const int vec_ok = d.HoWo % 4 == 0 && ((uintptr_t)gout & 15) == 0;
        dim3 grid((d.M + 127) / 128, d.N2 / 64, d.G);
        mma_forward_kernel<1><<<grid, 256, smem, s>>>(d, apad, wb, gout, Dh, vec_ok, flag);
        GEO_CUDA_CHECK(cudaGetLastError());
    }
    TcTile wtile;
    if (grad_weight && tc_wgrad_plan(d, p.slice_len, &wtile)) {   // wide layers: tcgen05 (sc_guide_tc.cu)
        int rc = launch_tc_wgrad(d, apad, Dh, partial, p.S, p.slice_len, flag, s);
        if (rc) return rc;
        launch_wgrad_reduce(d, p.S, partial, weight, grad_weight, flag, s);
        GEO_CUDA_CHECK(cudaGetLastError());
    } else if (grad_weight) {
        constexpr size_t smem = (size_t)WSTG * (WP * 128 * 4);
        static bool done[64] = {};
        int rc = opt_in_smem(mma_wgrad_kernel, smem, done);
        if (rc) return rc;
        dim3 grid(p.S, (d.Kp + 63) / 64, d.G * (d.N2 / 64));
        mma_wgrad_kernel<<<grid, 64, smem, s>>>(d, apad, Dh, partial, p.slice_len, flag);
        launch_wgrad_reduce(d, p.S, partial, weight, grad_weight, flag, s);
        GEO_CUDA_CHECK(cudaGetLastError());
    }
    if (grad_act) {
        mma_prep_wd_kernel<<<grid1((long long)p.Cn * d.K2 * d.K3 * d.N2), 256, 0, s>>>(d, p.Cn, weight, wd);
        // widest channel tile that still leaves four CTAs of work per SM
        const long long ptiles = ((long long)d.B * d.H * d.W + 127) / 128;
        int rc;
        TcTile tile;
        // wide layers: tcgen05.mma with tensor-memory accumulators and TMA tiles (sc_guide_tc.cu)
        if (tc_dgrad_plan(d, p.Cn, &tile)) rc = launch_tc_dgrad(d, p.Cn, Dh, wd, grad_act, flag, s);
        else if (p.Cn % 128 == 0 && ptiles * (p.Cn / 128) >= sm_count() * 4) rc = launch_dgrad<4>(d, p.Cn, Dh, wd, grad_act, flag, s);
        else if (p.Cn % 64 == 0 && ptiles * (p.Cn / 64) >= sm_count() * 4) rc = launch_dgrad<2>(d, p.Cn, Dh, wd, grad_act, flag, s);
        else rc = launch_dgrad<1>(d, p.Cn, Dh, wd, grad_act, flag, s);
        if (rc) return rc;
    }
    return GEO_SC_OK;
}

}  // namespace geo
