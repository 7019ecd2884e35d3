// Activation gradient of the float guide on the fifth-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory, operand tiles brought in by TMA), for wide layers.
//
//   grad_a[pix][c] = sum over filter taps, columns n2 and the three bf16 terms of D of
//                    D_term[g(tap)][pos(pix, tap)][n2] * Wd[c][tap * N2 + n2]
//
// (sc_guide_mma.cu has the mathematics and the layouts: D as three bf16 terms [term][group][position][N2],
// Wd [channel][tap * N2 + n2] bf16.)  A CTA owns 128 input pixels -- a box of whole rows of one image, or several
// whole small images -- and 128 input channels.  Per (tap, 64 columns) one pipeline stage: three 128 x 64 tiles
// of D (one per term), fetched by one 5-d tensor-map copy each whose coordinates carry the tap's shift (positions
// outside the output image arrive as zeros, which is exactly the convolution's padding), and one 128 x 64 tile of
// Wd; twelve tcgen05.mma (128 x 128 x 16, bf16 in, fp32 out) accumulate the stage in tensor memory.
//
// Tensor-core accumulation does not round to nearest, so long sums would drift beyond the 1e-5 the gradients are
// held to; as in the mma.sync kernels the running sum therefore lives in ordinary fp32 registers: after every
// stage the eight epilogue warps read the stage's accumulator out of tensor memory (tcgen05.ld) and add it to
// their sums while the MMA warp fills the other of two accumulators.
//
// Warps: 0 = TMA producer (one lane), 1 = MMA issuer (one lane; the warp also allocates tensor memory), 2..9 =
// epilogue (a warp may only read the tensor-memory lanes 32 * (warp % 4) .. + 31; two warps share a lane quarter
// and take 64 columns each).  Every wait on an mbarrier is bounded: when a wait runs out the CTA raises an error
// count, stops waiting anywhere and leaves; the host reads the count through geo_sc_device_error_count().
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

#include "sc_common.h"
#include "sc_guide_mma.h"
#include "sc_guide_tc.h"

namespace geo {

__device__ int g_tc_errors = 0;   // mbarrier waits that ran out, over the life of the process

namespace {

constexpr int TC_THREADS = 320;
constexpr int TC_STAGES = 3;
constexpr int TC_TILE_BYTES = 128 * 128;                 // 128 rows x 64 bf16
constexpr int TC_STAGE_BYTES = 4 * TC_TILE_BYTES;        // three terms of D + one tile of Wd
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 1024;   // + slack to align the tiles to 1024 bytes
constexpr int TC_SPIN_LIMIT = 1 << 22;
constexpr uint32_t TC_TMEM_COLS = 256;                   // two accumulators of 128 fp32 columns

// kind::f16 instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, N = 128, M = 128
constexpr uint32_t TC_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Waits for the phase of `bar` with parity `parity`, at most TC_SPIN_LIMIT polls; false = gave up (or another
// wait of this CTA already had: *abort is set, and nobody waits any more).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort) {
    for (int i = 0; i < TC_SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abort) return false;
    }
    if (!*abort) {
        *abort = 1;
        atomicAdd(&g_tc_errors, 1);
    }
    return false;
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3,
                                            int c4) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows under the 128-byte swizzle: 8-row groups of
// 1024 bytes follow each other (stride-byte-offset 1024); the leading-byte-offset is not used by this layout.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(TC_IDESC), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
                   "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
                   "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

struct TcDgradParams {
    float *ga;            // [B][C][H][W]
    const int *inexact;   // the tensor-core family stands down when this is set
    int B, C, H, W, ph, pw;
    int K2, K3, N2, G, mode;
    int bw, bh, nb;       // pixel tile: nb images x bh rows x bw columns = 128 pixels
    int tiles_x, tiles_y; // tiles per image row / column (nb == 1), else 1
};

__global__ void __launch_bounds__(TC_THREADS, 1)
tc_dgrad_kernel(const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_w, TcDgradParams pr) {
    if (*pr.inexact) return;
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * TC_STAGES + 4];   // full[3], empty[3], acc_full[2], acc_empty[2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    unsigned char *tiles = (unsigned char *)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t tiles_s = smem_u32(tiles);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (TC_STAGES + s); };
    auto accf_bar = [&](int a) { return bar0 + 8u * (2 * TC_STAGES + a); };
    auto acce_bar = [&](int a) { return bar0 + 8u * (2 * TC_STAGES + 2 + a); };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < TC_STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {   // one warp allocates tensor memory for the CTA and gives up the right to allocate more
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abort = &abort_flag;

    // pixel tile of this CTA
    int b0, y0, x0;
    {
        const int t = blockIdx.x;
        if (pr.nb > 1) { b0 = t * pr.nb; y0 = 0; x0 = 0; }
        else {
            const int per_img = pr.tiles_x * pr.tiles_y;
            b0 = t / per_img;
            const int r = t % per_img;
            y0 = (r / pr.tiles_x) * pr.bh;
            x0 = (r % pr.tiles_x) * pr.bw;
        }
    }
    const int c0 = blockIdx.y * 128;
    const int spt = pr.N2 / 64;                       // stages per tap
    const int n_iters = pr.K2 * pr.K3 * spt;

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < n_iters; it++) {
                const int s = it % TC_STAGES;
                if (!mbar_wait(empty_bar(s), ((it / TC_STAGES) & 1) ^ 1, abort)) break;
                mbar_expect_tx(full_bar(s), TC_STAGE_BYTES);
                const int tap = it / spt, n0 = (it % spt) * 64;
                const int ky = tap / pr.K3, kx = tap % pr.K3;
                const int g = pr.mode == GEO_SC_MODE_1D ? kx : (pr.mode == GEO_SC_MODE_2D ? tap : 0);
                const uint32_t dst = tiles_s + (uint32_t)s * TC_STAGE_BYTES;
                // output position of input pixel (y, x) under this tap: (y + ph - ky, x + pw - kx)
                for (int term = 0; term < 3; term++)
                    tma_load_5d(dst + term * TC_TILE_BYTES, &map_d, full_bar(s), n0, x0 + pr.pw - kx, y0 + pr.ph - ky, b0,
                                term * pr.G + g);
                tma_load_2d(dst + 3 * TC_TILE_BYTES, &map_w, full_bar(s), tap * pr.N2 + n0, c0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int it = 0; it < n_iters; it++) {
                const int s = it % TC_STAGES, a = it & 1;
                if (!mbar_wait(full_bar(s), (it / TC_STAGES) & 1, abort)) break;
                if (!mbar_wait(acce_bar(a), ((it >> 1) & 1) ^ 1, abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t st = tiles_s + (uint32_t)s * TC_STAGE_BYTES;
                const uint64_t bdesc = umma_desc(st + 3 * TC_TILE_BYTES);
                for (int term = 0; term < 3; term++) {
                    const uint64_t adesc = umma_desc(st + term * TC_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; k++)   // 16 bf16 = 32 bytes further along K: + 2 in units of 16 bytes
                        umma_bf16(tmem_base + a * 128, adesc + 2 * k, bdesc + 2 * k, (term | k) != 0);
                }
                umma_commit(empty_bar(s));   // the stage's tiles may be overwritten once these MMAs have read them
                umma_commit(accf_bar(a));    // and the accumulator is complete
            }
        }
    } else {
        const int ew = warp - 2, quarter = warp & 3, half = ew >> 2;
        float sum[64];
#pragma unroll
        for (int i = 0; i < 64; i++) sum[i] = 0.f;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 64;
        bool ok = true;
        for (int it = 0; it < n_iters && ok; it++) {
            const int a = it & 1;
            ok = mbar_wait(accf_bar(a), (it >> 1) & 1, abort);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            float v[32];
            tmem_ld32(lane_addr + a * 128, v);
#pragma unroll
            for (int i = 0; i < 32; i++) sum[i] += v[i];
            tmem_ld32(lane_addr + a * 128 + 32, v);
#pragma unroll
            for (int i = 0; i < 32; i++) sum[32 + i] += v[i];
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(a));
        }
        if (ok) {
            // row of this thread: pixel quarter * 32 + lane of the tile, in (image, row, column) order
            const int r = quarter * 32 + lane;
            const int xl = r % pr.bw, yl = (r / pr.bw) % pr.bh, bl = r / (pr.bw * pr.bh);
            const int b = b0 + bl, y = y0 + yl, x = x0 + xl;
            if (b < pr.B && y < pr.H && x < pr.W) {
                float *dst = pr.ga + ((size_t)b * pr.C + c0 + half * 64) * pr.H * pr.W + (size_t)y * pr.W + x;
#pragma unroll
                for (int j = 0; j < 64; j++)
                    if (c0 + half * 64 + j < pr.C) dst[(size_t)j * pr.H * pr.W] = sum[j];
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}


// ---- forward product and D = gout * exp(-y) ------------------------------------------------------------------
// y[m][n2] = sum over the members k' = (tap, c) of group g of a[pos(m) + tap][c] * Wb[g][n2][k'], then
// D = gout * exp(-y) split into three bf16 terms (sc_guide_mma.cu: mma_forward_kernel does the same on mma.sync).
// A CTA owns 128 output positions (whole rows of one image or whole small images) x 128 columns of one group.
// Stages of 64 members: a 128 x 64 tile of the padded NHWC activations, fetched by one 4-d tensor-map copy whose
// coordinates carry the tap's offset, and a 128 x 64 tile of Wb.  Two stages (eight MMAs, 128 members) make one
// accumulator batch, flushed into the epilogue warps' fp32 sums like in the kernel above.
constexpr int TF_STAGES = 4;
constexpr int TF_STAGE_BYTES = 2 * TC_TILE_BYTES;
constexpr int TF_GOUT_BYTES = 128 * 128 * 4;                       // gout of the tile: 128 channels x 128 positions fp32
constexpr int TF_SMEM = TF_STAGES * TF_STAGE_BYTES + TF_GOUT_BYTES + 1024;
static_assert(TF_STAGES * TF_STAGE_BYTES >= 6 * TC_TILE_BYTES, "the stage buffers double as staging for the three terms of D");

struct TcForwardParams {
    const float *gout;        // [B][O][Ho][Wo]
    __nv_bfloat16 *Dh;        // [3][G][M][N2]
    const int *inexact;
    int B, O, Opad, Ho, Wo, HoWo, M, N2, G, K3, mode;
    int cpb;                  // 64-channel blocks per tap (Cp / 64)
    int nkb;                  // stages: taps * cpb
    int bh, nb;               // position tile: nb images x bh rows x Wo columns = 128 positions
    int tiles_y;              // tiles per image (nb == 1), else 1
    int staged;               // gout arrives by TMA and D leaves by TMA through shared memory (else plain loads / stores)
    int ppi, ob;              // staged: positions per image in the tile, channels in the gout box
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];\n"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

__global__ void __launch_bounds__(TC_THREADS, 1)
tc_forward_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                  const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_o, TcForwardParams pr) {
    if (*pr.inexact) return;
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * TF_STAGES + 5];   // full, empty, acc_full[2], acc_empty[2], gout
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    unsigned char *tiles = (unsigned char *)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t tiles_s = smem_u32(tiles);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (TF_STAGES + s); };
    auto accf_bar = [&](int a) { return bar0 + 8u * (2 * TF_STAGES + a); };
    auto acce_bar = [&](int a) { return bar0 + 8u * (2 * TF_STAGES + 2 + a); };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < TF_STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), 8); }
        mbar_init(bar0 + 8u * (2 * TF_STAGES + 4), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abort = &abort_flag;
    const uint32_t gout_bar = bar0 + 8u * (2 * TF_STAGES + 4);
    unsigned char *gout_tile = tiles + TF_STAGES * TF_STAGE_BYTES;

    int b0, oy0;
    if (pr.nb > 1) { b0 = blockIdx.x * pr.nb; oy0 = 0; }
    else { b0 = blockIdx.x / pr.tiles_y; oy0 = (blockIdx.x % pr.tiles_y) * pr.bh; }
    const int m0 = (b0 * pr.Ho + oy0) * pr.Wo;
    const int n0 = blockIdx.y * 128, g = blockIdx.z;
    const int nkb = pr.nkb, nbatch = (nkb + 1) / 2;

    if (warp == 0) {
        if (lane == 0) {
            if (pr.staged) {   // gout of the tile, [image][channel][position]; channels past c_out arrive as zeros
                mbar_expect_tx(gout_bar, (uint32_t)(pr.ob * 128 * 4));
                tma_load_3d(smem_u32(gout_tile), &map_g, gout_bar, oy0 * pr.Wo, n0 % pr.Opad, b0);
            }
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % TF_STAGES;
                if (!mbar_wait(empty_bar(s), ((kb / TF_STAGES) & 1) ^ 1, abort)) break;
                mbar_expect_tx(full_bar(s), TF_STAGE_BYTES);
                const int tap = kb / pr.cpb, c0 = (kb % pr.cpb) * 64;
                int ky, kx;   // 1d_bin groups are filter columns (taps = rows), 2d_bin groups single taps, full_or all taps
                if (pr.mode == GEO_SC_MODE_1D) { ky = tap; kx = g; }
                else if (pr.mode == GEO_SC_MODE_2D) { ky = g / pr.K3; kx = g % pr.K3; }
                else { ky = tap / pr.K3; kx = tap % pr.K3; }
                const uint32_t dst = tiles_s + (uint32_t)s * TF_STAGE_BYTES;
                tma_load_4d(dst, &map_a, full_bar(s), c0, kx, oy0 + ky, b0);
                tma_load_2d(dst + TC_TILE_BYTES, &map_w, full_bar(s), kb * 64, g * pr.N2 + n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; kb++) {
                const int s = kb % TF_STAGES, batch = kb >> 1, a = batch & 1;
                if (!mbar_wait(full_bar(s), (kb / TF_STAGES) & 1, abort)) break;
                if ((kb & 1) == 0 && !mbar_wait(acce_bar(a), ((batch >> 1) & 1) ^ 1, abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t st = tiles_s + (uint32_t)s * TF_STAGE_BYTES;
                const uint64_t adesc = umma_desc(st), bdesc = umma_desc(st + TC_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < 4; k++) umma_bf16(tmem_base + a * 128, adesc + 2 * k, bdesc + 2 * k, ((kb & 1) | k) != 0);
                umma_commit(empty_bar(s));
                if ((kb & 1) == 1 || kb == nkb - 1) umma_commit(accf_bar(a));
            }
        }
    } else {
        const int ew = warp - 2, quarter = warp & 3, half = ew >> 2;
        float sum[64];
#pragma unroll
        for (int i = 0; i < 64; i++) sum[i] = 0.f;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 64;
        bool ok = true;
        for (int batch = 0; batch < nbatch; batch++) {
            const int a = batch & 1;
            ok = mbar_wait(accf_bar(a), (batch >> 1) & 1, abort);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            float v[32];
            tmem_ld32(lane_addr + a * 128, v);
#pragma unroll
            for (int i = 0; i < 32; i++) sum[i] += v[i];
            tmem_ld32(lane_addr + a * 128 + 32, v);
#pragma unroll
            for (int i = 0; i < 32; i++) sum[32 + i] += v[i];
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(a));
        }
        const int r = quarter * 32 + lane, m = m0 + r;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
        if (pr.staged) {
            // gout from shared memory, D through shared memory: the thread's 64 columns are one 128-byte row of the
            // (term, half) box, written in the 128-byte swizzle that the tensor-map store undoes; the stage buffers
            // are free (every MMA that read them has completed before the last accumulator was handed over)
            if (ok) ok = mbar_wait(gout_bar, 0, abort);
            const float *gs = (const float *)gout_tile + (size_t)(r / pr.ppi) * pr.ob * pr.ppi + r % pr.ppi;
            if (ok) {
#pragma unroll
                for (int c8 = 0; c8 < 8; c8++) {
                    uint32_t t0[4], t1[4], t2[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int j = c8 * 8 + e * 2;
                        const int o0 = (half * 64 + j) % pr.ob, o1 = (half * 64 + j + 1) % pr.ob;
                        const float v0 = gs[o0 * pr.ppi] * expf(-sum[j]), v1 = gs[o1 * pr.ppi] * expf(-sum[j + 1]);
                        __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                        const uint32_t p0 = *(uint32_t *)&h;
                        const float r0 = v0 - __uint_as_float(p0 << 16), r1 = v1 - __uint_as_float(p0 & 0xffff0000u);
                        h = __floats2bfloat162_rn(r0, r1);
                        const uint32_t p1 = *(uint32_t *)&h;
                        const float s0 = r0 - __uint_as_float(p1 << 16), s1 = r1 - __uint_as_float(p1 & 0xffff0000u);
                        h = __floats2bfloat162_rn(s0, s1);
                        t0[e] = p0; t1[e] = p1; t2[e] = *(uint32_t *)&h;
                    }
                    unsigned char *row = tiles + (size_t)half * TC_TILE_BYTES + r * 128 + ((c8 ^ (r & 7)) << 4);
                    *(uint4 *)(row) = make_uint4(t0[0], t0[1], t0[2], t0[3]);
                    *(uint4 *)(row + 2 * TC_TILE_BYTES) = make_uint4(t1[0], t1[1], t1[2], t1[3]);
                    *(uint4 *)(row + 4 * TC_TILE_BYTES) = make_uint4(t2[0], t2[1], t2[2], t2[3]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("bar.sync 1, 256;\n" ::: "memory");   // the eight epilogue warps
            if (ew == 0 && lane == 0 && !*abort) {
                for (int term = 0; term < 3; term++)
                    for (int hh = 0; hh < 2; hh++)
                        tma_store_3d(&map_o, tiles_s + (uint32_t)(term * 2 + hh) * TC_TILE_BYTES, n0 + hh * 64, m0, term * pr.G + g);
                asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");   // shared memory is read out before the CTA may leave
            }
        } else if (ok && b < pr.B && m < pr.M) {
            const size_t plane = (size_t)pr.G * pr.M * pr.N2;
            __nv_bfloat16 *row = pr.Dh + ((size_t)g * pr.M + m) * pr.N2 + n0 + half * 64;
            const float *grow = pr.gout + (size_t)b * pr.O * pr.HoWo + rem;
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++) {
                uint32_t t0[4], t1[4], t2[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int j = c8 * 8 + e * 2;
                    const int o0 = (n0 + half * 64 + j) % pr.Opad, o1 = (n0 + half * 64 + j + 1) % pr.Opad;
                    const float g0 = o0 < pr.O ? __ldg(grow + (size_t)o0 * pr.HoWo) : 0.0f;
                    const float g1 = o1 < pr.O ? __ldg(grow + (size_t)o1 * pr.HoWo) : 0.0f;
                    const float v0 = g0 * expf(-sum[j]), v1 = g1 * expf(-sum[j + 1]);
                    // three-term bf16 split of both values at once (cvt.rn.bf16x2.f32)
                    __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                    const uint32_t p0 = *(uint32_t *)&h;
                    const float r0 = v0 - __uint_as_float(p0 << 16), r1 = v1 - __uint_as_float(p0 & 0xffff0000u);
                    h = __floats2bfloat162_rn(r0, r1);
                    const uint32_t p1 = *(uint32_t *)&h;
                    const float s0 = r0 - __uint_as_float(p1 << 16), s1 = r1 - __uint_as_float(p1 & 0xffff0000u);
                    h = __floats2bfloat162_rn(s0, s1);
                    t0[e] = p0; t1[e] = p1; t2[e] = *(uint32_t *)&h;
                }
                *(uint4 *)(row + c8 * 8) = make_uint4(t0[0], t0[1], t0[2], t0[3]);
                *(uint4 *)(row + plane + c8 * 8) = make_uint4(t1[0], t1[1], t1[2], t1[3]);
                *(uint4 *)(row + 2 * plane + c8 * 8) = make_uint4(t2[0], t2[1], t2[2], t2[3]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ---- weight gradient ----------------------------------------------------------------------------------------
// partial[slice][g][k'][n2] = sum over the slice's positions m of a[pos(m) + tap][c] * D_term[g][m][n2] over the
// three terms: the contraction runs over positions, so both operands are "MN-major" for the tensor core -- a stage
// holds 64 positions as rows of 128 bytes, [64 m][64 channels] twice for the 128 members k' = (tap, c0 .. c0 + 127)
// of the tile and [64 m][64 columns] twice per term for its 128 columns, exactly as the tensor-map copies deliver
// them.  Descriptor: 128-byte swizzle, leading-byte-offset = distance between the two 64-wide blocks (8 KB),
// stride-byte-offset = distance between groups of eight positions (1 KB); an MMA consumes 16 positions (2 KB).
// The epilogue is the one of the activation-gradient kernel: the sum over positions is long and of mixed sign, so
// every stage's accumulator is added into fp32 registers.  One CTA per (slice of positions, 128 members, 128 columns,
// group); mma_wgrad_reduce_kernel adds the slices and applies the sign masks.
constexpr int TW_BLOCK_BYTES = 64 * 128;                       // 64 positions x 64 bf16
constexpr int TW_STAGE_BYTES = 8 * TW_BLOCK_BYTES;             // A: 2 blocks, D: 3 terms x 2 blocks
constexpr int TW_SMEM = TC_STAGES * TW_STAGE_BYTES + 1024;
constexpr uint32_t TW_IDESC = TC_IDESC | (1u << 15) | (1u << 16);   // A and B MN-major

__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
__device__ __forceinline__ void umma_bf16_mn(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(TW_IDESC), "r"(accumulate)
                 : "memory");
}

struct TcWgradParams {
    float *partial;           // [S][G][Kp][N2]
    const int *inexact;
    int M, Ho, Wo, HoWo, N2, G, Kp, Cp, K3, mode;
    int slice_len;            // positions per slice, a multiple of 64
    int n2tiles;              // N2 / 128
    uint32_t lbo, sbo;
};

__global__ void __launch_bounds__(TC_THREADS, 1)
tc_wgrad_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_d, TcWgradParams pr) {
    if (*pr.inexact) return;
    extern __shared__ unsigned char tc_smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * TC_STAGES + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    unsigned char *tiles = (unsigned char *)(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t tiles_s = smem_u32(tiles);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (TC_STAGES + s); };
    auto accf_bar = [&](int a) { return bar0 + 8u * (2 * TC_STAGES + a); };
    auto acce_bar = [&](int a) { return bar0 + 8u * (2 * TC_STAGES + 2 + a); };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < TC_STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), 8); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abort = &abort_flag;

    const int slice = blockIdx.x, k0 = blockIdx.y * 128;
    const int g = blockIdx.z / pr.n2tiles, n0 = (blockIdx.z % pr.n2tiles) * 128;
    const int tap = k0 / pr.Cp, c0 = k0 % pr.Cp;
    int ky, kx;
    if (pr.mode == GEO_SC_MODE_1D) { ky = tap; kx = g; }
    else if (pr.mode == GEO_SC_MODE_2D) { ky = g / pr.K3; kx = g % pr.K3; }
    else { ky = tap / pr.K3; kx = tap % pr.K3; }
    const int mbeg = slice * pr.slice_len, mend = min(pr.M, mbeg + pr.slice_len);
    const int n_iters = (mend - mbeg + 63) / 64;

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < n_iters; it++) {
                const int s = it % TC_STAGES;
                if (!mbar_wait(empty_bar(s), ((it / TC_STAGES) & 1) ^ 1, abort)) break;
                mbar_expect_tx(full_bar(s), TW_STAGE_BYTES);
                const int m0 = mbeg + it * 64;
                const int b0 = m0 / pr.HoWo, oy0 = (m0 % pr.HoWo) / pr.Wo;
                const uint32_t dst = tiles_s + (uint32_t)s * TW_STAGE_BYTES;
                tma_load_4d(dst, &map_a, full_bar(s), c0, kx, oy0 + ky, b0);
                tma_load_4d(dst + TW_BLOCK_BYTES, &map_a, full_bar(s), c0 + 64, kx, oy0 + ky, b0);
                for (int term = 0; term < 3; term++)
                    for (int h = 0; h < 2; h++)
                        tma_load_5d(dst + (2 + term * 2 + h) * TW_BLOCK_BYTES, &map_d, full_bar(s), n0 + h * 64, 0, oy0, b0,
                                    term * pr.G + g);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int it = 0; it < n_iters; it++) {
                const int s = it % TC_STAGES, a = it & 1;
                if (!mbar_wait(full_bar(s), (it / TC_STAGES) & 1, abort)) break;
                if (!mbar_wait(acce_bar(a), ((it >> 1) & 1) ^ 1, abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t st = tiles_s + (uint32_t)s * TW_STAGE_BYTES;
                for (int term = 0; term < 3; term++) {
#pragma unroll
                    for (int k = 0; k < 4; k++) {   // 16 positions = two groups of eight rows = 2 KB further
                        const uint64_t adesc = umma_desc_mn(st + k * 2048, pr.lbo, pr.sbo);
                        const uint64_t bdesc = umma_desc_mn(st + (2 + term * 2) * TW_BLOCK_BYTES + k * 2048, pr.lbo, pr.sbo);
                        umma_bf16_mn(tmem_base + a * 128, adesc, bdesc, (term | k) != 0);
                    }
                }
                umma_commit(empty_bar(s));
                umma_commit(accf_bar(a));
            }
        }
    } else {
        const int ew = warp - 2, quarter = warp & 3, half = ew >> 2;
        float sum[64];
#pragma unroll
        for (int i = 0; i < 64; i++) sum[i] = 0.f;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + half * 64;
        bool ok = true;
        for (int it = 0; it < n_iters; it++) {
            const int a = it & 1;
            ok = mbar_wait(accf_bar(a), (it >> 1) & 1, abort);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            float v[32];
            tmem_ld32(lane_addr + a * 128, v);
#pragma unroll
            for (int i = 0; i < 32; i++) sum[i] += v[i];
            tmem_ld32(lane_addr + a * 128 + 32, v);
#pragma unroll
            for (int i = 0; i < 32; i++) sum[32 + i] += v[i];
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(a));
        }
        if (ok) {
            const int k = k0 + quarter * 32 + lane;   // accumulator row = member of the tile
            float *dst = pr.partial + (((size_t)slice * pr.G + g) * pr.Kp + k) * pr.N2 + n0 + half * 64;
#pragma unroll
            for (int j = 0; j < 64; j += 4) *(float4 *)(dst + j) = make_float4(sum[j], sum[j + 1], sum[j + 2], sum[j + 3]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, []() {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

}  // namespace

bool tc_dgrad_plan(const MmaDims &d, int Cn, TcTile *tile) {
    static const bool disabled = std::getenv("GEO_SC_NO_TCGEN05") != nullptr;
    if (disabled || !encode_fn()) return false;
    if (d.N2 % 64 != 0 || Cn % 128 != 0 || d.C < 128) return false;
    if (d.mode != GEO_SC_MODE_1D && d.mode != GEO_SC_MODE_2D && d.mode != GEO_SC_MODE_FULL_OR) return false;
    const int W = d.W, H = d.H;
    if (W < 1 || W > 128 || (W & (W - 1)) != 0) return false;          // rows of the box: a power of two up to 128
    int bw = W, bh, nb;
    if (H * W >= 128) {                                                // part of one image: whole rows
        bh = 128 / bw; nb = 1;
        if (H % bh != 0) return false;
    } else {                                                           // several whole images
        bh = H;
        if (128 % (bw * bh) != 0) return false;
        nb = 128 / (bw * bh);
    }
    if (bw > 256 || bh > 256 || nb > 256 || nb > d.B) return false;   // a box never exceeds the tensor it is cut from
    if ((long long)d.M * d.N2 * 2 >= (1LL << 40)) return false;
    tile->bw = bw; tile->bh = bh; tile->nb = nb;
    return true;
}

int launch_tc_dgrad(const MmaDims &d, int Cn, const void *Dh, const void *wd, float *grad_act, const int *flag,
                    cudaStream_t s) {
    TcTile tile;
    if (!tc_dgrad_plan(d, Cn, &tile)) return fail(GEO_SC_ERR_UNSUPPORTED, "shape not served by the tcgen05 activation-gradient kernel");
    CUtensorMap map_d, map_w;
    {
        const cuuint64_t dims[5] = {(cuuint64_t)d.N2, (cuuint64_t)d.Wo, (cuuint64_t)d.Ho, (cuuint64_t)d.B, (cuuint64_t)(3 * d.G)};
        const cuuint64_t strides[4] = {(cuuint64_t)d.N2 * 2, (cuuint64_t)d.Wo * d.N2 * 2, (cuuint64_t)d.HoWo * d.N2 * 2,
                                       (cuuint64_t)d.M * d.N2 * 2};
        const cuuint32_t box[5] = {64, (cuuint32_t)tile.bw, (cuuint32_t)tile.bh, (cuuint32_t)tile.nb, 1};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUresult r = encode_fn()(&map_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(Dh), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (D) failed: %d", (int)r);
    }
    {
        const cuuint64_t R = (cuuint64_t)d.K2 * d.K3 * d.N2;
        const cuuint64_t dims[2] = {R, (cuuint64_t)Cn};
        const cuuint64_t strides[1] = {R * 2};
        const cuuint32_t box[2] = {64, 128};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = encode_fn()(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(wd), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (Wd) failed: %d", (int)r);
    }
    TcDgradParams pr;
    pr.ga = grad_act; pr.inexact = flag;
    pr.B = d.B; pr.C = d.C; pr.H = d.H; pr.W = d.W; pr.ph = d.ph; pr.pw = d.pw;
    pr.K2 = d.K2; pr.K3 = d.K3; pr.N2 = d.N2; pr.G = d.G; pr.mode = d.mode;
    pr.bw = tile.bw; pr.bh = tile.bh; pr.nb = tile.nb;
    pr.tiles_x = tile.nb > 1 ? 1 : d.W / tile.bw;
    pr.tiles_y = tile.nb > 1 ? 1 : d.H / tile.bh;
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(tc_dgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    const unsigned ptiles = tile.nb > 1 ? (unsigned)((d.B + tile.nb - 1) / tile.nb) : (unsigned)(d.B * pr.tiles_x * pr.tiles_y);
    dim3 grid(ptiles, (unsigned)(Cn / 128), 1);
    tc_dgrad_kernel<<<grid, TC_THREADS, TC_SMEM, s>>>(map_d, map_w, pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

// Position tile over an Ho x Wo image: nb images x bh rows x all Wo columns = 128 positions.
static bool position_tile(int H, int W, int *bh, int *nb) {
    if (W < 1 || W > 128 || (W & (W - 1)) != 0) return false;
    if (H * W >= 128) {
        *bh = 128 / W; *nb = 1;
        return H % *bh == 0;
    }
    *bh = H;
    if (128 % (W * H) != 0) return false;
    *nb = 128 / (W * H);
    return *nb <= 256;
}

bool tc_forward_plan(const MmaDims &d, TcTile *tile) {
    static const bool disabled = std::getenv("GEO_SC_NO_TCGEN05") != nullptr;
    if (disabled || !encode_fn() || d.linear) return false;
    if (d.N2 % 128 != 0 || d.Cp % 64 != 0) return false;
    if (d.mode != GEO_SC_MODE_1D && d.mode != GEO_SC_MODE_2D && d.mode != GEO_SC_MODE_FULL_OR) return false;
    if (d.Kp != d.taps * d.Cp) return false;
    if ((long long)d.M * d.N2 * 2 >= (1LL << 40)) return false;
    int bh, nb;
    if (!position_tile(d.Ho, d.Wo, &bh, &nb) || nb > d.B) return false;
    tile->bw = d.Wo; tile->bh = bh; tile->nb = nb;
    return true;
}

int launch_tc_forward(const MmaDims &d, const void *apad, const void *wb, const float *gout, void *Dh, const int *flag,
                      cudaStream_t s) {
    TcTile tile;
    if (!tc_forward_plan(d, &tile)) return fail(GEO_SC_ERR_UNSUPPORTED, "shape not served by the tcgen05 forward kernel");
    CUtensorMap map_a, map_w;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)d.Cp, (cuuint64_t)d.Wp, (cuuint64_t)d.Hp, (cuuint64_t)d.B};
        const cuuint64_t strides[3] = {(cuuint64_t)d.Cp * 2, (cuuint64_t)d.Wp * d.Cp * 2, (cuuint64_t)d.Hp * d.Wp * d.Cp * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)tile.bw, (cuuint32_t)tile.bh, (cuuint32_t)tile.nb};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = encode_fn()(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(apad), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (activations) failed: %d", (int)r);
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)d.Kp, (cuuint64_t)d.G * d.N2};
        const cuuint64_t strides[1] = {(cuuint64_t)d.Kp * 2};
        const cuuint32_t box[2] = {64, 128};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = encode_fn()(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(wb), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (Wb) failed: %d", (int)r);
    }
    // gout arrives by TMA when the positions of an image inside the tile are at least 16 bytes; D leaves by TMA then
    const int ppi = tile.nb > 1 ? d.HoWo : 128, ob = d.Opad < 128 ? d.Opad : 128;
    const bool staged = ppi % 4 == 0 && ((uintptr_t)gout & 15) == 0 && (d.HoWo * 4) % 16 == 0;
    CUtensorMap map_g = map_a, map_o = map_a;   // placeholders when not staged (never dereferenced)
    if (staged) {
        const cuuint64_t gdims[3] = {(cuuint64_t)d.HoWo, (cuuint64_t)d.O, (cuuint64_t)d.B};
        const cuuint64_t gstrides[2] = {(cuuint64_t)d.HoWo * 4, (cuuint64_t)d.O * d.HoWo * 4};
        const cuuint32_t gbox[3] = {(cuuint32_t)ppi, (cuuint32_t)ob, (cuuint32_t)tile.nb};
        const cuuint32_t gestr[3] = {1, 1, 1};
        CUresult r = encode_fn()(&map_g, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(gout), gdims, gstrides, gbox, gestr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (gout) failed: %d", (int)r);
        const cuuint64_t odims[3] = {(cuuint64_t)d.N2, (cuuint64_t)d.M, (cuuint64_t)(3 * d.G)};
        const cuuint64_t ostrides[2] = {(cuuint64_t)d.N2 * 2, (cuuint64_t)d.M * d.N2 * 2};
        const cuuint32_t obox[3] = {64, 128, 1};
        r = encode_fn()(&map_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, Dh, odims, ostrides, obox, gestr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (D store) failed: %d", (int)r);
    }
    TcForwardParams pr;
    pr.staged = staged ? 1 : 0; pr.ppi = ppi; pr.ob = ob;
    pr.gout = gout; pr.Dh = (__nv_bfloat16 *)Dh; pr.inexact = flag;
    pr.B = d.B; pr.O = d.O; pr.Opad = d.Opad; pr.Ho = d.Ho; pr.Wo = d.Wo; pr.HoWo = d.HoWo; pr.M = d.M; pr.N2 = d.N2; pr.G = d.G;
    pr.K3 = d.K3; pr.mode = d.mode;
    pr.cpb = d.Cp / 64; pr.nkb = d.taps * pr.cpb;
    pr.bh = tile.bh; pr.nb = tile.nb;
    pr.tiles_y = tile.nb > 1 ? 1 : d.Ho / tile.bh;
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(tc_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TF_SMEM));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    const unsigned ptiles = tile.nb > 1 ? (unsigned)((d.B + tile.nb - 1) / tile.nb) : (unsigned)(d.B * pr.tiles_y);
    dim3 grid(ptiles, (unsigned)(d.N2 / 128), (unsigned)d.G);
    tc_forward_kernel<<<grid, TC_THREADS, TF_SMEM, s>>>(map_a, map_w, map_g, map_o, pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

bool tc_wgrad_plan(const MmaDims &d, int slice_len, TcTile *tile) {
    static const bool disabled = std::getenv("GEO_SC_NO_TCGEN05") != nullptr;
    if (disabled || !encode_fn()) return false;
    if (d.N2 % 128 != 0 || d.Cp % 128 != 0 || d.Kp != d.taps * d.Cp) return false;
    if (d.mode != GEO_SC_MODE_1D && d.mode != GEO_SC_MODE_2D && d.mode != GEO_SC_MODE_FULL_OR) return false;
    if (slice_len % 64 != 0 || d.M % 64 != 0) return false;
    const int W = d.Wo, H = d.Ho;
    if (W < 1 || W > 64 || (W & (W - 1)) != 0) return false;
    int bh, nb;
    if (H * W >= 64) { bh = 64 / W; nb = 1; if (H % bh != 0) return false; }
    else { bh = H; if (64 % (W * H) != 0) return false; nb = 64 / (W * H); }
    if (nb > d.B) return false;
    if ((long long)d.M * d.N2 * 2 >= (1LL << 40)) return false;
    tile->bw = W; tile->bh = bh; tile->nb = nb;
    return true;
}

int launch_tc_wgrad(const MmaDims &d, const void *apad, const void *Dh, float *partial, int S, int slice_len, const int *flag,
                    cudaStream_t s) {
    TcTile tile;
    if (!tc_wgrad_plan(d, slice_len, &tile)) return fail(GEO_SC_ERR_UNSUPPORTED, "shape not served by the tcgen05 weight-gradient kernel");
    CUtensorMap map_a, map_d;
    {
        const cuuint64_t dims[4] = {(cuuint64_t)d.Cp, (cuuint64_t)d.Wp, (cuuint64_t)d.Hp, (cuuint64_t)d.B};
        const cuuint64_t strides[3] = {(cuuint64_t)d.Cp * 2, (cuuint64_t)d.Wp * d.Cp * 2, (cuuint64_t)d.Hp * d.Wp * d.Cp * 2};
        const cuuint32_t box[4] = {64, (cuuint32_t)tile.bw, (cuuint32_t)tile.bh, (cuuint32_t)tile.nb};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = encode_fn()(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(apad), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (activations) failed: %d", (int)r);
    }
    {
        const cuuint64_t dims[5] = {(cuuint64_t)d.N2, (cuuint64_t)d.Wo, (cuuint64_t)d.Ho, (cuuint64_t)d.B, (cuuint64_t)(3 * d.G)};
        const cuuint64_t strides[4] = {(cuuint64_t)d.N2 * 2, (cuuint64_t)d.Wo * d.N2 * 2, (cuuint64_t)d.HoWo * d.N2 * 2,
                                       (cuuint64_t)d.M * d.N2 * 2};
        const cuuint32_t box[5] = {64, (cuuint32_t)tile.bw, (cuuint32_t)tile.bh, (cuuint32_t)tile.nb, 1};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUresult r = encode_fn()(&map_d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(Dh), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(GEO_SC_ERR_CUDA, "cuTensorMapEncodeTiled (D) failed: %d", (int)r);
    }
    TcWgradParams pr;
    pr.partial = partial; pr.inexact = flag;
    pr.M = d.M; pr.Ho = d.Ho; pr.Wo = d.Wo; pr.HoWo = d.HoWo; pr.N2 = d.N2; pr.G = d.G; pr.Kp = d.Kp; pr.Cp = d.Cp; pr.K3 = d.K3;
    pr.mode = d.mode;
    pr.slice_len = slice_len;
    pr.n2tiles = d.N2 / 128;
    // leading-byte-offset: from one 64-wide block of members (or columns) to the next; stride-byte-offset: from one
    // group of eight positions to the next
    pr.lbo = TW_BLOCK_BYTES;
    pr.sbo = 1024;
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(tc_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TW_SMEM));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    dim3 grid((unsigned)S, (unsigned)(d.Kp / 128), (unsigned)(d.G * pr.n2tiles));
    tc_wgrad_kernel<<<grid, TC_THREADS, TW_SMEM, s>>>(map_a, map_d, pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int tc_error_count(int *count) {
    GEO_CUDA_CHECK(cudaMemcpyFromSymbol(count, g_tc_errors, sizeof(int)));
    return GEO_SC_OK;
}

}  // namespace geo
