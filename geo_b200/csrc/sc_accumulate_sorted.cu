// SC accumulation with the members of a group sorted by the sign pattern of four output channels.
//
// A weight is positive or negative, so one of its two streams is all zeros and half of the dense
// kernel's LOP3 (sc_accumulate.cu) OR zeros into an accumulator.  Here a warp owns four output
// channels (a "quad") and 128 positions (four per lane).  At weight-preparation time the members of a
// group (in chunks of at most kSortChunkMax) are sorted, per quad, by which of the four weights are
// negative -- 16 patterns -- and only the non-zero stream word of each weight is kept.  The kernel
// then runs one straight-line loop per pattern, in which every activation word meets exactly one
// LOP3 per channel, into the accumulator of the right polarity: 16 LOP3 per member and lane instead
// of the 32 the dense tile spends on the same 4 positions x 4 channels.  Members whose four weights
// are all zero are dropped.  The price: the quads of a CTA walk the members in different orders, so
// the activation words of a whole chunk must sit in shared memory at once, and their reads are no
// longer shared between channel groups.
#include "sc_common.h"
#include "sc_sorted.h"

namespace geo {

namespace {

__device__ __forceinline__ void cp4(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp16(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }

struct SortedParams {
    const uint32_t *as;    // [B][P][C][Hp][Wp]
    const int32_t *aoff;   // [G][Kp]
    const uint4 *sw;       // [P][G][NCH][Q][SL]: the four non-zero stream words of a sorted member
    const uint16_t *srow;  // [G][NCH][Q][SL]: 32 * (row of the member inside its chunk) = its uint4 offset in the tile
    const uint16_t *sbeg;  // [G][NCH][Q][18]: first slot of each of the 16 patterns, then the end
    int32_t *out;          // [B][O][Ho][Wo]
    int M, O, HoWo, Wo, Wp;
    int P, G, Kp, NCH, KCH, SL, Q;
    int img_words, pack_words, aoff_mul, splits;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

// One pattern's members: PAT bit j set = the weight of channel j is negative.  atile: shared address of the lane's
// four positions in row 0 of the tile; sw / srow: shared addresses of the quad's lists of stream
// words and of tile rows.  Explicit 32-bit shared addresses: generic pointers cost the sibling kernels 3-6 %.
template <int PAT>
__device__ __forceinline__ void run_bucket(uint32_t (&accp)[4][4], uint32_t (&accn)[4][4], uint32_t atile, uint32_t sw,
                                           uint32_t srow, int i0, int i1) {
#pragma unroll 4
    for (int i = i0; i < i1; i++) {
        const uint4 w = lds128(sw + (uint32_t)i * 16);
        const uint4 a = lds128(atile + lds16(srow + (uint32_t)i * 2) * 16);   // list entries are in units of 16 bytes
        const uint32_t av[4] = {a.x, a.y, a.z, a.w};
        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int p = 0; p < 4; p++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (PAT & (1 << j)) accn[p][j] |= av[p] & wv[j];
                else accp[p][j] |= av[p] & wv[j];
            }
    }
}

// Shared memory: activation words of one chunk [KCH][128], then the sorted lists of the CTA's NQ quads
// for the current (pack, group, chunk): stream words [NQ][SL] uint4, tile offsets [NQ][SL] u16 and
// pattern boundaries [NQ][18] u16.
template <int NQ>
__global__ void __launch_bounds__(NQ * 32, 2) accumulate_sorted_kernel(SortedParams pr) {
    extern __shared__ __align__(16) uint32_t smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int m0 = blockIdx.x * 128;
    const int q0 = blockIdx.y * NQ, q = q0 + warp;     // this warp's channel quad
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sw_base = smem_base + (uint32_t)pr.KCH * 128 * 4;
    const uint32_t srow_base = sw_base + (uint32_t)NQ * pr.SL * 16;
    const uint32_t sbeg_base = srow_base + (uint32_t)NQ * pr.SL * 2;
    const uint32_t atile = smem_base + (uint32_t)lane * 16;
    const uint32_t swl = sw_base + (uint32_t)(warp * pr.SL) * 16;
    const uint32_t srl = srow_base + (uint32_t)(warp * pr.SL) * 2;
    const uint16_t *sbl = (const uint16_t *)(smem + pr.KCH * 128 + NQ * pr.SL * 4 + NQ * pr.SL / 2) + warp * 18;

    // gather assignment: thread t copies position t % 128 of rows t / 128 + i * (NQ / 4)
    constexpr int RSTEP = NQ * 32 / 128;
    int abase;
    {
        int m = m0 + (t & 127);
        if (m >= pr.M) m = pr.M - 1;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
        abase = b * pr.img_words + ((rem / pr.Wo) * pr.Wp + (rem % pr.Wo)) * pr.aoff_mul;
    }
    const int pairs = pr.P * pr.G;
    const int pair0 = (int)((long long)pairs * blockIdx.z / pr.splits);
    const int pair1 = (int)((long long)pairs * (blockIdx.z + 1) / pr.splits);

    int osum[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) osum[i][j] = 0;

    for (int pair = pair0; pair < pair1; pair++) {
        const int p = pair / pr.G, g = pair % pr.G;
        uint32_t accp[4][4], accn[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) { accp[i][j] = 0; accn[i][j] = 0; }
        for (int c = 0; c < pr.NCH; c++) {
            const int k0 = c * pr.KCH, rows = min(pr.KCH, pr.Kp - k0);
            const size_t gcq0 = ((size_t)g * pr.NCH + c) * pr.Q + q0;
            __syncthreads();   // every warp is done with the previous chunk
            {
                const uint32_t *src = pr.as + p * pr.pack_words + abase;
                const int32_t *aoff = pr.aoff + g * pr.Kp + k0;
                for (int r = t >> 7; r < rows; r += RSTEP)
                    cp4(smem_base + (uint32_t)(r * 128 + (t & 127)) * 4, src + __ldg(aoff + r) * pr.aoff_mul);
                // the NQ quads' lists are contiguous in global memory
                const uint4 *wsrc = pr.sw + ((size_t)p * pr.G * pr.NCH * pr.Q + gcq0) * pr.SL;
                for (int i = t; i < NQ * pr.SL; i += NQ * 32) cp16(sw_base + (uint32_t)i * 16, wsrc + i);
                const uint4 *rsrc = (const uint4 *)(pr.srow + gcq0 * pr.SL);
                for (int i = t; i < NQ * pr.SL / 8; i += NQ * 32) cp16(srow_base + (uint32_t)i * 16, rsrc + i);
                // and so are their pattern boundaries: NQ x 18 u16 = NQ * 36 bytes
                if (t < NQ * 36 / 16) cp16(sbeg_base + (uint32_t)t * 16, (const uint4 *)(pr.sbeg + gcq0 * 18) + t);
                cp_commit();
                cp_wait_all();
            }
            __syncthreads();
            // lane b holds the first slot of pattern b; the loops get their bounds by shuffle
            const int mybeg = lane < 17 ? (int)sbl[lane] : 0;
#define GEO_BUCKET(B)                                                                                \
    run_bucket<B>(accp, accn, atile, swl, srl, __shfl_sync(0xffffffffu, mybeg, B), __shfl_sync(0xffffffffu, mybeg, B + 1));
            GEO_BUCKET(0) GEO_BUCKET(1) GEO_BUCKET(2) GEO_BUCKET(3) GEO_BUCKET(4) GEO_BUCKET(5) GEO_BUCKET(6) GEO_BUCKET(7)
            GEO_BUCKET(8) GEO_BUCKET(9) GEO_BUCKET(10) GEO_BUCKET(11) GEO_BUCKET(12) GEO_BUCKET(13) GEO_BUCKET(14) GEO_BUCKET(15)
#undef GEO_BUCKET
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) osum[i][j] += __popc(accp[i][j]) - __popc(accn[i][j]);
    }

    // store: lane owns positions m0 + 4*lane .. + 3, channels 4*q .. + 3
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + lane * 4 + i;
        if (m < pr.M) {
            const int b = m / pr.HoWo, rem = m % pr.HoWo;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int o = q * 4 + j;
                if (o < pr.O) {
                    int32_t *dst = pr.out + ((size_t)b * pr.O + o) * pr.HoWo + rem;
                    if (pr.splits > 1) atomicAdd(dst, osum[i][j]);
                    else *dst = osum[i][j];
                }
            }
        }
    }
}

// ---- preparation: sort the members of every (group, chunk) per channel quad ---------------------------
// Reads the dense prepared streams ws[P][G][Kp][Opad][2].  One CTA per (quad, group * chunk).
__global__ void __launch_bounds__(128) sort_members_kernel(const uint32_t *__restrict__ ws, int P, int G, int Kp, int Opad,
                                                           int NCH, int KCH, int SL, int Q, uint4 *__restrict__ sw,
                                                           uint16_t *__restrict__ srow, uint16_t *__restrict__ sbeg) {
    __shared__ int cnt[16], cur[16], start[17];
    __shared__ unsigned char pats[kSortChunkMax];
    const int q = blockIdx.x, g = blockIdx.y / NCH, c = blockIdx.y % NCH;
    const int k0 = c * KCH, rows = min(KCH, Kp - k0);
    const int t = threadIdx.x;
    if (t < 16) { cnt[t] = 0; cur[t] = 0; }
    __syncthreads();
    for (int r = t; r < rows; r += 128) {
        int pat = 0, any = 0;
        for (int j = 0; j < 4; j++) {
            uint32_t wp = 0, wn = 0;
            for (int p = 0; p < P; p++) {
                const uint32_t *e = ws + ((((size_t)p * G + g) * Kp + k0 + r) * Opad + q * 4 + j) * 2;
                wp |= e[0];
                wn |= e[1];
            }
            if (wn) pat |= 1 << j;
            any |= (wp | wn) != 0;
        }
        pats[r] = any ? (unsigned char)pat : (unsigned char)255;   // 255: contributes nothing, dropped
        if (any) atomicAdd(&cnt[pat], 1);
    }
    __syncthreads();
    const size_t gcq = ((size_t)g * NCH + c) * Q + q;
    if (t == 0) {
        int s = 0;
        for (int b = 0; b < 16; b++) { start[b] = s; s += cnt[b]; }
        start[16] = s;
        for (int b = 0; b < 17; b++) sbeg[gcq * 18 + b] = (uint16_t)start[b];
        sbeg[gcq * 18 + 17] = 0;
    }
    __syncthreads();
    for (int r = t; r < rows; r += 128) {
        const int pat = pats[r];
        if (pat == 255) continue;
        const int slot = start[pat] + atomicAdd(&cur[pat], 1);
        srow[gcq * SL + slot] = (uint16_t)(r * 32);   // uint4 offset of the row in the activation tile
        for (int p = 0; p < P; p++) {
            uint32_t w[4];
            for (int j = 0; j < 4; j++) {
                const uint32_t *e = ws + ((((size_t)p * G + g) * Kp + k0 + r) * Opad + q * 4 + j) * 2;
                w[j] = (pat >> j) & 1 ? e[1] : e[0];
            }
            sw[((size_t)p * G * NCH * Q + gcq) * SL + slot] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

}  // namespace

SortedPlan sorted_plan(const Geometry &g) {
    SortedPlan sp;
    sp.layout = g.Kp >= 64 && g.Opad % 32 == 0;
    sp.eligible = sp.layout && g.M >= 128;
    sp.NCH = (g.Kp + kSortChunkMax - 1) / kSortChunkMax;
    sp.KCH = ((g.Kp + sp.NCH - 1) / sp.NCH + 7) / 8 * 8;   // multiple of 8: the u16 lists are copied 16 bytes at a time
    sp.SL = sp.KCH;
    sp.Q = g.Opad / 4;
    const size_t gcq = (size_t)g.G * sp.NCH * sp.Q;
    sp.sw_bytes = align_up((size_t)g.P * gcq * sp.SL * 16, 256);
    sp.srow_bytes = align_up(gcq * sp.SL * 2, 256);
    sp.sbeg_bytes = align_up(gcq * 18 * 2, 256);
    return sp;
}

int launch_sort_members(const Geometry &g, const uint32_t *wstream, void *sorted, cudaStream_t s) {
    const SortedPlan sp = sorted_plan(g);
    uint4 *sw = (uint4 *)sorted;
    uint16_t *srow = (uint16_t *)((char *)sorted + sp.sw_bytes);
    uint16_t *sbeg = (uint16_t *)((char *)sorted + sp.sw_bytes + sp.srow_bytes);
    sort_members_kernel<<<dim3(sp.Q, g.G * sp.NCH), 128, 0, s>>>(wstream, g.P, g.G, g.Kp, g.Opad, sp.NCH, sp.KCH, sp.SL,
                                                                sp.Q, sw, srow, sbeg);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_accumulate_sorted(const Geometry &g, const uint32_t *astream, const int32_t *aoff, const void *sorted,
                             int32_t *out, cudaStream_t s) {
    const SortedPlan sp = sorted_plan(g);
    SortedParams pr;
    pr.as = astream; pr.aoff = aoff; pr.out = out;
    pr.sw = (const uint4 *)sorted;
    pr.srow = (const uint16_t *)((const char *)sorted + sp.sw_bytes);
    pr.sbeg = (const uint16_t *)((const char *)sorted + sp.sw_bytes + sp.srow_bytes);
    pr.M = (int)g.M; pr.O = g.O; pr.HoWo = g.Ho * g.Wo; pr.Wo = g.Wo; pr.Wp = g.Wp;
    pr.P = g.P; pr.G = g.G; pr.Kp = g.Kp; pr.NCH = sp.NCH; pr.KCH = sp.KCH; pr.SL = sp.SL; pr.Q = sp.Q;
    pr.pack_words = act_pack_words(g);
    pr.img_words = act_img_words(g);
    pr.aoff_mul = act_pixel_stride(g);
    constexpr int NQ = 8;
    const size_t smem = (size_t)sp.KCH * 128 * 4 + (size_t)NQ * sp.SL * 18 + NQ * 36;
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(accumulate_sorted_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)((size_t)kSortChunkMax * 128 * 4 + (size_t)NQ * kSortChunkMax * 18 + NQ * 36)));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    dim3 grid((unsigned)((g.M + 127) / 128), (unsigned)(sp.Q / NQ), 1);
    const long long tiles = (long long)grid.x * grid.y, slots = (long long)sm_count() * 2, pairs = (long long)g.P * g.G;
    long long splits = 1, best = -1;
    for (long long c = 1; c <= pairs && c <= 32; c++) {
        const long long waves = (tiles * c + slots - 1) / slots;
        const long long cost = waves * (((pairs + c - 1) / c) * g.Kp + 24);
        if (best < 0 || cost < best) { best = cost; splits = c; }
    }
    pr.splits = (int)splits;
    grid.z = (unsigned)splits;
    if (splits > 1) GEO_CUDA_CHECK(cudaMemsetAsync(out, 0, (size_t)g.M * g.O * sizeof(int32_t), s));
    accumulate_sorted_kernel<NQ><<<grid, NQ * 32, smem, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

}  // namespace geo
