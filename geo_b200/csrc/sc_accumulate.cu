// SC accumulation: out[m][o] = sum over packs p and groups g of
//     popc( OR_k  A[m][g][k][p] & Wpos[g][k][o][p] ) - popc( OR_k A[m][g][k][p] & Wneg[g][k][o][p] )
// where m runs over output positions (b, oy, ox), k over the OR-accumulated members of a
// group and g over the binary-accumulated groups.  Replaces the reference's
// stream_compute_add_direct_variable (sc_cuda_kernel.cu:694-1002) and matmul_outer (:43-86).
//
// Structure: an implicit-GEMM register-tiled kernel.  A CTA owns MT positions x NT output
// channels; a thread owns 8 positions x 4 channels x 2 polarities = 64 OR-accumulators, so
// every activation word loaded from shared memory feeds 8 LOP3 and every weight word 8.
// The reduction is walked as a flat list of stages (pack, group, chunk of KC members); the
// activation words of a stage are gathered from the packed stream image with 4-byte
// cp.async (implicit im2col through the per-member offset table), the weight words with
// 16-byte cp.async, through an NSTAGE-deep ring so that the copies of later stages overlap
// the LOP3 work of the current one.  At the end of each group the 64 accumulators are
// popcounted into 32 int32 sums that stay in registers until the final store.
#include "sc_common.h"

namespace geo {

constexpr int TM = 8;       // positions per thread
constexpr int TN = 4;       // output channels per thread

struct AccParams {
    const uint32_t *as;   // [B][P][C][Hp][Wp]
    const uint32_t *ws;   // [P][G][K][Opad][2]
    const int32_t *aoff;  // [G][K]
    int32_t *out;         // [B][O][Ho][Wo]
    int M, O, Opad, HoWo, Wo, Wp;
    int P, G, K;          // K: members per group as laid out (padded to a multiple of 16)
    int img_words;        // words between images, between packs, between pixels (act_img_words ...): the pixel
    int pack_words;       // stride also scales the member offsets
    int aoff_mul;
    int splits;           // CTAs along grid.z sharing one output tile; > 1 => atomic accumulation
};

__device__ __forceinline__ void cp_async4(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

template <int NT, int NTHREADS, int KC, int NSTAGE>
struct Tile {
    static constexpr int TY = NT / TN;          // thread rows over channels
    static constexpr int TX = NTHREADS / TY;    // thread columns over positions
    static constexpr int MT = TX * TM;          // positions per CTA
    static constexpr int A_WORDS = KC * MT;
    static constexpr int W_WORDS = KC * NT * 2;
    static constexpr int STAGE_WORDS = A_WORDS + W_WORDS;
    static constexpr size_t SMEM = (size_t)NSTAGE * STAGE_WORDS * 4;
    static_assert(TX % 8 == 0 && TY % 4 == 0, "warps are 8 positions x 4 channel rows");
};

template <int NT, int NTHREADS, int KC, int NSTAGE, int MINB>
__global__ void __launch_bounds__(NTHREADS, MINB) accumulate_kernel(AccParams pr) {
    using T = Tile<NT, NTHREADS, KC, NSTAGE>;
    constexpr int MT = T::MT, TX = T::TX;
    extern __shared__ __align__(16) uint32_t smem[];

    const int t = threadIdx.x;
    // A warp covers 8 thread columns x 4 thread rows, so that one 16-byte shared load of a
    // warp touches 8 distinct activation chunks (128 B) or 4 distinct weight chunks.
    const int lane = t & 31, warp = t >> 5;
    constexpr int WX = TX / 8;
    const int tx = (warp % WX) * 8 + (lane & 7);
    const int ty = (warp / WX) * 4 + (lane >> 3);

    const int m0 = blockIdx.x * MT;
    const int o0 = blockIdx.y * NT;

    // ---- gather assignment: this thread copies rows r = r0 + i*RSTEP of column(s) mcol ----
    constexpr int MPT = MT > NTHREADS ? MT / NTHREADS : 1;     // columns per thread
    constexpr int RSTEP = NTHREADS > MT ? NTHREADS / MT : 1;   // rows advanced per pass
    const int r0 = NTHREADS > MT ? t / MT : 0;
    int abase[MPT];
#pragma unroll
    for (int j = 0; j < MPT; j++) {
        const int mcol = (t % MT) + j * NTHREADS;
        int m = m0 + mcol;
        if (m >= pr.M) m = pr.M - 1;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
        abase[j] = b * pr.img_words + ((rem / pr.Wo) * pr.Wp + (rem % pr.Wo)) * pr.aoff_mul;
    }
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    const int chunks = pr.K / KC;   // pr.K is the padded member count, a multiple of KC
    // This CTA owns the (pack, group) pairs [pair0, pair1) of the P*G pairs; the sum over pairs is
    // an integer sum, so splitting it over CTAs and adding atomically is exact and order-free.
    const int pairs = pr.P * pr.G;
    const int pair0 = (int)((long long)pairs * blockIdx.z / pr.splits);
    const int pair1 = (int)((long long)pairs * (blockIdx.z + 1) / pr.splits);
    const int nstages = (pair1 - pair0) * chunks;

    // stage cursor for the producer side
    int ld_p = pair0 / pr.G, ld_g = pair0 % pr.G, ld_c = 0, ld_s = 0;
    auto issue_stage = [&]() {
        if (ld_s < nstages) {
            const int buf = ld_s % NSTAGE;
            const uint32_t a_s = smem_base + (uint32_t)buf * T::STAGE_WORDS * 4;
            const uint32_t w_s = a_s + T::A_WORDS * 4;
            const int k0 = ld_c * KC;
            const int32_t *aoff = pr.aoff + ld_g * pr.K + k0;
            const uint32_t *asrc = pr.as + ld_p * pr.pack_words;
            // The prepared layout pads every group to a multiple of 16 members with all-zero weight
            // streams (and offset 0), so every stage is full: no per-row predicates, and the
            // consumer always runs all KC rows of a stage, fully unrolled.
            constexpr int CPR = NT / 2;                       // 16-byte weight chunks per row
            constexpr int WROWS = NTHREADS / CPR;             // weight rows covered per pass
            static_assert(NTHREADS % CPR == 0, "weight rows are covered by whole passes");
    constexpr int WPASS = (KC + WROWS - 1) / WROWS;
            const uint32_t *wsrc = pr.ws + ((size_t)(ld_p * pr.G + ld_g) * pr.K + k0) * pr.Opad * 2 + o0 * 2 +
                                   (size_t)(t / CPR) * pr.Opad * 2 + (t % CPR) * 4;
            const uint32_t w_dst = w_s + (uint32_t)((t / CPR) * NT * 2 + (t % CPR) * 4) * 4;
#pragma unroll
            for (int j = 0; j < MPT; j++) {
                const uint32_t *src = asrc + abase[j];
                const uint32_t dst = a_s + (uint32_t)((t % MT) + j * NTHREADS + r0 * MT) * 4;
#pragma unroll
                for (int i = 0; i < (KC + RSTEP - 1) / RSTEP; i++)
                    if (KC % RSTEP == 0 || r0 + i * RSTEP < KC)
                        cp_async4(dst + (uint32_t)(i * RSTEP * MT) * 4, src + __ldg(aoff + r0 + i * RSTEP) * pr.aoff_mul);
            }
#pragma unroll
            for (int i = 0; i < WPASS; i++)
                if (KC % WROWS == 0 || t / CPR + i * WROWS < KC)
                    cp_async16(w_dst + (uint32_t)(i * WROWS * NT * 2) * 4, wsrc + (size_t)i * WROWS * pr.Opad * 2);
            ld_s++;
            if (++ld_c == chunks) {
                ld_c = 0;
                if (++ld_g == pr.G) { ld_g = 0; ld_p++; }
            }
        }
        cp_async_commit();
    };

#pragma unroll
    for (int s = 0; s < NSTAGE - 1; s++) issue_stage();

    uint32_t accp[TM][TN], accn[TM][TN];
    int osum[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) { accp[i][j] = 0; accn[i][j] = 0; osum[i][j] = 0; }

    int cs_c = 0;  // chunk index inside the current group (consumer side)
    for (int s = 0; s < nstages; s++) {
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        issue_stage();  // refills the buffer that stage s-1 used; every thread is past it

        const int buf = s % NSTAGE;
        const uint32_t *a_s = smem + (size_t)buf * T::STAGE_WORDS;
        const uint32_t *w_s = a_s + T::A_WORDS;
        const uint4 *a4 = (const uint4 *)a_s + tx;
        const uint4 *w4 = (const uint4 *)w_s + ty * 2;
#pragma unroll
        for (int r = 0; r < KC; r++) {
            const uint4 a_lo = a4[r * (MT / 4)];
            const uint4 a_hi = a4[r * (MT / 4) + MT / 8];
            const uint4 w_a = w4[r * (NT / 2)];
            const uint4 w_b = w4[r * (NT / 2) + 1];
            const uint32_t a[TM] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
            const uint32_t wp[TN] = {w_a.x, w_a.z, w_b.x, w_b.z};
            const uint32_t wn[TN] = {w_a.y, w_a.w, w_b.y, w_b.w};
            if (r == 0 && cs_c == 0) {   // first member of a group starts the OR chains afresh
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < TN; j++) {
                        accp[i][j] = a[i] & wp[j];
                        accn[i][j] = a[i] & wn[j];
                    }
            } else {
#pragma unroll
                for (int i = 0; i < TM; i++)
#pragma unroll
                    for (int j = 0; j < TN; j++) {
                        accp[i][j] |= a[i] & wp[j];
                        accn[i][j] |= a[i] & wn[j];
                    }
            }
        }
        if (++cs_c == chunks) {  // group finished: binary accumulation of its popcounts
            cs_c = 0;
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) osum[i][j] += __popc(accp[i][j]) - __popc(accn[i][j]);
        }
    }
    cp_async_wait<0>();

    // ---- store: thread positions are m0 + tx*4 + {0..3} and m0 + MT/2 + tx*4 + {0..3} ----
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + (i < 4 ? tx * 4 + i : MT / 2 + tx * 4 + (i - 4));
        if (m < pr.M) {
            const int b = m / pr.HoWo, rem = m % pr.HoWo;
#pragma unroll
            for (int j = 0; j < TN; j++) {
                const int o = o0 + ty * TN + j;
                if (o < pr.O) {
                    int32_t *dst = pr.out + ((size_t)b * pr.O + o) * pr.HoWo + rem;
                    if (pr.splits > 1) atomicAdd(dst, osum[i][j]);
                    else *dst = osum[i][j];
                }
            }
        }
    }
}

template <int NT, int NTHREADS, int KC = 16, int NSTAGE = 4, int MINB = 384 / NTHREADS>
static int launch_tile(const Geometry &g, AccParams pr, cudaStream_t s) {
    using T = Tile<NT, NTHREADS, KC, NSTAGE>;
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(accumulate_kernel<NT, NTHREADS, KC, NSTAGE, MINB>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    dim3 grid((unsigned)((g.M + T::MT - 1) / T::MT), (unsigned)(g.Opad / NT), 1);
    // CTAs along grid.z share an output tile and split its (pack, group) pairs.  The split count is
    // the one that minimises (waves of resident CTAs) x (work of the longest CTA), where a CTA's
    // fixed cost (pipeline fill, epilogue) is put at 12 members' worth of work.
    const long long tiles = (long long)grid.x * grid.y, slots = (long long)sm_count() * MINB;
    const long long pairs = (long long)g.P * g.G;
    long long splits = 1, best = -1;
    for (long long c = 1; c <= pairs && c <= 32; c++) {
        const long long waves = (tiles * c + slots - 1) / slots;
        const long long cost = waves * (((pairs + c - 1) / c) * g.Kp + 12);
        if (best < 0 || cost < best) { best = cost; splits = c; }
    }
    pr.splits = (int)splits;
    grid.z = (unsigned)splits;
    if (splits > 1) GEO_CUDA_CHECK(cudaMemsetAsync(pr.out, 0, (size_t)g.M * g.O * sizeof(int32_t), s));
    accumulate_kernel<NT, NTHREADS, KC, NSTAGE, MINB><<<grid, NTHREADS, T::SMEM, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_accumulate(const Geometry &g, const uint32_t *astream, const uint32_t *wstream, const int32_t *aoff,
                      int32_t *out, cudaStream_t s) {
    AccParams pr;
    pr.as = astream; pr.ws = wstream; pr.aoff = aoff; pr.out = out;
    pr.M = (int)g.M; pr.O = g.O; pr.Opad = g.Opad; pr.HoWo = g.Ho * g.Wo; pr.Wo = g.Wo; pr.Wp = g.Wp;
    pr.P = g.P; pr.G = g.G; pr.K = g.Kp;
    pr.pack_words = act_pack_words(g);
    pr.img_words = act_img_words(g);
    pr.aoff_mul = act_pixel_stride(g);
    pr.splits = 1;
    // Long groups use 32-member stages (half as many barriers per LOP3); short ones 16-member
    // stages, because a stage is always executed in full and its zero-filled tail rows are wasted.
    const bool long_groups = g.Kp >= 64 && g.Kp % 32 == 0;
    if (g.Kp < 16) {   // short groups: one stage per group, 4 / 8 / 12 members
        switch (g.NT * 100 + g.Kp) {
        case 1604: return launch_tile<16, 128, 4, 6>(g, pr, s);
        case 1608: return launch_tile<16, 128, 8, 6>(g, pr, s);
        case 1612: return launch_tile<16, 128, 12, 4>(g, pr, s);
        case 3204: return launch_tile<32, 128, 4, 6>(g, pr, s);
        case 3208: return launch_tile<32, 128, 8, 6>(g, pr, s);
        case 3212: return launch_tile<32, 128, 12, 4>(g, pr, s);
        case 6404: return launch_tile<64, 128, 4, 6>(g, pr, s);
        case 6408: return launch_tile<64, 128, 8, 6>(g, pr, s);
        default: return launch_tile<64, 128, 12, 4>(g, pr, s);
        }
    }
    switch (g.NT) {
    case 16:   // small launches: one-warp and two-warp CTAs, so that a few hundred positions still spread over the SMs
        if (g.M <= 512) return launch_tile<16, 32, 16, 4, 12>(g, pr, s);
        return g.M <= 2048 ? launch_tile<16, 64>(g, pr, s) : launch_tile<16, 128>(g, pr, s);
    case 32: return long_groups ? launch_tile<32, 128, 32, 3>(g, pr, s) : launch_tile<32, 128>(g, pr, s);
    default: return long_groups ? launch_tile<64, 128, 32, 3>(g, pr, s) : launch_tile<64, 128>(g, pr, s);
    }
}

}  // namespace geo
