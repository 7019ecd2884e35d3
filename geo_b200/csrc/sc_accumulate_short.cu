// SC accumulation for short OR groups with one LOP3 per weight: sign-sorted members on im2col tiles.
//
// A weight has a positive or a negative stream, never both (split-unipolar, sc_cuda_kernel.cu:694-1002), so of the
// two AND-OR updates per (activation word, weight) that the dense kernel (sc_accumulate.cu) issues, one works on
// a zero word.  As in the kernels for long groups, the members are sorted, per four output channels (a "quad"),
// by which of the four weights are negative, and each of the 16 patterns is a loop of its own whose 32 LOP3 go to
// the positive or the negative accumulator of each channel; members whose four weights are all zero (the
// padding of a group, zero weights) are dropped from the lists.  What differs is the scale: a stage is one chunk of
// at most 16 members of one group, sorted on its own, so a pattern's loop runs once or twice and what counts is
// that everything around it is cheap -- the pattern bounds of a chunk are 16 bytes read with one load, every
// load carries an explicit 32-bit shared address, and the branches are direct.
//
// A warp owns one quad and 256 positions (a lane: two runs of four), a CTA four quads; tiles are im2col tiles as in
// the dense kernel: 256 positions x KC members per stage, gathered with 4-byte cp.async through the member offset
// table, in a ring of NSTAGE stages.  The running sums of two channels share a register as two 16-bit halves
// where P * G * 32 fits 15 bits, which brings the kernel to 128 registers and four CTAs per SM (else three).
// Each pattern's loop is kept rolled: sixteen unrolled loop bodies do not fit the instruction cache, and with one
// or two members per pattern there is nothing to gain from unrolling.
#include "sc_common.h"
#include "sc_short.h"

namespace geo {

namespace {

constexpr int kShThreads = 128;
constexpr int kShMT = 256;   // positions per CTA
constexpr int kShNT = 16;    // channels per CTA: one quad per warp

struct ShortParams {
    const uint32_t *as;          // [B][P][C][Hp][Wp]
    const uint4 *wl;             // [P][G][NCH][Q][KC]
    const unsigned char *meta;   // [G][NCH][Q][32]
    const int32_t *aoff;         // [G][K]
    int32_t *out;                // [B][O][Ho][Wo]
    int M, O, Q, HoWo, Wo, Wp;
    int P, G, K, NCH;            // K: members per group as laid out
    int img_words, pack_words, pix_stride, Bp;
    int splits, CT;   // CTAs sharing one output tile; channel tiles (of 16)
    uint32_t row_bytes;   // 1024, as a run-time value (see imad)
    int four;   // bytes per unit of the member offset table: 4, times the pixel stride of the stream image
};

__device__ __forceinline__ void cp4(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp16(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
// a * b + c with a run-time b that the compiler cannot fold: an integer multiply-add, which issues on the FMA pipe
// instead of the ALU pipe that the LOP3s use
__device__ __forceinline__ uint32_t imad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// base + 4 * off as one wide multiply-add (FMA pipe) instead of a 64-bit add in two halves (ALU pipe)
__device__ __forceinline__ const uint32_t *word_address(const uint32_t *base, int off, int four) {
    const uint32_t *r;
    asm("mad.wide.s32 %0, %1, %2, %3;\n" : "=l"(r) : "r"(off), "r"(four), "l"(base));
    return r;
}

// One pattern's members: PAT bit j set = the weight of channel j is negative.  ra: shared address of the lane's
// first run of four positions in row 0 of the stage's tile (the second run is 512 bytes on); wl / ol: shared
// addresses of the quad's lists of stream words and of rows; members [i0, i1).
template <int PAT>
__device__ __forceinline__ void run_bucket(uint32_t (&accp)[8][4], uint32_t (&accn)[8][4], uint32_t ra, uint32_t wl,
                                           uint32_t ol, int i0, int i1, uint32_t row_bytes) {
#pragma unroll 1
    for (int i = i0; i < i1; i++) {
        const uint4 w = lds128(wl + i * 16);
        const uint32_t a = imad(lds8(ol + i), row_bytes, ra);
        const uint4 x = lds128(a);
        const uint4 y = lds128(a + 512);
        const uint32_t av[8] = {x.x, x.y, x.z, x.w, y.x, y.y, y.z, y.w};
        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int p = 0; p < 8; p++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (PAT & (1 << j)) accn[p][j] |= av[p] & wv[j];
                else accp[p][j] |= av[p] & wv[j];
            }
    }
}

// PACKED: the running sums of two channels share a register as two 16-bit halves (P*G*32 <= 32767 required)
// POSF: 1x1 images in the batch-innermost stream image -- a member's 256 positions are 1 KB of consecutive words
// and are copied 16 bytes at a time
template <int KC, int NSTAGE, int MINB, bool PACKED, bool POSF>
__global__ void __launch_bounds__(kShThreads, MINB) accumulate_short_kernel(ShortParams pr) {
    constexpr int A_BYTES = KC * 1024, W_BYTES = 4 * KC * 16;
    constexpr int STAGE = A_BYTES + W_BYTES + 4 * kShortMetaBytes;
    extern __shared__ __align__(16) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    // the CTAs that share a position tile (other channels, other pairs) are neighbours in launch order, so that the
    // tile's stream words are fetched from DRAM once and then found in L2
    const int cta_ct = (int)(blockIdx.x % pr.CT), cta_split = (int)((blockIdx.x / pr.CT) % pr.splits);
    const int m0 = (int)(blockIdx.x / (pr.CT * pr.splits)) * kShMT;
    const int q0 = cta_ct * 4;

    // gather: this thread copies columns t and t + 128 of every member row
    int abase[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        int m = m0 + t + j * kShThreads;
        if (m >= pr.M) m = pr.M - 1;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
        abase[j] = b * pr.img_words + ((rem / pr.Wo) * pr.Wp + (rem % pr.Wo)) * pr.pix_stride;
    }
    // POSF: this thread copies positions [pf_base, pf_base + 4) of rows t / 64, t / 64 + 2, ...; a chunk past the
    // padded batch is moved back inside it (its positions are never stored)
    const int pf_base = min(m0 + (t & 63) * 4, pr.Bp - 4);
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    // This CTA owns the (pack, group) pairs [pair0, pair1) of the P*G pairs; the sum over pairs is an integer
    // sum, so splitting it over CTAs and adding atomically is exact and order-free.
    const int pairs = pr.P * pr.G;
    const int pair0 = (int)((long long)pairs * cta_split / pr.splits);
    const int pair1 = (int)((long long)pairs * (cta_split + 1) / pr.splits);
    const int nstages = (pair1 - pair0) * pr.NCH;

    int ld_p = pair0 / pr.G, ld_g = pair0 % pr.G, ld_c = 0, ld_s = 0;
    auto issue_stage = [&]() {
        if (ld_s < nstages) {
            const uint32_t rows = smem_base + (uint32_t)(ld_s % NSTAGE) * STAGE;
            const int32_t *aoff = pr.aoff + ld_g * pr.K + ld_c * KC;
            const uint32_t *asrc = pr.as + (size_t)ld_p * pr.pack_words;
            if (POSF) {
                const uint32_t *s0 = asrc + pf_base;
                const uint32_t d0 = rows + (uint32_t)(t & 63) * 16;
#pragma unroll
                for (int r = 0; r < KC; r += 2)
                    if (r + 1 < KC || t < 64) cp16(d0 + (r + (t >> 6)) * 1024, word_address(s0, __ldg(aoff + r + (t >> 6)), pr.four));
            } else {
                const uint32_t *s0 = asrc + abase[0], *s1 = asrc + abase[1];
                const uint32_t d0 = rows + (uint32_t)t * 4;
#pragma unroll
                for (int r = 0; r < KC; r++) {
                    const int off = __ldg(aoff + r);
                    cp4(d0 + r * 1024, word_address(s0, off, pr.four));
                    cp4(d0 + r * 1024 + 512, word_address(s1, off, pr.four));
                }
            }
            const size_t gcq = ((size_t)ld_g * pr.NCH + ld_c) * pr.Q + q0;   // the CTA's four quads are contiguous
            if (t < 4 * KC) cp16(rows + A_BYTES + t * 16, pr.wl + ((size_t)ld_p * pr.G * pr.NCH * pr.Q + gcq) * KC + t);
            else if (t >= 64 && t < 64 + 4 * kShortMetaBytes / 16)
                cp16(rows + A_BYTES + W_BYTES + (t - 64) * 16, (const uint4 *)(pr.meta + gcq * kShortMetaBytes) + (t - 64));
            ld_s++;
            if (++ld_c == pr.NCH) {
                ld_c = 0;
                if (++ld_g == pr.G) { ld_g = 0; ld_p++; }
            }
        }
        cp_commit();
    };

#pragma unroll
    for (int s = 0; s < NSTAGE - 1; s++) issue_stage();

    uint32_t accp[8][4], accn[8][4];
    uint32_t osum[8][PACKED ? 2 : 4];
#pragma unroll
    for (int i = 0; i < 8; i++) {
#pragma unroll
        for (int j = 0; j < 4; j++) { accp[i][j] = 0; accn[i][j] = 0; }
#pragma unroll
        for (int j = 0; j < (PACKED ? 2 : 4); j++) osum[i][j] = 0;
    }

    int cs_c = 0;   // chunk inside the current group (consumer side)
    for (int s = 0; s < nstages; s++) {
        cp_wait<NSTAGE - 2>();
        __syncthreads();
        issue_stage();   // refills the buffer that stage s - 1 used; every thread is past it

        {
            const uint32_t rows = smem_base + (uint32_t)(s % NSTAGE) * STAGE;
            const uint32_t ra = rows + (uint32_t)lane * 16;
            const uint32_t wl = rows + A_BYTES + (uint32_t)warp * (KC * 16);
            const uint32_t ol = rows + A_BYTES + W_BYTES + (uint32_t)warp * kShortMetaBytes;
            const uint4 e = lds128(ol + 16);   // end slots of the 16 patterns, one byte each
            const uint32_t ew[4] = {e.x, e.y, e.z, e.w};
            int i0 = 0, i1;
#define GEO_BUCKET(B)                                             \
    i1 = (int)((ew[(B) >> 2] >> (8 * ((B) & 3))) & 0xffu);      \
    run_bucket<B>(accp, accn, ra, wl, ol, i0, i1, pr.row_bytes); \
    i0 = i1;
            GEO_BUCKET(0) GEO_BUCKET(1) GEO_BUCKET(2) GEO_BUCKET(3) GEO_BUCKET(4) GEO_BUCKET(5) GEO_BUCKET(6) GEO_BUCKET(7)
            GEO_BUCKET(8) GEO_BUCKET(9) GEO_BUCKET(10) GEO_BUCKET(11) GEO_BUCKET(12) GEO_BUCKET(13) GEO_BUCKET(14) GEO_BUCKET(15)
#undef GEO_BUCKET
        }
        if (++cs_c == pr.NCH) {   // group finished: binary accumulation of its popcounts, accumulators cleared
            cs_c = 0;
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int d = __popc(accp[i][j]) - __popc(accn[i][j]);
                    if (PACKED) osum[i][j >> 1] += (uint32_t)((j & 1) ? d * 65536 : d);
                    else osum[i][j] += (uint32_t)d;
                    accp[i][j] = 0;
                    accn[i][j] = 0;
                }
        }
    }
    cp_wait<0>();

    // store: the lane's positions are m0 + lane*4 + {0..3} and m0 + 128 + lane*4 + {0..3}
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? lane * 4 + i : 128 + lane * 4 + (i - 4));
        if (m < pr.M) {
            const int b = m / pr.HoWo, rem = m % pr.HoWo;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int v;
                if (PACKED) {   // low half sign-extended; the high half is what is left after taking it out
                    const int a = (int)osum[i][j >> 1], lo = (int)(short)(a & 0xffff);
                    v = (j & 1) ? (a - lo) >> 16 : lo;
                } else {
                    v = (int)osum[i][j];
                }
                const int o = (q0 + warp) * 4 + j;
                if (o < pr.O) {
                    int32_t *dst = pr.out + ((size_t)b * pr.O + o) * pr.HoWo + rem;
                    if (pr.splits > 1) atomicAdd(dst, v);
                    else *dst = v;
                }
            }
        }
    }
}

// Preparation: one warp per (group, chunk, quad) sorts the chunk's members by sign pattern, lane r holding member r.
// Reads the dense prepared streams ws[P][G][Kp][Opad][2].
__global__ void __launch_bounds__(128) sort_short_kernel(const uint32_t *__restrict__ ws, uint4 *__restrict__ wl,
                                                         unsigned char *__restrict__ meta, int P, int G, int Kp, int Opad,
                                                         int Q, int KC, int NCH) {
    __shared__ __align__(16) unsigned char ms[4][kShortMetaBytes];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long n = (long long)G * NCH * Q;
    const long long i = (long long)blockIdx.x * 4 + warp;
    if (i >= n) return;   // whole warps leave: no block-wide barrier below
    const int q = (int)(i % Q);
    const int c = (int)((i / Q) % NCH);
    const int g = (int)(i / ((long long)Q * NCH));
    const int r = lane;
    int pt = 16;   // 16: contributes nothing, dropped (lanes past the chunk, members whose four weights are zero)
    if (r < KC) {
        int bits = 0, any = 0;
        for (int j = 0; j < 4; j++) {
            uint32_t wp = 0, wn = 0;
            for (int p = 0; p < P; p++) {
                const uint32_t *e = ws + ((((size_t)p * G + g) * Kp + c * KC + r) * Opad + q * 4 + j) * 2;
                wp |= e[0];
                wn |= e[1];
            }
            if (wn) bits |= 1 << j;
            any |= (wp | wn) != 0;
        }
        if (any) pt = bits;
    }
    // counting sort across the warp: a member's slot = members of smaller patterns + earlier members of its own
    int before = 0, slot = 0;
    uint32_t ends = 0;   // lane b < 16: the slot after pattern b's last member
    for (int b = 0; b < 16; b++) {
        const uint32_t mask = __ballot_sync(0xffffffffu, pt == b);
        if (pt == b) slot = before + __popc(mask & ((1u << lane) - 1u));
        before += __popc(mask);
        if (lane == b) ends = (uint32_t)before;
    }
    const int kept = before;
    if (lane < 16) { ms[warp][lane] = 0; ms[warp][16 + lane] = (unsigned char)ends; }
    __syncwarp();
    if (pt != 16) ms[warp][slot] = (unsigned char)r;
    __syncwarp();
    const size_t base = ((size_t)g * NCH + c) * Q + q;
    if (lane < 2) ((uint4 *)(meta + base * kShortMetaBytes))[lane] = ((const uint4 *)ms[warp])[lane];
    for (int p = 0; p < P; p++) {
        uint4 *dst = wl + ((size_t)p * G * NCH * Q + base) * KC;
        if (pt != 16) {
            const uint32_t *e = ws + ((((size_t)p * G + g) * Kp + c * KC + r) * Opad + q * 4) * 2;
            uint4 v;
            v.x = (pt & 1) ? e[1] : e[0];
            v.y = (pt & 2) ? e[3] : e[2];
            v.z = (pt & 4) ? e[5] : e[4];
            v.w = (pt & 8) ? e[7] : e[6];
            dst[slot] = v;
        }
        if (lane >= kept && lane < KC) dst[lane] = make_uint4(0, 0, 0, 0);   // slots past the members kept
    }
}

template <int KC, int NSTAGE, int MINB, bool PACKED, bool POSF>
int launch_short(const Geometry &g, ShortParams pr, cudaStream_t s) {
    constexpr size_t SMEM = (size_t)NSTAGE * (KC * 1024 + 4 * KC * 16 + 4 * kShortMetaBytes);
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(accumulate_short_kernel<KC, NSTAGE, MINB, PACKED, POSF>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    dim3 grid((unsigned)((g.M + kShMT - 1) / kShMT), (unsigned)(g.Opad / kShNT), 1);
    // CTAs along grid.z share an output tile and split its (pack, group) pairs: the split count that minimises
    // (waves of resident CTAs) x (work of the longest CTA), a CTA's fixed cost put at 12 members' worth of work
    const long long tiles = (long long)grid.x * grid.y, slots = (long long)sm_count() * MINB;
    const long long pairs = (long long)g.P * g.G;
    long long splits = 1, best = -1;
    for (long long c = 1; c <= pairs && c <= 32; c++) {
        const long long waves = (tiles * c + slots - 1) / slots;
        const long long cost = waves * (((pairs + c - 1) / c) * g.Kp + 12);
        if (best < 0 || cost < best) { best = cost; splits = c; }
    }
    pr.splits = (int)splits;
    pr.CT = (int)grid.y;
    if (tiles * splits > 0x7fffffffLL) return fail(GEO_SC_ERR_TOO_LARGE, "%lld x %lld CTAs", tiles, splits);
    grid = dim3((unsigned)(tiles * splits), 1, 1);
    if (splits > 1) GEO_CUDA_CHECK(cudaMemsetAsync(pr.out, 0, (size_t)g.M * g.O * sizeof(int32_t), s));
    accumulate_short_kernel<KC, NSTAGE, MINB, PACKED, POSF><<<grid, kShThreads, SMEM, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

}  // namespace

ShortPlan short_plan(const Geometry &g) {
    ShortPlan sp = {};
    sp.layout = g.mode != GEO_SC_MODE_FULL_BIN && (g.Kp < 64 || g.Opad % 32 != 0);
    // A CTA's tile is 256 positions x 16 channels: with fewer positions the dense kernel's smaller tiles win, and so
    // they do where consecutive positions are not consecutive words of the stream image (images narrower than four
    // columns): there a gathered word costs a memory sector, and the dense tile shares it among up to 64 channels.
    // Linear layers (1x1 images) have the batch-innermost image: their positions are consecutive words.
    sp.eligible = sp.layout && g.M >= 192 && (g.Wo >= 4 || (g.batch_fast && g.Hp * g.Wp == 1));
    sp.KC = g.Kp < 16 ? g.Kp : 16;           // groups are laid out in multiples of 4 (up to 16 members) or of 16
    sp.NCH = g.Kp / sp.KC;
    sp.Q = g.Opad / 4;
    sp.wl_bytes = align_up((size_t)g.P * g.G * sp.NCH * sp.Q * sp.KC * 16, 256);
    sp.meta_bytes = align_up((size_t)g.G * sp.NCH * sp.Q * kShortMetaBytes, 256);
    return sp;
}

int launch_sort_short(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s) {
    const ShortPlan sp = short_plan(g);
    const long long n = (long long)g.G * sp.NCH * sp.Q;
    sort_short_kernel<<<(unsigned)((n + 3) / 4), 128, 0, s>>>(wstream, (uint4 *)section, (unsigned char *)section + sp.wl_bytes, g.P, g.G, g.Kp,
                                             g.Opad, sp.Q, sp.KC, sp.NCH);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_accumulate_short(const Geometry &g, const uint32_t *astream, const int32_t *aoff, const void *section,
                            int32_t *out, cudaStream_t s) {
    const ShortPlan sp = short_plan(g);
    ShortParams pr;
    pr.as = astream; pr.aoff = aoff; pr.out = out;
    pr.wl = (const uint4 *)section;
    pr.meta = (const unsigned char *)section + sp.wl_bytes;
    pr.M = (int)g.M; pr.O = g.O; pr.Q = sp.Q; pr.HoWo = g.Ho * g.Wo; pr.Wo = g.Wo; pr.Wp = g.Wp;
    pr.P = g.P; pr.G = g.G; pr.K = g.Kp; pr.NCH = sp.NCH;
    pr.pack_words = act_pack_words(g);
    pr.img_words = act_img_words(g);
    pr.pix_stride = act_pixel_stride(g);
    pr.Bp = g.Bp;
    pr.splits = 1;
    pr.row_bytes = 1024; pr.four = 4 * act_pixel_stride(g);
    // with packed sums the kernel fits 128 registers: four CTAs per SM instead of three
    const bool packed = (long long)g.P * g.G * 32 <= 32767;
    const int variant = sp.KC * 4 + (packed ? 2 : 0) + (g.batch_fast && g.Hp * g.Wp == 1 ? 1 : 0);
    switch (variant) {
    case 4 * 4 + 0: return launch_short<4, 6, 3, false, false>(g, pr, s);
    case 4 * 4 + 1: return launch_short<4, 6, 3, false, true>(g, pr, s);
    case 4 * 4 + 2: return launch_short<4, 6, 4, true, false>(g, pr, s);
    case 4 * 4 + 3: return launch_short<4, 6, 4, true, true>(g, pr, s);
    case 8 * 4 + 0: return launch_short<8, 6, 3, false, false>(g, pr, s);
    case 8 * 4 + 1: return launch_short<8, 6, 3, false, true>(g, pr, s);
    case 8 * 4 + 2: return launch_short<8, 5, 4, true, false>(g, pr, s);
    case 8 * 4 + 3: return launch_short<8, 5, 4, true, true>(g, pr, s);
    case 12 * 4 + 0: return launch_short<12, 4, 3, false, false>(g, pr, s);
    case 12 * 4 + 1: return launch_short<12, 4, 3, false, true>(g, pr, s);
    case 12 * 4 + 2: return launch_short<12, 4, 4, true, false>(g, pr, s);
    case 12 * 4 + 3: return launch_short<12, 4, 4, true, true>(g, pr, s);
    case 16 * 4 + 0: return launch_short<16, 4, 3, false, false>(g, pr, s);
    case 16 * 4 + 1: return launch_short<16, 4, 3, false, true>(g, pr, s);
    case 16 * 4 + 2: return launch_short<16, 3, 4, true, false>(g, pr, s);
    default: return launch_short<16, 3, 4, true, true>(g, pr, s);
    }
}

}  // namespace geo
