// SC accumulation, sign-sorted members on row tiles: the kernel for long OR groups on images whose width
// is a multiple of four.
//
// Like sc_accumulate_sorted.cu, the members of a group are sorted, per four output channels (a "quad"), by
// which of the four weights are negative, so that an activation word meets one LOP3 per channel instead of
// one per channel and polarity.  Three things differ:
//
//  * The activation tile is not an im2col tile.  A CTA owns whole output rows (512 or 256 positions); for each
//    (channel, filter column) it holds one "plane" -- the tile's rows plus K2 - 1 halo rows per image -- and the
//    K2 members that differ only in the filter row read it at K2 row offsets.  The tile is K2 x smaller (per
//    member) than an im2col tile, a whole group of the CNN layers fits in one stage, and the gather is a tenth of
//    the copy instructions.
//  * A lane owns eight positions (two runs of four output columns) x four channels: 32 LOP3 per member for
//    one 16-byte load of the member's stream words, one 4-byte load of its tile offset and two 16-byte loads of
//    activation words -- twice the logic ops per list load of the four-position form.
//  * One persistent CTA per SM (16 warps) walks a contiguous range of (position tile, channel tile, pack, group)
//    items through a two-stage cp.async pipeline: the copies of the next stage are in flight while the current
//    one is computed, within the CTA, and there are no waves to quantise.  The popcounts of an item are kept
//    in registers (two 16-bit sums per register) until the CTA leaves the tile, then added to the output.
#include "sc_common.h"
#include "sc_rows.h"

namespace geo {

namespace {

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

struct RowsParams {
    const uint32_t *as;     // [B][P][C][Hp][Wp]
    const uint4 *sw;        // [P][G][NCH][Q][SL]: the four non-zero stream words of a sorted member
    const uint32_t *soff;   // [G][NCH][Q][SL]: byte offset of the member's origin in the stage's activation tile
    const uint16_t *sbeg;   // [G][NCH][Q][24]: first slot of each of the 16 patterns, then the end
    const int32_t *pgoff;   // [G][NCH][NPL]: word offset of the plane's origin in a padded image of one pack
    int32_t *out;           // [B][O][Ho][Wo]
    int B, O, Ho, Wo, Wp, HoWo;
    int P, G, NCH, SL, NPL, Q, CT;
    int UCH, PU, units;
    int CG, H, PL, NS;
    int img_words, pack_words;
    int stage_bytes, a_bytes;
    int pairs;
    uint32_t one;   // 1, as a run-time value (see add_on_fma_pipe)
    long long n_items;
};

// Shared-memory loads with explicit 32-bit shared-space addresses: the inner loop is all address arithmetic and
// loads around the LOP3s, and generic 64-bit pointers would triple the integer instructions per member.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}

// base + off computed as a multiply-add by a run-time one: the integer multiply-add issues on the FMA pipe, which
// this kernel leaves idle, instead of the ALU pipe that the LOP3s saturate.
__device__ __forceinline__ uint32_t add_on_fma_pipe(uint32_t off, uint32_t one, uint32_t base) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(off), "r"(one), "r"(base));
    return r;
}

// One pattern's members: PAT bit j set = the weight of channel j is negative.  a_lo / a_hi: shared address of the
// lane's two runs of four positions in plane 0, row 0; sw / so: shared addresses of the quad's stream-word and
// offset lists; members [i0, i1) of the lists.  Every load carries an explicit 32-bit shared address (the list walk
// through generic pointers cost 6 % of the kernel on the second conv of the CNN); the loop is unrolled twice
// (once: 12 % slower, four times: registers spill).
template <int PAT>
__device__ __forceinline__ void run_bucket(uint32_t (&accp)[8][4], uint32_t (&accn)[8][4], uint32_t a_lo, uint32_t a_hi,
                                           uint32_t sw, uint32_t so, int i0, int i1, uint32_t one) {
#pragma unroll 2
    for (int i = i0; i < i1; i++) {
        const uint4 w = lds128(sw + (uint32_t)i * 16);
        const uint32_t on = lds32(so + (uint32_t)i * 4);
        const uint4 x = lds128(add_on_fma_pipe(on, one, a_lo));
        const uint4 y = lds128(add_on_fma_pipe(on, one, a_hi));
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

template <int NQ>
__global__ void __launch_bounds__(kRowsThreads, 1) accumulate_rows_kernel(RowsParams pr) {
    constexpr int NH = 16 / NQ;
    constexpr int TRQ = 64 * NH;   // row-quads of a position tile
    extern __shared__ __align__(16) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int ql = warp % NQ, h = warp / NQ;
    const long long i0 = pr.n_items * blockIdx.x / gridDim.x;
    const long long i1 = pr.n_items * (blockIdx.x + 1) / gridDim.x;
    if (i0 >= i1) return;
    const int nstages = (int)(i1 - i0) * pr.NCH;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const int sw_off = pr.a_bytes, so_off = sw_off + NQ * pr.SL * 16, sb_off = so_off + NQ * pr.SL * 4;

    // ---- producer side: the words of a plane that this thread copies, for the producer's position tile ----
    int prod_ptile = -1, nslots = 0;   // nslots: how many of this thread's slots hold a word of the tile
    int goff[kRowsGatherSlots];     // word offset in the stream image of one pack (image, row, column), -1: none
    auto set_gather_slots = [&](int ptile) {
        prod_ptile = ptile;
        const int u0 = ptile * TRQ;
        const int rho0 = u0 / pr.CG, rho1 = (u0 + TRQ - 1) / pr.CG;
        const int b0 = rho0 / pr.Ho, b1 = rho1 / pr.Ho;
        const int words = ((rho1 - rho0 + 1) + (b1 - b0 + 1) * pr.H) * pr.Wo;
#pragma unroll
        for (int s = 0; s < kRowsGatherSlots; s++) {
            goff[s] = -1;
            const int j = t + kRowsThreads * s;
            if (s < pr.NS && j < words) {
                const int sr = j / pr.Wo, col = j - sr * pr.Wo;
                int base = 0;
                for (int b = b0; b <= b1; b++) {
                    const int lo = max(rho0, b * pr.Ho), hi = min(rho1, (b + 1) * pr.Ho - 1);
                    const int rows = hi - lo + 1 + pr.H;
                    if (sr < base + rows) {
                        const int y = (lo - b * pr.Ho) + (sr - base);
                        goff[s] = min(b, pr.B - 1) * pr.img_words + y * pr.Wp + col;
                        break;
                    }
                    base += rows;
                }
            }
        }
        nslots = 0;
#pragma unroll
        for (int s = 0; s < kRowsGatherSlots; s++) nslots += goff[s] >= 0;
    };

    auto produce = [&](int s) {
        const long long item = i0 + s / pr.NCH;
        const int chunk = s % pr.NCH;
        const int tt = (int)(item / pr.pairs), pair = (int)(item % pr.pairs);
        const int ptile = tt / pr.CT, ctile = tt % pr.CT;
        const int p = pair / pr.G, g = pair % pr.G;
        if (ptile != prod_ptile) set_gather_slots(ptile);
        const uint32_t dst = smem_base + (uint32_t)(s & 1) * pr.stage_bytes;
        const int gc = g * pr.NCH + chunk;
        const int npl = min(pr.UCH, pr.units - chunk * pr.UCH) * pr.PU;
        const uint32_t *src = pr.as + (size_t)p * pr.pack_words;
        const int32_t *pg = pr.pgoff + (size_t)gc * pr.NPL;
        uint32_t dp = dst + (uint32_t)t * 4;
        for (int pl = 0; pl < npl; pl++, dp += (uint32_t)pr.PL * 4) {
            const uint32_t *sp = src + __ldg(pg + pl);
#pragma unroll
            for (int k = 0; k < kRowsGatherSlots; k++)   // slots past the tile's words (goff < 0) are the last ones
                if (k < nslots) cp4(dp + k * kRowsThreads * 4, sp + goff[k]);
        }
        // the NQ quads' lists are contiguous
        const size_t gcq = (size_t)gc * pr.Q + ctile * NQ;
        const uint4 *wsrc = pr.sw + ((size_t)p * pr.G * pr.NCH * pr.Q + gcq) * pr.SL;
        for (int i = t; i < NQ * pr.SL; i += kRowsThreads) cp16(dst + sw_off + (uint32_t)i * 16, wsrc + i);
        const uint4 *osrc = (const uint4 *)(pr.soff + gcq * pr.SL);
        for (int i = t; i < NQ * pr.SL / 4; i += kRowsThreads) cp16(dst + so_off + (uint32_t)i * 16, osrc + i);
        if (t < NQ * 3) cp16(dst + sb_off + (uint32_t)t * 16, (const uint4 *)(pr.sbeg + gcq * 24) + t);
    };

    // ---- consumer side ----
    uint32_t accp[8][4], accn[8][4];
    int sumA[8], sumB[8];   // per position: channels 0,1 and 2,3 of the quad as two 16-bit sums each
    int cons_tt = -1, cons_ptile = -1;
    uint32_t lane_off[2] = {0, 0};
    int out_base[2] = {-1, -1};   // index of (b, channel 0, oy, 4*cg) in the output, -1: outside the batch

    auto flush = [&]() {
        if (cons_tt < 0) return;
        const int ctile = cons_tt % pr.CT;
        const bool exclusive = (long long)cons_tt * pr.pairs >= i0 && (long long)(cons_tt + 1) * pr.pairs <= i1;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            if (out_base[r] < 0) continue;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int a = sumA[r * 4 + i], b = sumB[r * 4 + i];
                const int a0 = (int)(short)(a & 0xffff), b0 = (int)(short)(b & 0xffff);
                const int v[4] = {a0, (a - a0) >> 16, b0, (b - b0) >> 16};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int o = (ctile * NQ + ql) * 4 + j;
                    if (o < pr.O) {
                        int32_t *dst = pr.out + (size_t)out_base[r] + (size_t)o * pr.HoWo + i;
                        if (exclusive) *dst = v[j];
                        else atomicAdd(dst, v[j]);
                    }
                }
            }
        }
    };

    auto set_lane_positions = [&](int ptile) {
        cons_ptile = ptile;
        const int u0 = ptile * TRQ;
        const int rho0 = u0 / pr.CG, b0 = rho0 / pr.Ho;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int u = u0 + h * 64 + lane + 32 * r;
            const int rho = u / pr.CG, cg = u - rho * pr.CG;
            const int b = rho / pr.Ho, oy = rho - b * pr.Ho;
            const int sr = (rho - rho0) + (b - b0) * pr.H;
            lane_off[r] = (uint32_t)(sr * pr.Wo + cg * 4) * 4;
            out_base[r] = b < pr.B ? (b * pr.O * pr.Ho + oy) * pr.Wo + cg * 4 : -1;
        }
    };

    produce(0);
    cp_commit();
    for (int s = 0; s < nstages; s++) {
        if (s + 1 < nstages) produce(s + 1);   // its buffer was read last at stage s - 1; every warp is past that
        cp_commit();
        cp_wait<1>();
        __syncthreads();

        const long long item = i0 + s / pr.NCH;
        const int chunk = s % pr.NCH;
        const int tt = (int)(item / pr.pairs);
        if (tt != cons_tt) {
            flush();
            cons_tt = tt;
            if (tt / pr.CT != cons_ptile) set_lane_positions(tt / pr.CT);
#pragma unroll
            for (int i = 0; i < 8; i++) { sumA[i] = 0; sumB[i] = 0; }
        }
        if (chunk == 0) {
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) { accp[i][j] = 0; accn[i][j] = 0; }
        }
        {
            const uint32_t stage = smem_base + (uint32_t)(s & 1) * pr.stage_bytes;
            const uint32_t a_lo = stage + lane_off[0], a_hi = stage + lane_off[1];
            const unsigned char *stage_ptr = smem + (size_t)(s & 1) * pr.stage_bytes;
            const uint32_t swl = stage + (uint32_t)sw_off + (uint32_t)(ql * pr.SL) * 16;
            const uint32_t sol = stage + (uint32_t)so_off + (uint32_t)(ql * pr.SL) * 4;
            const uint16_t *sbl = (const uint16_t *)(smem + (size_t)(s & 1) * pr.stage_bytes + sb_off) + ql * 24;
            // lane b holds the first slot of pattern b; the loops get their bounds by shuffle
            const int mybeg = lane < 17 ? (int)sbl[lane] : 0;
#define GEO_BUCKET(B) \
    run_bucket<B>(accp, accn, a_lo, a_hi, swl, sol, __shfl_sync(0xffffffffu, mybeg, B), __shfl_sync(0xffffffffu, mybeg, B + 1), pr.one);
            GEO_BUCKET(0) GEO_BUCKET(1) GEO_BUCKET(2) GEO_BUCKET(3) GEO_BUCKET(4) GEO_BUCKET(5) GEO_BUCKET(6) GEO_BUCKET(7)
            GEO_BUCKET(8) GEO_BUCKET(9) GEO_BUCKET(10) GEO_BUCKET(11) GEO_BUCKET(12) GEO_BUCKET(13) GEO_BUCKET(14) GEO_BUCKET(15)
#undef GEO_BUCKET
        }
        if (chunk == pr.NCH - 1) {   // the group is complete: binary accumulation of its popcounts
#pragma unroll
            for (int i = 0; i < 8; i++) {
                sumA[i] += (__popc(accp[i][0]) - __popc(accn[i][0])) + (__popc(accp[i][1]) - __popc(accn[i][1])) * 65536;
                sumB[i] += (__popc(accp[i][2]) - __popc(accn[i][2])) + (__popc(accp[i][3]) - __popc(accn[i][3])) * 65536;
            }
        }
        __syncthreads();   // every warp is done with this stage's buffer before the next produce() refills it
    }
    cp_wait<0>();
    flush();
}

// ---- preparation: sort the members of every (group, chunk) per channel quad ---------------------------
// Reads the dense prepared streams ws[P][G][Kp][Opad][2].  One CTA per (quad, group * chunk).
struct SortRowsParams {
    const uint32_t *ws;
    uint4 *sw;
    uint32_t *soff;
    uint16_t *sbeg;
    int32_t *pgoff;
    int P, G, K, Kp, Opad, Q;
    int mode, C, K2, K3, z, Hp, Wp, Wo;
    int U, PU, units, UCH, NCH, SL, NPL, PL;
};

// Filter coordinates of member k of group g, the member's unit and its plane inside the unit.
__device__ __forceinline__ void decode_member(const SortRowsParams &sp, int g, int k, int *c, int *ky, int *kx, int *un,
                                              int *pin) {
    switch (sp.mode) {
    case GEO_SC_MODE_1D: *kx = g; *c = k / sp.K2; *ky = k % sp.K2; *un = *c; *pin = 0; break;
    case GEO_SC_MODE_Z: *c = g; *ky = k / sp.K3; *kx = k % sp.K3; *un = 0; *pin = *kx; break;
    case GEO_SC_MODE_YZ: {
        const int cz = k / sp.K2;
        *kx = g % sp.K3;
        *c = (g / sp.K3) * sp.z + cz;
        *ky = k % sp.K2;
        *un = cz;
        *pin = 0;
        break;
    }
    case GEO_SC_MODE_2D: *ky = g / sp.K3; *kx = g % sp.K3; *c = k; *un = k; *pin = 0; break;
    default: *c = k / (sp.K2 * sp.K3); *ky = (k / sp.K3) % sp.K2; *kx = k % sp.K3; *un = *c; *pin = *kx; break;
    }
}

__global__ void __launch_bounds__(128) sort_rows_kernel(SortRowsParams sp) {
    __shared__ int cnt[16], cur[16], start[17];
    __shared__ unsigned char pats[kRowsSlotsMax];
    const int q = blockIdx.x, g = blockIdx.y / sp.NCH, ch = blockIdx.y % sp.NCH;
    const int un0 = ch * sp.UCH;
    const int k0 = un0 * sp.U, k1 = min(min(un0 + sp.UCH, sp.units) * sp.U, sp.K);
    const int rows = k1 - k0;
    const int t = threadIdx.x;
    if (t < 16) { cnt[t] = 0; cur[t] = 0; }
    __syncthreads();
    for (int r = t; r < rows; r += 128) {
        int pat = 0, any = 0;
        for (int j = 0; j < 4; j++) {
            uint32_t wp = 0, wn = 0;
            for (int p = 0; p < sp.P; p++) {
                const uint32_t *e = sp.ws + ((((size_t)p * sp.G + g) * sp.Kp + k0 + r) * sp.Opad + q * 4 + j) * 2;
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
    const size_t gc = (size_t)g * sp.NCH + ch;
    const size_t gcq = gc * sp.Q + q;
    if (t == 0) {
        int s = 0;
        for (int b = 0; b < 16; b++) { start[b] = s; s += cnt[b]; }
        start[16] = s;
        for (int b = 0; b < 17; b++) sp.sbeg[gcq * 24 + b] = (uint16_t)start[b];
        for (int b = 17; b < 24; b++) sp.sbeg[gcq * 24 + b] = 0;
    }
    __syncthreads();
    // slots past the members kept hold zero words and offset 0: whatever reads them by mistake adds nothing
    for (int sl = start[16] + t; sl < sp.SL; sl += 128) {
        sp.soff[gcq * sp.SL + sl] = 0;
        for (int p = 0; p < sp.P; p++)
            sp.sw[((size_t)p * sp.G * sp.NCH * sp.Q + gcq) * sp.SL + sl] = make_uint4(0, 0, 0, 0);
    }
    for (int r = t; r < rows; r += 128) {
        int c, ky, kx, un, pin;
        decode_member(sp, g, k0 + r, &c, &ky, &kx, &un, &pin);
        const int plane = (un - un0) * sp.PU + pin;
        // the quad of the first channels also records where each plane of the chunk starts in the stream image
        // (its first member: filter row 0; in 2d_bin a plane has one member, of the group's filter row, and the
        // plane still starts at row 0 -- the member's offset carries the row)
        if (q == 0 && (ky == 0 || sp.mode == GEO_SC_MODE_2D))
            sp.pgoff[gc * sp.NPL + plane] = c < sp.C ? c * sp.Hp * sp.Wp + kx : 0;
        const int pat = pats[r];
        if (pat == 255) continue;
        const int slot = start[pat] + atomicAdd(&cur[pat], 1);
        sp.soff[gcq * sp.SL + slot] = (uint32_t)(plane * sp.PL + ky * sp.Wo) * 4u;
        for (int p = 0; p < sp.P; p++) {
            uint32_t w[4];
            for (int j = 0; j < 4; j++) {
                const uint32_t *e = sp.ws + ((((size_t)p * sp.G + g) * sp.Kp + k0 + r) * sp.Opad + q * 4 + j) * 2;
                w[j] = (pat >> j) & 1 ? e[1] : e[0];
            }
            sp.sw[((size_t)p * sp.G * sp.NCH * sp.Q + gcq) * sp.SL + slot] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

}  // namespace

RowsPlan rows_plan(const Geometry &g) {
    RowsPlan rp = {};
    rp.layout = false;
    rp.eligible = false;
    if (g.Kp < 64 || g.Opad % 32 != 0 || g.Wo % 4 != 0) return rp;
    switch (g.mode) {
    case GEO_SC_MODE_1D: rp.U = g.K2; rp.PU = 1; rp.units = g.C; break;
    case GEO_SC_MODE_YZ: rp.U = g.K2; rp.PU = 1; rp.units = g.z; break;
    case GEO_SC_MODE_FULL_OR: rp.U = g.K2 * g.K3; rp.PU = g.K3; rp.units = g.C; break;
    case GEO_SC_MODE_2D: rp.U = 1; rp.PU = 1; rp.units = g.C; break;
    case GEO_SC_MODE_Z: rp.U = g.K2 * g.K3; rp.PU = g.K3; rp.units = 1; break;
    default: return rp;
    }
    if ((long long)g.P * g.G * 32 > 32767) return rp;   // the 16-bit running sums of a tile must hold P*G*32
    rp.NQ = g.Opad % 64 == 0 ? 16 : 8;
    rp.NH = 16 / rp.NQ;
    rp.Q = g.Opad / 4;
    rp.CG = g.Wo / 4;
    rp.H = g.K2 - 1;
    // rows of a plane in shared memory, at most, over every phase of a tile's first row against the image rows
    const int trq = 64 * rp.NH;
    const long long period = (long long)g.Ho * rp.CG;
    int rt = 0;
    for (long long ti = 0; ti < period && ti < 4096; ti++) {
        const long long u0 = ti * trq;
        const long long rho0 = u0 / rp.CG, rho1 = (u0 + trq - 1) / rp.CG;
        const long long b0 = rho0 / g.Ho, b1 = rho1 / g.Ho;
        const long long rows = (rho1 - rho0 + 1) + (b1 - b0 + 1) * rp.H;
        if (rows > rt) rt = (int)rows;
    }
    rp.RT = rt;
    rp.PL = rt * g.Wo;
    rp.NS = (rp.PL + kRowsThreads - 1) / kRowsThreads;
    if (rp.NS > kRowsGatherSlots) return rp;
    // units per chunk: as many as two pipeline stages hold
    auto stage_bytes = [&](int uch) {
        const size_t sl = (size_t)((uch * rp.U + 3) / 4 * 4);
        return (size_t)uch * rp.PU * rp.PL * 4 + (size_t)rp.NQ * sl * 20 + (size_t)rp.NQ * 48;
    };
    int uch = 0;
    while (uch < rp.units && 2 * stage_bytes(uch + 1) <= kRowsSmemBudget && (uch + 1) * rp.U <= kRowsSlotsMax) uch++;
    if (uch < 1) return rp;
    rp.NCH = (rp.units + uch - 1) / uch;
    rp.UCH = (rp.units + rp.NCH - 1) / rp.NCH;
    // A chunk is sorted into 16 patterns and every pattern is a loop of its own: with few members per pattern the
    // loops' fixed costs show.  Where planes are not shared between members (2d_bin: one member per plane) a
    // stage holds 64 members and the im2col form (160 per chunk) is the faster one (largest layer: 29.6 against
    // 42.7 ms); at 96 members per chunk (3x3 filters, 64 channels in two chunks) the row form is 7 % ahead.
    if (rp.NCH > 1 && rp.UCH * rp.U < 96) return rp;
    rp.SL = (rp.UCH * rp.U + 3) / 4 * 4;
    rp.NPL = rp.UCH * rp.PU;
    rp.stage_bytes = stage_bytes(rp.UCH);
    const size_t gc = (size_t)g.G * rp.NCH, gcq = gc * rp.Q;
    rp.sw_bytes = align_up((size_t)g.P * gcq * rp.SL * 16, 256);
    rp.soff_bytes = align_up(gcq * rp.SL * 4, 256);
    rp.sbeg_bytes = align_up(gcq * 24 * 2, 256);
    rp.pgoff_bytes = align_up(gc * rp.NPL * 4, 256);
    rp.layout = true;
    rp.eligible = g.M >= 256LL * rp.NH;
    return rp;
}

int launch_sort_rows(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s) {
    const RowsPlan rp = rows_plan(g);
    SortRowsParams sp;
    sp.ws = wstream;
    sp.sw = (uint4 *)section;
    sp.soff = (uint32_t *)((char *)section + rp.sw_bytes);
    sp.sbeg = (uint16_t *)((char *)section + rp.sw_bytes + rp.soff_bytes);
    sp.pgoff = (int32_t *)((char *)section + rp.sw_bytes + rp.soff_bytes + rp.sbeg_bytes);
    sp.P = g.P; sp.G = g.G; sp.K = g.K; sp.Kp = g.Kp; sp.Opad = g.Opad; sp.Q = rp.Q;
    sp.mode = g.mode; sp.C = g.C; sp.K2 = g.K2; sp.K3 = g.K3; sp.z = g.z; sp.Hp = g.Hp; sp.Wp = g.Wp; sp.Wo = g.Wo;
    sp.U = rp.U; sp.PU = rp.PU; sp.units = rp.units; sp.UCH = rp.UCH; sp.NCH = rp.NCH; sp.SL = rp.SL; sp.NPL = rp.NPL;
    sp.PL = rp.PL;
    // planes of a last, shorter chunk that no member names keep offset 0 (never read: the kernel copies only
    // the planes of the units a chunk has)
    GEO_CUDA_CHECK(cudaMemsetAsync(sp.pgoff, 0, rp.pgoff_bytes, s));
    sort_rows_kernel<<<dim3(rp.Q, g.G * rp.NCH), 128, 0, s>>>(sp);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

template <int NQ>
static int launch_rows(const Geometry &g, const RowsPlan &rp, RowsParams pr, cudaStream_t s) {
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(accumulate_rows_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)kRowsSmemBudget));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    const long long ctas = pr.n_items < sm_count() ? pr.n_items : sm_count();
    GEO_CUDA_CHECK(cudaMemsetAsync(pr.out, 0, (size_t)g.M * g.O * sizeof(int32_t), s));
    accumulate_rows_kernel<NQ><<<(unsigned)ctas, kRowsThreads, 2 * rp.stage_bytes, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_accumulate_rows(const Geometry &g, const uint32_t *astream, const void *section, int32_t *out,
                           cudaStream_t s) {
    const RowsPlan rp = rows_plan(g);
    RowsParams pr;
    pr.as = astream; pr.out = out;
    pr.sw = (const uint4 *)section;
    pr.soff = (const uint32_t *)((const char *)section + rp.sw_bytes);
    pr.sbeg = (const uint16_t *)((const char *)section + rp.sw_bytes + rp.soff_bytes);
    pr.pgoff = (const int32_t *)((const char *)section + rp.sw_bytes + rp.soff_bytes + rp.sbeg_bytes);
    pr.B = g.B; pr.O = g.O; pr.Ho = g.Ho; pr.Wo = g.Wo; pr.Wp = g.Wp; pr.HoWo = g.Ho * g.Wo;
    pr.P = g.P; pr.G = g.G; pr.NCH = rp.NCH; pr.SL = rp.SL; pr.NPL = rp.NPL; pr.Q = rp.Q; pr.CT = rp.Q / rp.NQ;
    pr.UCH = rp.UCH; pr.PU = rp.PU; pr.units = rp.units;
    pr.CG = rp.CG; pr.H = rp.H; pr.PL = rp.PL; pr.NS = rp.NS;
    pr.pack_words = g.C * g.Hp * g.Wp;
    pr.img_words = g.P * pr.pack_words;
    pr.stage_bytes = (int)rp.stage_bytes;
    pr.a_bytes = rp.NPL * rp.PL * 4;
    pr.pairs = g.P * g.G;
    pr.one = 1;
    const long long total_rq = (long long)g.B * g.Ho * rp.CG;
    const long long ptiles = (total_rq + 64 * rp.NH - 1) / (64 * rp.NH);
    pr.n_items = ptiles * pr.CT * pr.pairs;
    return rp.NQ == 16 ? launch_rows<16>(g, rp, pr, s) : launch_rows<8>(g, rp, pr, s);
}

}  // namespace geo
