// SC accumulation, sign-sorted members on tap tiles: the kernel for long OR groups over many channels (>= 64) in
// 1d_bin, full_or and 2d_bin.
//
// The inner loops are those of sc_accumulate_rows.cu -- members sorted per channel quad by the signs of the four
// weights, one loop per pattern, one LOP3 per weight, eight positions x four channels per lane, a persistent
// 512-thread CTA per SM with a two-stage cp.async pipeline.  What differs is what a position tile is.  The stream
// image is batch-innermost ([pack][c][Hp][Wp][Bp]), and a lane's run of four positions is four consecutive images
// at ONE output pixel, so:
//
//  * the activation words that a member (c, ky, kx) needs for a run are four consecutive words of the image: a
//    member's row of a tile is copied with 16-byte cp.async, one per run, with no halo and no im2col buffer;
//  * the runs of a tile share a border class (the pixels are walked in border-class order), and a filter tap that
//    falls outside the image for that class meets only the all-zero streams of the padding: its chunks are skipped
//    outright.  With 3x3 filters and padding 1 that is 56 % of the work on 2x2 images, 31 % on 4x4, 16 % on 8x8
//    (5x5, padding 2: 28 % on 8x8) -- work that the other kernels spend on ANDs with zero words.  Skipping it is
//    exact.  Tiles that mix classes (small batches) take the union of their pixels' live taps.
//
// A group's members are walked tap by tap, the channels of a tap in chunks (sc_taps.h); a chunk is one pipeline
// stage: its members' rows (1 KB per member and 256 positions) and the quads' sorted lists.  Because tiles cost
// different amounts, the CTAs' contiguous item ranges are cut by live-chunk count, on the host, and travel as
// kernel arguments.
#include <algorithm>
#include <map>
#include <vector>

#include "sc_common.h"
#include "sc_taps.h"

namespace geo {

namespace {

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
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
// base + off as a multiply-add by a run-time one: issues on the FMA pipe instead of the ALU pipe of the LOP3s
__device__ __forceinline__ uint32_t add_on_fma_pipe(uint32_t off, uint32_t one, uint32_t base) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(off), "r"(one), "r"(base));
    return r;
}

struct TapsStarts {
    int n;                           // CTAs
    long long item[kTapsMaxCtas + 1];   // CTA b owns items [item[b], item[b + 1])
};

struct TapsParams {
    const uint32_t *as;     // [P][C][Hp][Wp][Bp]
    const uint4 *sw;        // [P][G][NCH][Q][SL]: the four non-zero stream words of a sorted member
    const uint32_t *soff;   // [G][NCH][Q][SL]: byte offset of the member's row in the stage's tile
    const uint16_t *sbeg;   // [G][NCH][Q][24]: first slot of each of the 16 patterns, then the end
    const int32_t *moff;    // [G][NCH][UCH]: word offset of the member in a padded image of one pack (one image)
    const uint32_t *pix;    // [Ho*Wo]: output pixels (oy << 16 | ox) in border-class order
    int32_t *out;           // [B][O][Ho][Wo]
    int B, Bp, Bq, O, Ho, Wo, Wp, HoWo, H, W;
    int K2, K3, pad_h, pad_w, mode;
    int P, G, NCH, NCS, UCH, C, SL, Q, CT;
    int pack_words, stage_bytes, a_bytes, row_bytes;
    int pairs;
    long long NR;           // runs in all: Ho * Wo * Bq
    uint32_t one;
};

// One pattern's members: PAT bit j set = the weight of channel j is negative.  a_lo: shared address of the lane's
// first run in row 0 of the stage's tile; sw / so: shared addresses of the quad's lists of stream words and of row
// offsets; members [i0, i1).  All loads carry explicit 32-bit shared addresses: with generic pointers the list
// walk cost 3 % of the kernel's time.
template <int PAT>
__device__ __forceinline__ void run_bucket(uint32_t (&accp)[8][4], uint32_t (&accn)[8][4], uint32_t a_lo, uint32_t sw,
                                           uint32_t so, int i0, int i1, uint32_t one) {
#pragma unroll 2
    for (int i = i0; i < i1; i++) {
        const uint4 w = lds128(sw + (uint32_t)i * 16);
        const uint32_t a = add_on_fma_pipe(lds32(so + (uint32_t)i * 4), one, a_lo);
        const uint4 x = lds128(a);
        const uint4 y = lds128(a + 512);   // the lane's second run: 32 runs of 16 bytes further on
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
__global__ void __launch_bounds__(kTapsThreads, 1) accumulate_taps_kernel(TapsParams pr, TapsStarts st) {
    constexpr int NH = 16 / NQ;
    constexpr int TR = 64 * NH;   // runs of a position tile
    extern __shared__ __align__(16) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int ql = warp % NQ, h = warp / NQ;
    const long long i0 = st.item[blockIdx.x], i1 = st.item[blockIdx.x + 1];
    if (i0 >= i1) return;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const int sw_off = pr.a_bytes, so_off = sw_off + NQ * pr.SL * 16, sb_off = so_off + NQ * pr.SL * 4;

    // origin of run `rho` of the position order in one channel plane of the stream image, in words
    auto run_origin = [&](long long rho, int *oy, int *ox, int *b0) {
        const int pi = (int)(rho / pr.Bq);
        const uint32_t px = __ldg(pr.pix + pi);
        *oy = (int)(px >> 16);
        *ox = (int)(px & 0xffffu);
        *b0 = (int)(rho - (long long)pi * pr.Bq) * 4;
        return ((*oy) * pr.Wp + (*ox)) * pr.Bp + *b0;
    };
    // live taps of a tile: the union over its pixels
    auto tile_mask = [&](int tile) {
        const long long r0 = (long long)tile * TR, r1 = min(r0 + TR, pr.NR) - 1;
        unsigned long long m = 0;
        for (int pi = (int)(r0 / pr.Bq); pi <= (int)(r1 / pr.Bq); pi++) {
            const uint32_t px = __ldg(pr.pix + pi);
            m |= taps_live_mask((int)(px >> 16), (int)(px & 0xffffu), pr.K2, pr.K3, pr.pad_h, pr.pad_w, pr.H, pr.W);
        }
        return m;
    };

    // ---- the sequence of live stages (item, chunk), walked one stage ahead by the producer ----
    int cache_tile = -1;
    unsigned long long cache_mask = 0;
    auto live = [&](long long item, int ch) {
        const int tt = (int)(item / pr.pairs), g = (int)(item % pr.pairs) % pr.G;
        const int tile = tt / pr.CT;
        if (tile != cache_tile) { cache_tile = tile; cache_mask = tile_mask(tile); }
        return (cache_mask >> taps_tap_of(pr.mode, g, ch / pr.NCS, pr.K3)) & 1ull;
    };
    auto advance = [&](long long &item, int &ch) {   // to the next live stage; item == i1: none left
        for (;;) {
            if (++ch == pr.NCH) { ch = 0; item++; }
            if (item >= i1 || live(item, ch)) return;
        }
    };

    // ---- producer ----
    int prod_tile = -1, prod_origin = 0;
    constexpr int RG = kTapsThreads / TR;   // member rows copied per pass
    const int pj = t % TR, prg = t / TR;    // this thread's run of the tile, and its first member row
    auto produce = [&](long long item, int ch, int buf) {
        const int tt = (int)(item / pr.pairs), pair = (int)(item % pr.pairs);
        const int tile = tt / pr.CT, ctile = tt % pr.CT;
        const int p = pair / pr.G, g = pair % pr.G;
        if (tile != prod_tile) {
            prod_tile = tile;
            int oy, ox, b0;
            prod_origin = run_origin(min((long long)tile * TR + pj, pr.NR - 1), &oy, &ox, &b0);
        }
        const uint32_t dst = smem_base + (uint32_t)buf * pr.stage_bytes;
        const int gc = g * pr.NCH + ch;
        const int nmem = min(pr.UCH, pr.C - (ch % pr.NCS) * pr.UCH);
        const uint32_t *src = pr.as + (size_t)p * pr.pack_words + prod_origin;
        const int32_t *mo = pr.moff + (size_t)gc * pr.UCH;
        for (int m = prg; m < nmem; m += RG)
            cp16(dst + (uint32_t)m * pr.row_bytes + (uint32_t)pj * 16, src + (size_t)__ldg(mo + m) * pr.Bp);
        const size_t gcq = (size_t)gc * pr.Q + ctile * NQ;   // the NQ quads' lists are contiguous
        const uint4 *wsrc = pr.sw + ((size_t)p * pr.G * pr.NCH * pr.Q + gcq) * pr.SL;
        for (int i = t; i < NQ * pr.SL; i += kTapsThreads) cp16(dst + sw_off + (uint32_t)i * 16, wsrc + i);
        const uint4 *osrc = (const uint4 *)(pr.soff + gcq * pr.SL);
        for (int i = t; i < NQ * pr.SL / 4; i += kTapsThreads) cp16(dst + so_off + (uint32_t)i * 16, osrc + i);
        if (t < NQ * 3) cp16(dst + sb_off + (uint32_t)t * 16, (const uint4 *)(pr.sbeg + gcq * 24) + t);
    };

    // ---- consumer ----
    uint32_t accp[8][4], accn[8][4];
    int sumA[8], sumB[8];   // per position: channels 0,1 and 2,3 of the quad as two 16-bit sums each
    int cons_tt = -1, cons_tile = -1;
    long long cons_item = -1;
    int out_base[2] = {-1, -1};   // index of (b0, channel 0, oy, ox) in the output, -1: run outside the image list
    int run_b0[2] = {0, 0};
    const long long img_stride = (long long)pr.O * pr.HoWo;

    auto flush = [&]() {
        if (cons_tt < 0) return;
        const int ctile = cons_tt % pr.CT;
        const bool exclusive = (long long)cons_tt * pr.pairs >= i0 && (long long)(cons_tt + 1) * pr.pairs <= i1;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            if (out_base[r] < 0) continue;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (run_b0[r] + i >= pr.B) continue;   // images past the batch: padding of the stream image
                const int a = sumA[r * 4 + i], b = sumB[r * 4 + i];
                const int a0 = (int)(short)(a & 0xffff), b0 = (int)(short)(b & 0xffff);
                const int v[4] = {a0, (a - a0) >> 16, b0, (b - b0) >> 16};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int o = (ctile * NQ + ql) * 4 + j;
                    if (o < pr.O) {
                        int32_t *dst = pr.out + (size_t)out_base[r] + (size_t)i * img_stride + (size_t)o * pr.HoWo;
                        if (exclusive) *dst = v[j];
                        else atomicAdd(dst, v[j]);
                    }
                }
            }
        }
    };

    auto set_lane_positions = [&](int tile) {
        cons_tile = tile;
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const long long rho = (long long)tile * TR + h * 64 + lane + 32 * r;
            if (rho < pr.NR) {
                int oy, ox, b0;
                run_origin(rho, &oy, &ox, &b0);
                run_b0[r] = b0;
                out_base[r] = (b0 * pr.O * pr.Ho + oy) * pr.Wo + ox;
            } else {
                out_base[r] = -1;
            }
        }
    };

    long long cur_item = i0;
    int cur_ch = -1;
    advance(cur_item, cur_ch);
    long long nxt_item = cur_item;
    int nxt_ch = cur_ch;
    int s = 0;
    if (cur_item < i1) {
        produce(cur_item, cur_ch, 0);
        advance(nxt_item, nxt_ch);
    }
    cp_commit();
    while (cur_item < i1) {
        if (nxt_item < i1) produce(nxt_item, nxt_ch, (s + 1) & 1);   // its buffer was read last at stage s - 1
        cp_commit();
        cp_wait<1>();
        __syncthreads();

        const int tt = (int)(cur_item / pr.pairs);
        if (tt != cons_tt) {
            flush();
            cons_tt = tt;
            if (tt / pr.CT != cons_tile) set_lane_positions(tt / pr.CT);
#pragma unroll
            for (int i = 0; i < 8; i++) { sumA[i] = 0; sumB[i] = 0; }
        }
        if (cur_item != cons_item) {   // first live chunk of a group
            cons_item = cur_item;
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) { accp[i][j] = 0; accn[i][j] = 0; }
        }
        {
            const uint32_t stage = smem_base + (uint32_t)(s & 1) * pr.stage_bytes;
            const uint32_t a_lo = stage + (uint32_t)(h * 64 + lane) * 16;
            const unsigned char *stage_ptr = smem + (size_t)(s & 1) * pr.stage_bytes;
            const uint32_t swl = stage + (uint32_t)sw_off + (uint32_t)(ql * pr.SL) * 16;
            const uint32_t sol = stage + (uint32_t)so_off + (uint32_t)(ql * pr.SL) * 4;
            const uint16_t *sbl = (const uint16_t *)(stage_ptr + sb_off) + ql * 24;
            // lane b holds the first slot of pattern b; the loops get their bounds by shuffle
            const int mybeg = lane < 17 ? (int)sbl[lane] : 0;
#define GEO_BUCKET(B) \
    run_bucket<B>(accp, accn, a_lo, swl, sol, __shfl_sync(0xffffffffu, mybeg, B), __shfl_sync(0xffffffffu, mybeg, B + 1), pr.one);
            GEO_BUCKET(0) GEO_BUCKET(1) GEO_BUCKET(2) GEO_BUCKET(3) GEO_BUCKET(4) GEO_BUCKET(5) GEO_BUCKET(6) GEO_BUCKET(7)
            GEO_BUCKET(8) GEO_BUCKET(9) GEO_BUCKET(10) GEO_BUCKET(11) GEO_BUCKET(12) GEO_BUCKET(13) GEO_BUCKET(14) GEO_BUCKET(15)
#undef GEO_BUCKET
        }
        if (nxt_item != cur_item) {   // last live chunk of the group: binary accumulation of its popcounts
#pragma unroll
            for (int i = 0; i < 8; i++) {
                sumA[i] += (__popc(accp[i][0]) - __popc(accn[i][0])) + (__popc(accp[i][1]) - __popc(accn[i][1])) * 65536;
                sumB[i] += (__popc(accp[i][2]) - __popc(accn[i][2])) + (__popc(accp[i][3]) - __popc(accn[i][3])) * 65536;
            }
        }
        __syncthreads();   // every warp is done with this stage's buffer before the next produce() refills it
        cur_item = nxt_item;
        cur_ch = nxt_ch;
        if (nxt_item < i1) advance(nxt_item, nxt_ch);
        s++;
    }
    cp_wait<0>();
    flush();
}

// ---- preparation ------------------------------------------------------------------------------------------
struct SortTapsParams {
    const uint32_t *ws;   // dense prepared streams [P][G][Kp][Opad][2]
    uint4 *sw;
    uint32_t *soff;
    uint16_t *sbeg;
    int32_t *moff;
    int P, G, Kp, Opad, Q;
    int mode, C, K2, K3, Hp, Wp;
    int UCH, NCS, NCH, SL, row_bytes;
};

// One CTA per (quad, group * chunk): sorts the chunk's members (the channels of one tap) by sign pattern.
__global__ void __launch_bounds__(128) sort_taps_kernel(SortTapsParams sp) {
    __shared__ int cnt[16], cur[16], start[17];
    const int q = blockIdx.x, g = blockIdx.y / sp.NCH, ch = blockIdx.y % sp.NCH;
    const int tap = ch / sp.NCS, c0 = (ch % sp.NCS) * sp.UCH;
    const int rows = min(sp.UCH, sp.C - c0);
    const int tk = taps_tap_of(sp.mode, g, tap, sp.K3), ky = tk / sp.K3, kx = tk % sp.K3;
    const int t = threadIdx.x;
    // index of member (c, ky, kx) inside its group in the dense layout
    auto dense_k = [&](int c) {
        switch (sp.mode) {
        case GEO_SC_MODE_1D: return c * sp.K2 + ky;
        case GEO_SC_MODE_2D: return c;
        default: return (c * sp.K2 + ky) * sp.K3 + kx;
        }
    };
    if (t < 16) { cnt[t] = 0; cur[t] = 0; }
    __syncthreads();
    // A thread owns one member (a chunk has at most 256, two passes of 128): its 2 x 4 stream words of every pack
    // (+/- of the quad's four channels, 32 consecutive bytes) are read once, with 16-byte loads, and kept in registers
    // from the pattern pass to the write pass.
    const size_t gc = (size_t)g * sp.NCH + ch;
    const size_t gcq = gc * sp.Q + q;
    uint4 lo[2][kMaxPacks], hi[2][kMaxPacks];
    int mypat[2] = {255, 255};
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int r = t + 128 * it;
        if (r >= rows) continue;
        const int k = dense_k(c0 + r);
        uint32_t any_p[4] = {0, 0, 0, 0}, any_n[4] = {0, 0, 0, 0};
#pragma unroll
        for (int p = 0; p < kMaxPacks; p++) {
            if (p >= sp.P) break;
            const uint4 *e = (const uint4 *)(sp.ws + ((((size_t)p * sp.G + g) * sp.Kp + k) * sp.Opad + q * 4) * 2);
            lo[it][p] = __ldg(e);       // + 0, - 0, + 1, - 1
            hi[it][p] = __ldg(e + 1);   // + 2, - 2, + 3, - 3
            any_p[0] |= lo[it][p].x; any_n[0] |= lo[it][p].y; any_p[1] |= lo[it][p].z; any_n[1] |= lo[it][p].w;
            any_p[2] |= hi[it][p].x; any_n[2] |= hi[it][p].y; any_p[3] |= hi[it][p].z; any_n[3] |= hi[it][p].w;
        }
        int pat = 0, any = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (any_n[j]) pat |= 1 << j;
            any |= (any_p[j] | any_n[j]) != 0;
        }
        mypat[it] = any ? pat : 255;   // 255: contributes nothing, dropped
        if (any) atomicAdd(&cnt[pat], 1);
    }
    __syncthreads();
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
    for (int r = t; r < sp.UCH; r += 128)
        if (q == 0) sp.moff[gc * sp.UCH + r] = r < rows ? ((c0 + r) * sp.Hp + ky) * sp.Wp + kx : 0;
#pragma unroll
    for (int it = 0; it < 2; it++) {
        const int r = t + 128 * it;
        const int pat = mypat[it];
        if (r >= rows || pat == 255) continue;
        const int slot = start[pat] + atomicAdd(&cur[pat], 1);
        sp.soff[gcq * sp.SL + slot] = (uint32_t)r * (uint32_t)sp.row_bytes;
#pragma unroll
        for (int p = 0; p < kMaxPacks; p++) {
            if (p >= sp.P) break;
            const uint4 a = lo[it][p], b = hi[it][p];
            sp.sw[((size_t)p * sp.G * sp.NCH * sp.Q + gcq) * sp.SL + slot] =
                make_uint4(pat & 1 ? a.y : a.x, pat & 2 ? a.w : a.z, pat & 4 ? b.y : b.x, pat & 8 ? b.w : b.z);
        }
    }
}

// Position of output pixel (oy, ox) in the order (border class of oy, border class of ox, oy, ox).
__host__ __device__ inline int taps_pixel_rank(int oy, int ox, int Ho, int Wo, int K2, int K3, int pad_h, int pad_w, int H,
                                               int W) {
    const int cy = taps_border_class(oy, pad_h, K2, H), cx = taps_border_class(ox, pad_w, K3, W);
    int y_less = 0, y_same = 0, y_before = 0, x_less = 0, x_same = 0, x_before = 0;
    for (int y = 0; y < Ho; y++) {
        const int c = taps_border_class(y, pad_h, K2, H);
        y_less += c < cy;
        y_same += c == cy;
        y_before += c == cy && y < oy;
    }
    for (int x = 0; x < Wo; x++) {
        const int c = taps_border_class(x, pad_w, K3, W);
        x_less += c < cx;
        x_same += c == cx;
        x_before += c == cx && x < ox;
    }
    return y_less * Wo + y_same * x_less + y_before * x_same + x_before;
}

__global__ void taps_pixel_order_kernel(uint32_t *pix, int Ho, int Wo, int K2, int K3, int pad_h, int pad_w, int H, int W) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Ho * Wo) return;
    const int oy = i / Wo, ox = i % Wo;
    pix[taps_pixel_rank(oy, ox, Ho, Wo, K2, K3, pad_h, pad_w, H, W)] = ((uint32_t)oy << 16) | (uint32_t)ox;
}

// ---- host side: the CTAs' item ranges, cut by live-chunk count --------------------------------------------------
struct PartitionKey {
    int v[16];
    bool operator<(const PartitionKey &o) const { return std::lexicographical_compare(v, v + 16, o.v, o.v + 16); }
};

void compute_starts(const Geometry &g, const TapsPlan &tp, int nctas, TapsStarts *st) {
    const int TR = 64 * tp.NH, Bq = g.Bp / 4, CT = tp.Q / tp.NQ, HoWo = g.Ho * g.Wo;
    const long long NR = (long long)HoWo * Bq;
    const int tiles = (int)((NR + TR - 1) / TR);
    // pixels in the kernel's order
    std::vector<uint32_t> pix((size_t)HoWo);
    for (int oy = 0; oy < g.Ho; oy++)
        for (int ox = 0; ox < g.Wo; ox++)
            pix[(size_t)taps_pixel_rank(oy, ox, g.Ho, g.Wo, g.K2, g.K3, g.pad_h, g.pad_w, g.H, g.W)] = ((uint32_t)oy << 16) | (uint32_t)ox;
    // live chunks of every group, per tile, and the running cost of the tiles
    std::vector<int> live((size_t)tiles * g.G);
    std::vector<long long> before((size_t)tiles + 1, 0);
    const long long blocks = (long long)CT * g.P;   // (channel tile, pack) blocks of a tile: same cost each
    for (int t = 0; t < tiles; t++) {
        const long long r0 = (long long)t * TR, r1 = std::min(r0 + TR, NR) - 1;
        unsigned long long m = 0;
        for (int pi = (int)(r0 / Bq); pi <= (int)(r1 / Bq); pi++)
            m |= taps_live_mask((int)(pix[(size_t)pi] >> 16), (int)(pix[(size_t)pi] & 0xffffu), g.K2, g.K3, g.pad_h, g.pad_w, g.H, g.W);
        long long sum = 0;
        for (int gi = 0; gi < g.G; gi++) {
            int n = 0;
            for (int tap = 0; tap < tp.TG; tap++) n += (int)((m >> taps_tap_of(g.mode, gi, tap, g.K3)) & 1ull) * tp.NCS;
            live[(size_t)t * g.G + gi] = n;
            sum += n;
        }
        before[(size_t)t + 1] = before[(size_t)t] + sum * blocks;
    }
    const long long total = before[(size_t)tiles];
    const long long n_items = (long long)tiles * blocks * g.G;
    st->n = nctas;
    for (int b = 0; b <= nctas; b++) {
        if (b == nctas || total == 0) { st->item[b] = b == 0 ? 0 : n_items; continue; }
        const long long target = total * b / nctas;
        const int t = (int)(std::upper_bound(before.begin(), before.end(), target) - before.begin()) - 1;   // before[t] <= target
        const int tt = std::min(t, tiles - 1);
        long long per_block = 0;
        for (int gi = 0; gi < g.G; gi++) per_block += live[(size_t)tt * g.G + gi];
        long long rem = target - before[(size_t)tt];
        long long blk = per_block ? rem / per_block : 0;
        if (blk >= blocks) blk = blocks - 1;
        rem -= blk * per_block;
        int gi = 0;
        while (gi < g.G - 1 && rem >= live[(size_t)tt * g.G + gi]) { rem -= live[(size_t)tt * g.G + gi]; gi++; }
        st->item[b] = ((long long)tt * blocks + blk) * g.G + gi;
    }
    st->item[0] = 0;   // items without live chunks before the first cut still belong to someone
    for (int b = 1; b <= nctas; b++)
        if (st->item[b] < st->item[b - 1]) st->item[b] = st->item[b - 1];
}

// the ranges depend on the geometry alone: computed once per geometry and CTA count
TapsStarts cached_starts(const Geometry &g, const TapsPlan &tp, int nctas) {
    static std::mutex m;
    static std::map<PartitionKey, TapsStarts> cache;
    PartitionKey k = {{g.B, g.C, g.H, g.W, g.pad_h, g.pad_w, g.O, g.K2, g.K3, g.L, g.mode, nctas, tp.UCH, tp.NQ, 0, 0}};
    std::lock_guard<std::mutex> lock(m);
    auto it = cache.find(k);
    if (it == cache.end()) {
        if (cache.size() > 256) cache.clear();
        TapsStarts st;
        compute_starts(g, tp, nctas, &st);
        it = cache.emplace(k, st).first;
    }
    return it->second;
}

}  // namespace

TapsPlan taps_plan(const Geometry &g) {
    TapsPlan tp = {};
    tp.layout = false;
    tp.eligible = false;
    if (g.mode != GEO_SC_MODE_1D && g.mode != GEO_SC_MODE_FULL_OR && g.mode != GEO_SC_MODE_2D) return tp;
    // fewer than 64 channels: a tap's chunk would put two or three members into each pattern loop (measured on the
    // 32-channel layers of the 4-layer CNN: 0.73 against 0.58 ms and 0.33 against 0.30 ms on row tiles)
    if (g.C < 64 || g.Kp < 64 || g.Opad % 32 != 0 || g.K2 * g.K3 > 64 || g.Ho > 65535 || g.Wo > 65535) return tp;
    if (g.Hp * g.Wp == 1) return tp;                      // linear layers have kernels of their own
    if ((long long)g.P * g.G * 32 > 32767) return tp;     // the 16-bit running sums of a tile must hold P*G*32
    tp.NQ = g.Opad % 64 == 0 ? 16 : 8;
    tp.NH = 16 / tp.NQ;
    tp.Q = g.Opad / 4;
    tp.TG = g.mode == GEO_SC_MODE_1D ? g.K2 : (g.mode == GEO_SC_MODE_2D ? 1 : g.K2 * g.K3);
    const int row_bytes = 1024 * tp.NH;
    auto stage_bytes = [&](int uch) {
        const size_t sl = (size_t)((uch + 3) / 4 * 4);
        return (size_t)uch * row_bytes + (size_t)tp.NQ * sl * 20 + (size_t)tp.NQ * 48;
    };
    int uch = 0;
    while (uch < g.C && uch < 256 && 2 * stage_bytes(uch + 1) <= kTapsSmemBudget) uch++;
    if (uch < 32) return tp;
    tp.NCS = (g.C + uch - 1) / uch;
    tp.UCH = (g.C + tp.NCS - 1) / tp.NCS;
    tp.NCH = tp.TG * tp.NCS;
    tp.SL = (tp.UCH + 3) / 4 * 4;
    tp.stage_bytes = stage_bytes(tp.UCH);
    const size_t gc = (size_t)g.G * tp.NCH, gcq = gc * tp.Q;
    tp.sw_bytes = align_up((size_t)g.P * gcq * tp.SL * 16, 256);
    tp.soff_bytes = align_up(gcq * tp.SL * 4, 256);
    tp.sbeg_bytes = align_up(gcq * 24 * 2, 256);
    tp.moff_bytes = align_up(gc * tp.UCH * 4, 256);
    tp.pix_bytes = align_up((size_t)g.Ho * g.Wo * 4, 256);
    tp.layout = true;
    tp.eligible = (long long)g.Ho * g.Wo * (g.Bp / 4) >= 64LL * tp.NH;
    return tp;
}

int launch_sort_taps(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s) {
    const TapsPlan tp = taps_plan(g);
    SortTapsParams sp;
    char *base = (char *)section;
    sp.ws = wstream;
    sp.sw = (uint4 *)base;
    sp.soff = (uint32_t *)(base + tp.sw_bytes);
    sp.sbeg = (uint16_t *)(base + tp.sw_bytes + tp.soff_bytes);
    sp.moff = (int32_t *)(base + tp.sw_bytes + tp.soff_bytes + tp.sbeg_bytes);
    uint32_t *pix = (uint32_t *)(base + tp.sw_bytes + tp.soff_bytes + tp.sbeg_bytes + tp.moff_bytes);
    sp.P = g.P; sp.G = g.G; sp.Kp = g.Kp; sp.Opad = g.Opad; sp.Q = tp.Q;
    sp.mode = g.mode; sp.C = g.C; sp.K2 = g.K2; sp.K3 = g.K3; sp.Hp = g.Hp; sp.Wp = g.Wp;
    sp.UCH = tp.UCH; sp.NCS = tp.NCS; sp.NCH = tp.NCH; sp.SL = tp.SL; sp.row_bytes = 1024 * tp.NH;
    sort_taps_kernel<<<dim3(tp.Q, g.G * tp.NCH), 128, 0, s>>>(sp);
    GEO_CUDA_CHECK(cudaGetLastError());
    const int npix = g.Ho * g.Wo;
    taps_pixel_order_kernel<<<(npix + 127) / 128, 128, 0, s>>>(pix, g.Ho, g.Wo, g.K2, g.K3, g.pad_h, g.pad_w, g.H, g.W);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

template <int NQ>
static int launch_taps(const Geometry &g, const TapsPlan &tp, const TapsParams &pr, cudaStream_t s) {
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(accumulate_taps_kernel<NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)kTapsSmemBudget));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    const int TR = 64 * tp.NH;
    const long long tiles = (pr.NR + TR - 1) / TR;
    const long long n_items = tiles * pr.CT * pr.pairs;
    int ctas = sm_count() < kTapsMaxCtas ? sm_count() : kTapsMaxCtas;
    if (n_items < ctas) ctas = (int)n_items;
    const TapsStarts st = cached_starts(g, tp, ctas);
    GEO_CUDA_CHECK(cudaMemsetAsync(pr.out, 0, (size_t)g.M * g.O * sizeof(int32_t), s));
    accumulate_taps_kernel<NQ><<<(unsigned)ctas, kTapsThreads, 2 * tp.stage_bytes, s>>>(pr, st);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_accumulate_taps(const Geometry &g, const uint32_t *astream, const void *section, int32_t *out, cudaStream_t s) {
    const TapsPlan tp = taps_plan(g);
    const char *base = (const char *)section;
    TapsParams pr;
    pr.as = astream; pr.out = out;
    pr.sw = (const uint4 *)base;
    pr.soff = (const uint32_t *)(base + tp.sw_bytes);
    pr.sbeg = (const uint16_t *)(base + tp.sw_bytes + tp.soff_bytes);
    pr.moff = (const int32_t *)(base + tp.sw_bytes + tp.soff_bytes + tp.sbeg_bytes);
    pr.pix = (const uint32_t *)(base + tp.sw_bytes + tp.soff_bytes + tp.sbeg_bytes + tp.moff_bytes);
    pr.B = g.B; pr.Bp = g.Bp; pr.Bq = g.Bp / 4; pr.O = g.O; pr.Ho = g.Ho; pr.Wo = g.Wo; pr.Wp = g.Wp; pr.HoWo = g.Ho * g.Wo;
    pr.H = g.H; pr.W = g.W;
    pr.K2 = g.K2; pr.K3 = g.K3; pr.pad_h = g.pad_h; pr.pad_w = g.pad_w; pr.mode = g.mode;
    pr.P = g.P; pr.G = g.G; pr.NCH = tp.NCH; pr.NCS = tp.NCS; pr.UCH = tp.UCH; pr.C = g.C; pr.SL = tp.SL; pr.Q = tp.Q;
    pr.CT = tp.Q / tp.NQ;
    pr.pack_words = act_pack_words(g);
    pr.stage_bytes = (int)tp.stage_bytes;
    pr.row_bytes = 1024 * tp.NH;
    pr.a_bytes = tp.UCH * pr.row_bytes;
    pr.pairs = g.P * g.G;
    pr.NR = (long long)pr.HoWo * pr.Bq;
    pr.one = 1;
    return tp.NQ == 16 ? launch_taps<16>(g, tp, pr, s) : launch_taps<8>(g, tp, pr, s);
}

}  // namespace geo
