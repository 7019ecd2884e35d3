/*
 * CPU restatement of the reference's stochastic-computing (SC) conv2d forward.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker used by tests/, by the
 * smoke test and by the CPU-baseline leg of bench.py.  The product path (the
 * CUDA library) never calls, links or imports it.
 *
 * Parity status: pinned.  The 1d_bin path without progressive loading is
 * checked bit-for-bit against the reference's own CPU kernel
 * (torch_c/sc-extension/sc.cpp, built unmodified) and, at L=128, against the
 * reference's bit-serial PyTorch simulation (utils_functional.py:516-609);
 * 1d_bin / z_bin / yz_bin with progressive loading are checked against the
 * reference's CUDA kernels (sc_cuda_kernel.cu, built unmodified for sm_100a)
 * through golden vectors committed under tests/golden/.  full_or with the LFSR
 * generator has no deterministic native reference kernel (the reference's GPU
 * full_or uses cuRAND with racy states); it is pinned only at L=128 against the
 * bit-serial PyTorch simulation.
 *
 * Every function cites the reference lines it restates (paths relative to the
 * reference project root).  The code is written for clarity, bit-serial, one
 * stream bit at a time, exactly in the order the reference uses.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GEO_MODE_1D 0      /* OR over (c,ky), binary add over kx           */
#define GEO_MODE_Z 1       /* OR over (ky,kx), binary add over c           */
#define GEO_MODE_YZ 2      /* OR over (c mod z, ky), binary add over (c div z, kx) */
#define GEO_MODE_FULL_OR 3 /* OR over (c,ky,kx)                             */
#define GEO_MODE_2D 4      /* OR over c, binary add over (ky,kx)            */
#define GEO_MODE_FULL_BIN 5 /* binary add over (c,ky,kx): no OR               */

/* LFSR width for a stream length: 8->3 ... 256->8
 * (torch_c/sc-extension/sc.cpp:313-334, sc_cuda_kernel.cu:113-134). */
static int lfsr_bits(int L) {
    switch (L) {
    case 8: return 3;
    case 16: return 4;
    case 32: return 5;
    case 64: return 6;
    case 128: return 7;
    case 256: return 8;
    default: return 0;
    }
}

/* One LFSR step, written with the reference's own divide/modulo arithmetic
 * (torch_c/sc-extension/sc.cpp:262-290, sc_cuda_kernel.cu:18-40,
 * utils_functional.py:104-137). */
int geo_oracle_lfsr_step(int v, int nbits) {
    switch (nbits) {
    case 8: return ((v / 128) + (v / 32) % 2 + (v / 16) % 2 + (v / 8) % 2) % 2 + 2 * (v % 128);
    case 7: return ((v / 32) % 2 + v / 64) % 2 + 2 * (v % 64);
    case 6: return ((v / 32) + (v / 16) % 2) % 2 + 2 * (v % 32);
    case 5: return ((v / 16) + (v / 4) % 2) % 2 + 2 * (v % 16);
    case 4: return ((v / 8) + (v / 4) % 2) % 2 + 2 * (v % 8);
    case 3: return ((v / 4) + (v / 2) % 2) % 2 + 2 * (v % 4);
    default: return -1;
    }
}

/* Float -> integer levels (sc_cuda.cpp:51-55, sc.cpp:301-304):
 *   A  = ceil(clamp(a*L, 0, L-1))
 *   Wp = ceil(clamp(w*L, 0, L-1))
 *   Wn = ceil(-clamp(w*L, 1-L, 0))                                         */
static float clampf(float x, float lo, float hi) { return x < lo ? lo : (x > hi ? hi : x); }
int geo_oracle_quant_act(float a, int L) { return (int)ceilf(clampf(a * (float)L, 0.0f, (float)(L - 1))); }
int geo_oracle_quant_wpos(float w, int L) { return (int)ceilf(clampf(w * (float)L, 0.0f, (float)(L - 1))); }
int geo_oracle_quant_wneg(float w, int L) { return (int)ceilf(-clampf(w * (float)L, (float)(1 - L), 0.0f)); }

/* Seed for generator index idx: (base + idx) mod (L-1) + 1
 * (sc.cpp:344-347,411-413; sc_cuda_kernel.cu:1757-1763,668-670). */
static int seed_of(int base, int idx, int L) { return (base + idx) % (L - 1) + 1; }

/* One packed stream.  For 1-based bit t: the visible width grows as
 *   cw = min(tw, (t / load_wait + 1) * load_width - 1),  V_t = (V >> (tw-cw)) << (tw-cw)
 * the LFSR is stepped first and then compared, bit = [V_t > state]; bits are
 * shifted in MSB-first, 32 per word (8 / 16 in total for L = 8 / 16), and the
 * state runs on from one word to the next
 * (sc_cuda_kernel.cu:151-168,678-690; sc.cpp:365-378,429-434). */
static void gen_stream(int V, int seed, int L, int tw, int lu, int lw, uint32_t *words) {
    int n = lfsr_bits(L);
    int packs = (L + 31) / 32;
    int unit = L < 32 ? L : 32;
    int s = seed, t = 0;
    for (int p = 0; p < packs; p++) {
        uint32_t w = 0;
        for (int b = 0; b < unit; b++) {
            t += 1;
            int cw = (t / lw + 1) * lu - 1;
            if (cw > tw) cw = tw;
            int Vt = (V >> (tw - cw)) << (tw - cw);
            s = geo_oracle_lfsr_step(s, n);
            w = w * 2u + (uint32_t)(Vt > s);
        }
        words[p] = w;
    }
}

/* Generator index of an activation element (padded coordinates):
 * (c*H+y)*W+x, or with c mod z in yz_bin
 * (sc_cuda_kernel.cu:667-670,1080; utils_functional.py:562-563 for full_or). */
static int act_seed_index(int mode, int z, int c, int y, int x, int H, int W) {
    int cc = (mode == GEO_MODE_YZ) ? (c % z) : c;
    return (cc * H + y) * W + x;
}

/* Generator index of a weight element
 *   1d_bin : c*K2+ky            (sc_cuda_kernel.cu:146, sc.cpp:363)
 *   z_bin  : ky*K3+kx           (sc_cuda_kernel.cu:322-324)
 *   yz_bin : (c mod z)*K2+ky    (sc_cuda_kernel.cu:231)
 *   full_or: (c*K2+ky)*K3+kx    (utils_functional.py:562-563,570)
 *   2d_bin : c                  (utils_functional.py:536-541,562: the filter is cut into 1x1 slices
 *                                before the generators are laid out over its last three dims)  */
static int w_seed_index(int mode, int z, int c, int ky, int kx, int K2, int K3) {
    switch (mode) {
    case GEO_MODE_1D: return c * K2 + ky;
    case GEO_MODE_Z: return ky * K3 + kx;
    case GEO_MODE_YZ: return (c % z) * K2 + ky;
    case GEO_MODE_2D: return c;
    default: return (c * K2 + ky) * K3 + kx;
    }
}

/* Activation streams of one batch, canonical layout [B][C][H][W][P].
 * act is the *padded* fp32 input [B][C][H][W]. */
int geo_oracle_act_streams(const float *act, int B, int C, int H, int W, int L, int mode, int z_unit,
                           int tw, int lu, int lw_a, uint32_t *out) {
    if (!lfsr_bits(L) || lu < 1 || lw_a < 1) return -1;
    int P = (L + 31) / 32;
    int z = z_unit < C ? z_unit : C;
    if (z < 1) z = 1;
    for (int b = 0; b < B; b++)
        for (int c = 0; c < C; c++)
            for (int y = 0; y < H; y++)
                for (int x = 0; x < W; x++) {
                    size_t e = (((size_t)b * C + c) * H + y) * W + x;
                    int V = geo_oracle_quant_act(act[e], L);
                    int sd = seed_of(0, act_seed_index(mode, z, c, y, x, H, W), L);
                    gen_stream(V, sd, L, tw, lu, lw_a, out + e * P);
                }
    return 0;
}

/* Weight streams, canonical layout [2][O][C][K2][K3][P]; plane 0 holds the
 * positive-magnitude streams (seed base 67), plane 1 the negative ones (base 37). */
int geo_oracle_weight_streams(const float *w, int O, int C, int K2, int K3, int L, int mode, int z_unit,
                              int tw, int lu, int lw_w, uint32_t *out) {
    if (!lfsr_bits(L) || lu < 1 || lw_w < 1) return -1;
    int P = (L + 31) / 32;
    int z = z_unit < C ? z_unit : C;
    if (z < 1) z = 1;
    size_t N = (size_t)O * C * K2 * K3;
    for (int o = 0; o < O; o++)
        for (int c = 0; c < C; c++)
            for (int ky = 0; ky < K2; ky++)
                for (int kx = 0; kx < K3; kx++) {
                    size_t e = (((size_t)o * C + c) * K2 + ky) * K3 + kx;
                    int idx = w_seed_index(mode, z, c, ky, kx, K2, K3);
                    gen_stream(geo_oracle_quant_wpos(w[e], L), seed_of(67, idx, L), L, tw, lu, lw_w, out + e * P);
                    gen_stream(geo_oracle_quant_wneg(w[e], L), seed_of(37, idx, L), L, tw, lu, lw_w, out + (N + e) * P);
                }
    return 0;
}

static int popc32(uint32_t v) { return __builtin_popcount(v); }

/* SC accumulate over prepared streams.  Output int32 [B][O][H-K2+1][W-K3+1] =
 * sum over packs and binary-accumulated groups of popc(OR(a & w+)) - popc(OR(a & w-)).
 *   1d_bin : sc_cuda_kernel.cu:694-1002, sc.cpp:12-259,457
 *   z_bin  : sc_cuda_kernel.cu:1218-1269 with matmul_outer :43-86
 *   yz_bin : sc_cuda_kernel.cu:1079-1136 (channels past C contribute nothing)
 *   full_or: utils_functional.py:590-609 (sign of the bit-wise conv == OR)   */
int geo_oracle_accumulate(const uint32_t *as, const uint32_t *ws, int B, int C, int H, int W, int O, int K2, int K3,
                          int L, int mode, int z_unit, int32_t *out) {
    int P = (L + 31) / 32;
    int Ho = H - K2 + 1, Wo = W - K3 + 1;
    if (Ho < 1 || Wo < 1) return -2;
    int z = z_unit < C ? z_unit : C;
    if (z < 1) z = 1;
    size_t N = (size_t)O * C * K2 * K3;
    const uint32_t *wp = ws, *wn = ws + N * P;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int o = 0; o < O; o++)
            for (int oy = 0; oy < Ho; oy++)
                for (int ox = 0; ox < Wo; ox++) {
                    int total = 0;
                    for (int p = 0; p < P; p++) {
#define A_AT(c, ky, kx) as[((((size_t)b * C + (c)) * H + oy + (ky)) * W + ox + (kx)) * P + p]
#define W_AT(base, c, ky, kx) base[((((size_t)o * C + (c)) * K2 + (ky)) * K3 + (kx)) * P + p]
                        if (mode == GEO_MODE_1D) {
                            for (int kx = 0; kx < K3; kx++) {
                                uint32_t ap = 0, an = 0;
                                for (int c = 0; c < C; c++)
                                    for (int ky = 0; ky < K2; ky++) {
                                        uint32_t a = A_AT(c, ky, kx);
                                        ap |= a & W_AT(wp, c, ky, kx);
                                        an |= a & W_AT(wn, c, ky, kx);
                                    }
                                total += popc32(ap) - popc32(an);
                            }
                        } else if (mode == GEO_MODE_Z) {
                            for (int c = 0; c < C; c++) {
                                uint32_t ap = 0, an = 0;
                                for (int ky = 0; ky < K2; ky++)
                                    for (int kx = 0; kx < K3; kx++) {
                                        uint32_t a = A_AT(c, ky, kx);
                                        ap |= a & W_AT(wp, c, ky, kx);
                                        an |= a & W_AT(wn, c, ky, kx);
                                    }
                                total += popc32(ap) - popc32(an);
                            }
                        } else if (mode == GEO_MODE_YZ) {
                            for (int c0 = 0; c0 < C; c0 += z)
                                for (int kx = 0; kx < K3; kx++) {
                                    uint32_t ap = 0, an = 0;
                                    for (int c = c0; c < c0 + z && c < C; c++)
                                        for (int ky = 0; ky < K2; ky++) {
                                            uint32_t a = A_AT(c, ky, kx);
                                            ap |= a & W_AT(wp, c, ky, kx);
                                            an |= a & W_AT(wn, c, ky, kx);
                                        }
                                    total += popc32(ap) - popc32(an);
                                }
                        } else if (mode == GEO_MODE_FULL_BIN) {   /* utils_functional.py:593-595,607-609 */
                            for (int c = 0; c < C; c++)
                                for (int ky = 0; ky < K2; ky++)
                                    for (int kx = 0; kx < K3; kx++) {
                                        uint32_t a = A_AT(c, ky, kx);
                                        total += popc32(a & W_AT(wp, c, ky, kx)) - popc32(a & W_AT(wn, c, ky, kx));
                                    }
                        } else if (mode == GEO_MODE_2D) {   /* utils_functional.py:597-601 */
                            for (int ky = 0; ky < K2; ky++)
                                for (int kx = 0; kx < K3; kx++) {
                                    uint32_t ap = 0, an = 0;
                                    for (int c = 0; c < C; c++) {
                                        uint32_t a = A_AT(c, ky, kx);
                                        ap |= a & W_AT(wp, c, ky, kx);
                                        an |= a & W_AT(wn, c, ky, kx);
                                    }
                                    total += popc32(ap) - popc32(an);
                                }
                        } else {
                            uint32_t ap = 0, an = 0;
                            for (int c = 0; c < C; c++)
                                for (int ky = 0; ky < K2; ky++)
                                    for (int kx = 0; kx < K3; kx++) {
                                        uint32_t a = A_AT(c, ky, kx);
                                        ap |= a & W_AT(wp, c, ky, kx);
                                        an |= a & W_AT(wn, c, ky, kx);
                                    }
                            total += popc32(ap) - popc32(an);
                        }
#undef A_AT
#undef W_AT
                    }
                    out[(((size_t)b * O + o) * Ho + oy) * Wo + ox] = total;
                }
    return 0;
}

/* Whole forward: padded fp32 activations and fp32 weights in, int32 counts out.
 * Mirrors sc_cuda.cpp:47-63 (quantise) followed by the launchers
 * sc_cuda_kernel.cu:1732-1834 (1d), :2126-2286 (z), :1972-2124 (yz). */
int geo_oracle_conv2d(const float *act, const float *w, int B, int C, int H, int W, int O, int K2, int K3, int L,
                      int mode, int z_unit, int tw, int lu, int lw_w, int lw_a, int32_t *out) {
    if (!lfsr_bits(L)) return -1;
    if (mode < 0 || mode > 5) return -3;
    int P = (L + 31) / 32;
    uint32_t *as = (uint32_t *)malloc((size_t)B * C * H * W * P * sizeof(uint32_t));
    uint32_t *ws = (uint32_t *)malloc((size_t)2 * O * C * K2 * K3 * P * sizeof(uint32_t));
    if (!as || !ws) {
        free(as);
        free(ws);
        return -4;
    }
    int rc = geo_oracle_act_streams(act, B, C, H, W, L, mode, z_unit, tw, lu, lw_a, as);
    if (!rc) rc = geo_oracle_weight_streams(w, O, C, K2, K3, L, mode, z_unit, tw, lu, lw_w, ws);
    if (!rc) rc = geo_oracle_accumulate(as, ws, B, C, H, W, O, K2, K3, L, mode, z_unit, out);
    free(as);
    free(ws);
    return rc;
}
