// Float "guide" of the SC convolution and its gradient (the straight-through backward used for
// training).  Replaces, as native fp32 kernels, what the reference obtains from PyTorch autograd
// over many small cuDNN convolutions (utils_functional.py:189-296 and :611-634):
//
//   w+ = clamp(w, 0, 100), w- = -clamp(w, -100, 0)
//   y±_g[m][o] = sum_k a[m, k_g] * w±[g][k][o]                 (one plain conv per group g)
//   out        = sum_g (1 - exp(-y+_g)) - sum_g (1 - exp(-y-_g))   (value replaced by the SC result)
//   d out / d y+_g = exp(-y+_g) =: E+_g,   d out / d y-_g = -exp(-y-_g) =: -E-_g
//   grad_w[o,c,ky,kx] = [w >= 0] * sum_m a * gout * E+_g  +  [w <= 0] * sum_m a * gout * E-_g
//   grad_a[b,c,y,x]   = sum_{ky,kx,o} gout * (E+_g * w+ - E-_g * w-)   at output (y+ph-ky, x+pw-kx)
//
// (clamp passes the gradient on both branches at w == 0, hence the two inclusive masks.)
//
// The guide's own value is never used (the reference overwrites it with the SC result), so nothing
// is computed in the forward pass: the whole guide runs in the backward pass, as three
// register-tiled FFMA implicit-GEMM kernels fed through cp.async rings:
//   guide_forward_kernel : D = gout * exp(-conv)        M = positions, N = 2*c_out, K = members
//   guide_wgrad_kernel   : sum_m a * D                  M = members,   N = 2*c_out, K = positions (split)
//   guide_dgrad_kernel   : conv of D with flipped w     M = input pixels, N = c_in block, K = ky*kx*2*c_out
// D layout: [group][polarity][c_out_padded][position], position = (b*Ho + oy)*Wo + ox.
#include "sc_common.h"
#include "sc_guide_mma.h"

namespace geo {

namespace {

__device__ __forceinline__ void cp4(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 4 : 0;  // src-size 0: the 4 destination bytes are zero-filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Decodes (group, member) into filter coordinates; returns false for zero-filled members
// (channels past c_in in the last yz group).
__host__ __device__ inline bool decode_member(int mode, int z, int C, int K2, int K3, int g, int k, int *c, int *ky,
                                              int *kx) {
    switch (mode) {
    case GEO_SC_MODE_1D: *kx = g; *c = k / K2; *ky = k % K2; break;
    case GEO_SC_MODE_Z: *c = g; *ky = k / K3; *kx = k % K3; break;
    case GEO_SC_MODE_YZ: *kx = g % K3; *c = (g / K3) * z + k / K2; *ky = k % K2; break;
    case GEO_SC_MODE_2D: *ky = g / K3; *kx = g % K3; *c = k; break;
    default: *c = k / (K2 * K3); *ky = (k / K3) % K2; *kx = k % K3; break;
    }
    return *c < C;
}

struct GuideDims {
    int B, C, H, W, ph, pw, Hp, Wp, O, K2, K3, Ho, Wo, HoWo;
    int mode, z, G, K, Opad, N2, M;
    int cb, J, cbpad;   // dgrad: channels per block sharing one set of D planes, blocks, padded width
    int Min;            // input pixels B*H*W
};

GuideDims guide_dims(const Geometry &g) {
    GuideDims d;
    d.B = g.B; d.C = g.C; d.H = g.H; d.W = g.W; d.ph = g.pad_h; d.pw = g.pad_w; d.Hp = g.Hp; d.Wp = g.Wp;
    d.O = g.O; d.K2 = g.K2; d.K3 = g.K3; d.Ho = g.Ho; d.Wo = g.Wo; d.HoWo = g.Ho * g.Wo;
    d.mode = g.mode; d.z = g.z; d.G = g.G; d.K = g.K; d.Opad = g.Opad; d.N2 = 2 * g.Opad; d.M = (int)g.M;
    switch (g.mode) {
    case GEO_SC_MODE_Z: d.cb = 1; d.J = g.C; break;
    case GEO_SC_MODE_YZ: d.cb = g.z; d.J = (g.C + g.z - 1) / g.z; break;
    default: d.cb = g.C; d.J = 1; break;
    }
    d.cbpad = d.cb <= 8 ? 8 : (d.cb <= 16 ? 16 : (d.cb <= 32 ? 32 : (d.cb + 63) / 64 * 64));
    d.Min = g.B * g.H * g.W;
    return d;
}

// ---- preparation: padded activations, split weights, tables --------------------------------
__global__ void __launch_bounds__(256) pad_act_kernel(GuideDims d, const float *__restrict__ act,
                                                      float *__restrict__ apad) {
    const long long total = (long long)d.B * d.C * d.Hp * d.Wp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int x = (int)(i % d.Wp), y = (int)((i / d.Wp) % d.Hp);
        const long long bc = i / ((long long)d.Wp * d.Hp);
        const int yi = y - d.ph, xi = x - d.pw;
        apad[i] = (yi >= 0 && yi < d.H && xi >= 0 && xi < d.W) ? act[(bc * d.H + yi) * d.W + xi] : 0.0f;
    }
}

// Wf[g][k][Opad][2] = (w+, w-) and aoff[g][k] = offset of the member inside a padded image.
__global__ void __launch_bounds__(256) guide_prep_fwd_kernel(GuideDims d, const float *__restrict__ w,
                                                             float *__restrict__ wf, int *__restrict__ aoff) {
    const long long total = (long long)d.G * d.K * d.Opad;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int o = (int)(i % d.Opad);
        const int gk = (int)(i / d.Opad), k = gk % d.K, g = gk / d.K;
        int c, ky, kx;
        const bool valid = decode_member(d.mode, d.z, d.C, d.K2, d.K3, g, k, &c, &ky, &kx);
        if (o == 0) aoff[gk] = valid ? (c * d.Hp + ky) * d.Wp + kx : 0;
        float v = 0.0f;
        if (valid && o < d.O) v = w[(((size_t)o * d.C + c) * d.K2 + ky) * d.K3 + kx];
        float2 r;
        r.x = fminf(fmaxf(v, 0.0f), 100.0f);
        r.y = -fminf(fmaxf(v, -100.0f), 0.0f);
        *(float2 *)(wf + (size_t)i * 2) = r;
    }
}

// Wd[j][(ky*K3+kx)*N2 + pol*Opad + o][cbpad] = w+ (pol 0) or -(w-) (pol 1) of channel j*cb+cc.
__global__ void __launch_bounds__(256) guide_prep_dgrad_kernel(GuideDims d, const float *__restrict__ w,
                                                               float *__restrict__ wd) {
    const int R = d.K2 * d.K3 * d.N2;
    const long long total = (long long)d.J * R * d.cbpad;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int cc = (int)(i % d.cbpad);
        const int r = (int)((i / d.cbpad) % R), j = (int)(i / ((long long)d.cbpad * R));
        const int n2 = r % d.N2, kk = r / d.N2, ky = kk / d.K3, kx = kk % d.K3;
        const int pol = n2 / d.Opad, o = n2 % d.Opad, c = j * d.cb + cc;
        float v = 0.0f;
        if (cc < d.cb && c < d.C && o < d.O) {
            const float x = w[(((size_t)o * d.C + c) * d.K2 + ky) * d.K3 + kx];
            v = pol == 0 ? fminf(fmaxf(x, 0.0f), 100.0f) : fminf(fmaxf(x, -100.0f), 0.0f);
        }
        wd[i] = v;
    }
}

// ---- D±_g = gout * exp(-conv_g) -------------------------------------------------------------
constexpr int FKC = 16, FSTAGE = 3;

struct FwdParams {
    const float *apad;  // [B][C][Hp][Wp]
    const float *wf;    // [G][K][Opad][2]
    const int *aoff;    // [G][K]
    const float *gout;  // [B][O][Ho][Wo]
    float *D;           // [G][2][Opad][M] = gout * exp(-y)
    int M, O, Opad, HoWo, Wo, Wp, K, img;
    int vec_ok;         // M and Ho*Wo multiples of 4 and gout 16-byte aligned: 4 positions per access
    const int *inexact; // when set: run only if *inexact != 0 (otherwise the tensor-core kernel did the work)
};

template <int NT, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS) guide_forward_kernel(FwdParams pr) {
    constexpr int TY = NT / 4, TX = NTHREADS / TY, MT = TX * 8;
    constexpr int A_F = FKC * MT, W_F = FKC * NT * 2, ST_F = A_F + W_F;
    extern __shared__ __align__(16) float fsm[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    constexpr int WX = TX / 8;
    const int tx = (warp % WX) * 8 + (lane & 7), ty = (warp / WX) * 4 + (lane >> 3);
    const int m0 = blockIdx.x * MT, o0 = blockIdx.y * NT, g = blockIdx.z;
    if (pr.inexact && *pr.inexact == 0) return;

    constexpr int MPT = MT > NTHREADS ? MT / NTHREADS : 1;
    constexpr int RSTEP = NTHREADS > MT ? NTHREADS / MT : 1;
    const int r0 = NTHREADS > MT ? t / MT : 0;
    int abase[MPT];
#pragma unroll
    for (int j = 0; j < MPT; j++) {
        int m = m0 + (t % MT) + j * NTHREADS;
        if (m >= pr.M) m = pr.M - 1;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
        abase[j] = b * pr.img + (rem / pr.Wo) * pr.Wp + (rem % pr.Wo);
    }
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(fsm);
    const int chunks = (pr.K + FKC - 1) / FKC;
    int ld = 0;
    auto issue = [&]() {
        if (ld < chunks) {
            const uint32_t a_s = sbase + (uint32_t)(ld % FSTAGE) * ST_F * 4, w_s = a_s + A_F * 4;
            const int k0 = ld * FKC, rows = min(FKC, pr.K - k0);
            const int *ao = pr.aoff + g * pr.K + k0;
#pragma unroll
            for (int j = 0; j < MPT; j++) {
                const int mcol = (t % MT) + j * NTHREADS;
                for (int r = r0; r < rows; r += RSTEP)
                    cp4(a_s + (uint32_t)(r * MT + mcol) * 4, pr.apad + abase[j] + __ldg(ao + r), true);
            }
            constexpr int CPR = NT / 2;
            const float *wsrc = pr.wf + ((size_t)(g * pr.K + k0) * pr.Opad + o0) * 2;
            for (int i = t; i < rows * CPR; i += NTHREADS) {
                const int r = i / CPR, ch = i % CPR;
                cp16(w_s + (uint32_t)(r * NT * 2 + ch * 4) * 4, wsrc + (size_t)r * pr.Opad * 2 + ch * 4, true);
            }
            ld++;
        }
        cp_commit();
    };
#pragma unroll
    for (int s = 0; s < FSTAGE - 1; s++) issue();

    float accp[8][4], accn[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) { accp[i][j] = 0.f; accn[i][j] = 0.f; }

    for (int s = 0; s < chunks; s++) {
        cp_wait<FSTAGE - 2>();
        __syncthreads();
        issue();
        const float *a_s = fsm + (size_t)(s % FSTAGE) * ST_F, *w_s = a_s + A_F;
        const int rows = min(FKC, pr.K - s * FKC);
        const float4 *a4 = (const float4 *)a_s + tx, *w4 = (const float4 *)w_s + ty * 2;
#pragma unroll 4
        for (int r = 0; r < rows; r++) {
            const float4 al = a4[r * (MT / 4)], ah = a4[r * (MT / 4) + MT / 8];
            const float4 wa = w4[r * (NT / 2)], wb = w4[r * (NT / 2) + 1];
            const float a[8] = {al.x, al.y, al.z, al.w, ah.x, ah.y, ah.z, ah.w};
            const float wp[4] = {wa.x, wa.z, wb.x, wb.z}, wn[4] = {wa.y, wa.w, wb.y, wb.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    accp[i][j] = fmaf(a[i], wp[j], accp[i][j]);
                    accn[i][j] = fmaf(a[i], wn[j], accn[i][j]);
                }
        }
    }
    cp_wait<0>();
    // epilogue: D = gout * exp(-y); the thread's positions are two runs of 4 consecutive ones
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int m = m0 + half * (MT / 2) + tx * 4;
        if (m >= pr.M) continue;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int o = o0 + ty * 4 + j;
            float *dp = pr.D + ((size_t)(g * 2 + 0) * pr.Opad + o) * pr.M + m;
            float *dn = pr.D + ((size_t)(g * 2 + 1) * pr.Opad + o) * pr.M + m;
            if (pr.vec_ok) {
                float4 go = make_float4(0.f, 0.f, 0.f, 0.f);  // padded channels have no upstream gradient
                if (o < pr.O) go = __ldg((const float4 *)(pr.gout + ((size_t)b * pr.O + o) * pr.HoWo + rem));
                float4 vp, vn;
                vp.x = go.x * expf(-accp[half * 4 + 0][j]); vn.x = go.x * expf(-accn[half * 4 + 0][j]);
                vp.y = go.y * expf(-accp[half * 4 + 1][j]); vn.y = go.y * expf(-accn[half * 4 + 1][j]);
                vp.z = go.z * expf(-accp[half * 4 + 2][j]); vn.z = go.z * expf(-accn[half * 4 + 2][j]);
                vp.w = go.w * expf(-accp[half * 4 + 3][j]); vn.w = go.w * expf(-accn[half * 4 + 3][j]);
                *(float4 *)dp = vp;
                *(float4 *)dn = vn;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int mi = m + i;
                    if (mi < pr.M) {
                        const int bi = mi / pr.HoWo, ri = mi % pr.HoWo;
                        const float go = o < pr.O ? __ldg(pr.gout + ((size_t)bi * pr.O + o) * pr.HoWo + ri) : 0.0f;
                        dp[i] = go * expf(-accp[half * 4 + i][j]);
                        dn[i] = go * expf(-accn[half * 4 + i][j]);
                    }
                }
            }
        }
    }
}

// ---- wgrad: partial[slice][g][k][n2] = sum_{m in slice} a[m, k_g] * D[g][n2][m] -----------------------
constexpr int WMC = 32, WRS = WMC + 4, WSTAGE = 3, WNT = 64;

struct WgradParams {
    const float *apad;
    const float *D;     // [G][N2][M]
    const int *aoff;    // [G][K]
    float *partial;     // [S][G][K][N2]
    int M, N2, HoWo, Wo, Wp, K, G, img;
    int slice_len;      // positions per slice, multiple of WMC
    const int *inexact; // when set: run only if *inexact != 0
};

template <int KT>
__global__ void __launch_bounds__(KT, KT <= 128 ? 3 : 2) guide_wgrad_kernel(WgradParams pr) {
    constexpr int NTHREADS = KT;           // (KT/8) member-threads x 8 channel-threads
    constexpr int KTH = KT / 8;
    constexpr int A_F = KT * WRS, D_F = WNT * WRS, ST_F = A_F + D_F;
    extern __shared__ __align__(16) float wsm[];
    if (pr.inexact && *pr.inexact == 0) return;
    const int t = threadIdx.x;
    const int kth = t % KTH, nth = t / KTH;
    const int g = blockIdx.z / ((pr.N2 + WNT - 1) / WNT), nt = blockIdx.z % ((pr.N2 + WNT - 1) / WNT);
    const int k0 = blockIdx.y * KT, n0 = nt * WNT;
    const int mbeg = blockIdx.x * pr.slice_len, mend = min(pr.M, mbeg + pr.slice_len);
    const int chunks = (mend - mbeg + WMC - 1) / WMC;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(wsm);
    const bool vec = (pr.M & 3) == 0;

    // gather assignment for A: column m = t % WMC, rows t / WMC + i * (NTHREADS / WMC)
    const int am = t % WMC, ar0 = t / WMC;
    constexpr int ARS = NTHREADS / WMC > 0 ? NTHREADS / WMC : 1;
    int ld = 0;
    auto issue = [&]() {
        if (ld < chunks) {
            const uint32_t a_s = sbase + (uint32_t)(ld % WSTAGE) * ST_F * 4, d_s = a_s + A_F * 4;
            const int mc = mbeg + ld * WMC;
            {
                const int m = mc + am;
                const bool mv = m < mend;
                const int mm = mv ? m : mbeg;
                const int b = mm / pr.HoWo, rem = mm % pr.HoWo;
                const float *src = pr.apad + b * pr.img + (rem / pr.Wo) * pr.Wp + (rem % pr.Wo);
                const int *ao = pr.aoff + g * pr.K;
                for (int r = ar0; r < KT; r += ARS) {
                    const int k = k0 + r;
                    const bool v = mv && k < pr.K;
                    cp4(a_s + (uint32_t)(r * WRS + am) * 4, src + (v ? __ldg(ao + k) : 0), v);
                }
            }
            if (vec) {
                for (int i = t; i < WNT * (WMC / 4); i += NTHREADS) {
                    const int r = i / (WMC / 4), c4 = i % (WMC / 4);
                    const int n = n0 + r, m = mc + c4 * 4;
                    const bool v = n < pr.N2 && m < mend;  // M % 4 == 0 and slices are multiples of 4
                    const float *src = pr.D + ((size_t)(g * pr.N2 + (v ? n : 0))) * pr.M + (v ? m : 0);
                    cp16(d_s + (uint32_t)(r * WRS + c4 * 4) * 4, src, v);
                }
            } else {
                for (int i = t; i < WNT * WMC; i += NTHREADS) {
                    const int r = i / WMC, c = i % WMC;
                    const int n = n0 + r, m = mc + c;
                    const bool v = n < pr.N2 && m < mend;
                    const float *src = pr.D + ((size_t)(g * pr.N2 + (v ? n : 0))) * pr.M + (v ? m : 0);
                    cp4(d_s + (uint32_t)(r * WRS + c) * 4, src, v);
                }
            }
            ld++;
        }
        cp_commit();
    };
#pragma unroll
    for (int s = 0; s < WSTAGE - 1; s++) issue();

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    for (int s = 0; s < chunks; s++) {
        cp_wait<WSTAGE - 2>();
        __syncthreads();
        issue();
        const float *a_s = wsm + (size_t)(s % WSTAGE) * ST_F, *d_s = a_s + A_F;
#pragma unroll 2
        for (int m4 = 0; m4 < WMC; m4 += 4) {
            float4 av[8];
#pragma unroll
            for (int i = 0; i < 8; i++) av[i] = *(const float4 *)(a_s + (kth + KTH * i) * WRS + m4);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float4 dv = *(const float4 *)(d_s + (nth + 8 * j) * WRS + m4);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    acc[i][j] = fmaf(av[i].x, dv.x, acc[i][j]);
                    acc[i][j] = fmaf(av[i].y, dv.y, acc[i][j]);
                    acc[i][j] = fmaf(av[i].z, dv.z, acc[i][j]);
                    acc[i][j] = fmaf(av[i].w, dv.w, acc[i][j]);
                }
            }
        }
    }
    cp_wait<0>();
    float *dst = pr.partial + ((size_t)blockIdx.x * pr.G + g) * pr.K * pr.N2;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int k = k0 + kth + KTH * i;
        if (k < pr.K) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int n = n0 + nth + 8 * j;
                if (n < pr.N2) dst[(size_t)k * pr.N2 + n] = acc[i][j];
            }
        }
    }
}

// Variant for groups of at most 16 members (first layer of the CNN: 15; 3x3 z_bin: 9; linear with
// z_unit 16): one member x 8 channels per thread, 16 member slots x 8 channel threads per CTA.
__global__ void __launch_bounds__(128) guide_wgrad_smallk_kernel(WgradParams pr) {
    constexpr int NTHREADS = 128, KS = 16;
    constexpr int A_F = KS * WRS, D_F = WNT * WRS, ST_F = A_F + D_F;
    extern __shared__ __align__(16) float wsm[];
    if (pr.inexact && *pr.inexact == 0) return;
    const int t = threadIdx.x;
    const int ks = t % KS, nth = t / KS;
    const int ntiles = (pr.N2 + WNT - 1) / WNT;
    const int g = blockIdx.y, n0 = blockIdx.z * WNT;
    (void)ntiles;
    const int mbeg = blockIdx.x * pr.slice_len, mend = min(pr.M, mbeg + pr.slice_len);
    const int chunks = (mend - mbeg + WMC - 1) / WMC;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(wsm);
    const bool vec = (pr.M & 3) == 0;
    const int am = t % WMC, ar0 = t / WMC;   // 4 rows per pass
    int ld = 0;
    auto issue = [&]() {
        if (ld < chunks) {
            const uint32_t a_s = sbase + (uint32_t)(ld % WSTAGE) * ST_F * 4, d_s = a_s + A_F * 4;
            const int mc = mbeg + ld * WMC;
            {
                const int m = mc + am;
                const bool mv = m < mend;
                const int mm = mv ? m : mbeg;
                const int b = mm / pr.HoWo, rem = mm % pr.HoWo;
                const float *src = pr.apad + b * pr.img + (rem / pr.Wo) * pr.Wp + (rem % pr.Wo);
                const int *ao = pr.aoff + g * pr.K;
                for (int r = ar0; r < KS; r += NTHREADS / WMC) {
                    const bool v = mv && r < pr.K;
                    cp4(a_s + (uint32_t)(r * WRS + am) * 4, src + (v ? __ldg(ao + r) : 0), v);
                }
            }
            if (vec) {
                for (int i = t; i < WNT * (WMC / 4); i += NTHREADS) {
                    const int r = i / (WMC / 4), c4 = i % (WMC / 4);
                    const int n = n0 + r, m = mc + c4 * 4;
                    const bool v = n < pr.N2 && m < mend;
                    const float *src = pr.D + ((size_t)(g * pr.N2 + (v ? n : 0))) * pr.M + (v ? m : 0);
                    cp16(d_s + (uint32_t)(r * WRS + c4 * 4) * 4, src, v);
                }
            } else {
                for (int i = t; i < WNT * WMC; i += NTHREADS) {
                    const int r = i / WMC, c = i % WMC;
                    const int n = n0 + r, m = mc + c;
                    const bool v = n < pr.N2 && m < mend;
                    const float *src = pr.D + ((size_t)(g * pr.N2 + (v ? n : 0))) * pr.M + (v ? m : 0);
                    cp4(d_s + (uint32_t)(r * WRS + c) * 4, src, v);
                }
            }
            ld++;
        }
        cp_commit();
    };
#pragma unroll
    for (int s = 0; s < WSTAGE - 1; s++) issue();
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    for (int s = 0; s < chunks; s++) {
        cp_wait<WSTAGE - 2>();
        __syncthreads();
        issue();
        const float *a_s = wsm + (size_t)(s % WSTAGE) * ST_F, *d_s = a_s + A_F;
#pragma unroll
        for (int m4 = 0; m4 < WMC; m4 += 4) {
            const float4 av = *(const float4 *)(a_s + ks * WRS + m4);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float4 dv = *(const float4 *)(d_s + (nth + 8 * j) * WRS + m4);
                acc[j] = fmaf(av.x, dv.x, acc[j]);
                acc[j] = fmaf(av.y, dv.y, acc[j]);
                acc[j] = fmaf(av.z, dv.z, acc[j]);
                acc[j] = fmaf(av.w, dv.w, acc[j]);
            }
        }
    }
    cp_wait<0>();
    if (ks < pr.K) {
        float *dst = pr.partial + (((size_t)blockIdx.x * pr.G + g) * pr.K + ks) * pr.N2;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int n = n0 + nth + 8 * j;
            if (n < pr.N2) dst[n] = acc[j];
        }
    }
}

// grad_w[o][c][ky][kx] = [w>=0] * sum_s partial[s][g][k][o] + [w<=0] * sum_s partial[s][g][k][Opad+o]
__global__ void __launch_bounds__(256) guide_wgrad_reduce_kernel(GuideDims d, int S, const float *__restrict__ partial,
                                                                 const float *__restrict__ w, float *__restrict__ gw,
                                                                 const int *inexact) {
    if (inexact && *inexact == 0) return;
    const long long total = (long long)d.G * d.K * d.O;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int o = (int)(i % d.O);
        const int gk = (int)(i / d.O), k = gk % d.K, g = gk / d.K;
        int c, ky, kx;
        if (!decode_member(d.mode, d.z, d.C, d.K2, d.K3, g, k, &c, &ky, &kx)) continue;
        float sp = 0.f, sn = 0.f;
        const size_t stride = (size_t)d.G * d.K * d.N2;
        const float *p = partial + ((size_t)g * d.K + k) * d.N2;
        for (int s = 0; s < S; s++) {
            sp += p[s * stride + o];
            sn += p[s * stride + d.Opad + o];
        }
        const size_t wi = (((size_t)o * d.C + c) * d.K2 + ky) * d.K3 + kx;
        const float wv = w[wi];
        gw[wi] = (wv >= 0.f && wv <= 100.f ? sp : 0.f) + (wv <= 0.f && wv >= -100.f ? sn : 0.f);
    }
}

// ---- dgrad: grad_a[b][c][y][x] = sum_{ky,kx,n2} D[g][n2][b, y+ph-ky, x+pw-kx] * Wd[j][(ky,kx,n2)][c] -----
constexpr int DKC = 16, DSTAGE = 3;

struct DgradParams {
    const float *D;    // [G][N2][M]
    const float *wd;   // [J][R][cbpad]
    float *ga;         // [B][C][H][W]
    int M, N2, Ho, Wo, H, W, C, ph, pw, K2, K3, mode, cb, cbpad, Min, R;
    const int *inexact; // when set: run only if *inexact != 0
};

template <int NT, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS) guide_dgrad_kernel(DgradParams pr) {
    constexpr int TY = NT / 8, TX = NTHREADS / TY, MT = TX * 8;   // thread tile: 8 pixels x 8 channels
    constexpr int A_F = DKC * MT, W_F = DKC * NT, ST_F = A_F + W_F;
    static_assert(MT % NTHREADS == 0, "each thread gathers MT/NTHREADS pixel columns");
    constexpr int MPT = MT / NTHREADS;
    extern __shared__ __align__(16) float dsm[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    int tx, ty;
    if constexpr (TY >= 4) {  // warps of 8 pixel columns x 4 channel rows
        constexpr int WX = TX / 8;
        tx = (warp % WX) * 8 + (lane & 7);
        ty = (warp / WX) * 4 + (lane >> 3);
    } else {
        tx = t % TX;
        ty = t / TX;
    }
    const int m0 = blockIdx.x * MT, c0 = blockIdx.y * NT, j = blockIdx.z;
    if (pr.inexact && *pr.inexact == 0) return;
    const int HoWo = pr.Ho * pr.Wo, HW = pr.H * pr.W;

    int pb[MPT], py[MPT], px[MPT];
#pragma unroll
    for (int q = 0; q < MPT; q++) {
        int m = m0 + t + q * NTHREADS;
        const bool v = m < pr.Min;
        if (!v) m = 0;
        const int b = m / HW, rem = m % HW;
        pb[q] = v ? b * HoWo : -1;
        py[q] = rem / pr.W + pr.ph;
        px[q] = rem % pr.W + pr.pw;
    }
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dsm);
    const int chunks = pr.R / DKC;   // R = K2*K3*N2 and N2 is a multiple of 32
    const int cpk = pr.N2 / DKC;     // chunks per (ky,kx)
    int ld = 0;
    auto issue = [&]() {
        if (ld < chunks) {
            const uint32_t a_s = sbase + (uint32_t)(ld % DSTAGE) * ST_F * 4, w_s = a_s + A_F * 4;
            const int kk = ld / cpk, n2 = (ld % cpk) * DKC;
            const int ky = kk / pr.K3, kx = kk % pr.K3;
            int g;
            switch (pr.mode) {
            case GEO_SC_MODE_1D: g = kx; break;
            case GEO_SC_MODE_Z: g = j; break;
            case GEO_SC_MODE_YZ: g = j * pr.K3 + kx; break;
            case GEO_SC_MODE_2D: g = kk; break;
            default: g = 0; break;
            }
            const float *plane = pr.D + (size_t)(g * pr.N2 + n2) * pr.M;
#pragma unroll
            for (int q = 0; q < MPT; q++) {
                const int oy = py[q] - ky, ox = px[q] - kx;
                const bool v = pb[q] >= 0 && oy >= 0 && oy < pr.Ho && ox >= 0 && ox < pr.Wo;
                const float *src = plane + (v ? pb[q] + oy * pr.Wo + ox : 0);
                const uint32_t dst = a_s + (uint32_t)(t + q * NTHREADS) * 4;
#pragma unroll
                for (int r = 0; r < DKC; r++) cp4(dst + (uint32_t)(r * MT) * 4, src + (size_t)r * pr.M, v);
            }
            const float *wsrc = pr.wd + ((size_t)j * pr.R + (size_t)ld * DKC) * pr.cbpad + c0;
            constexpr int CPR = NT / 4;
            for (int i = t; i < DKC * CPR; i += NTHREADS) {
                const int r = i / CPR, ch = i % CPR;
                cp16(w_s + (uint32_t)(r * NT + ch * 4) * 4, wsrc + (size_t)r * pr.cbpad + ch * 4, true);
            }
            ld++;
        }
        cp_commit();
    };
#pragma unroll
    for (int s = 0; s < DSTAGE - 1; s++) issue();

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int q = 0; q < 8; q++) acc[i][q] = 0.f;

    for (int s = 0; s < chunks; s++) {
        cp_wait<DSTAGE - 2>();
        __syncthreads();
        issue();
        const float *a_s = dsm + (size_t)(s % DSTAGE) * ST_F, *w_s = a_s + A_F;
        const float4 *a4 = (const float4 *)a_s + tx, *w4 = (const float4 *)w_s + ty * 2;
#pragma unroll 4
        for (int r = 0; r < DKC; r++) {
            const float4 al = a4[r * (MT / 4)], ah = a4[r * (MT / 4) + MT / 8];
            const float4 wa = w4[r * (NT / 4)], wb = w4[r * (NT / 4) + 1];
            const float a[8] = {al.x, al.y, al.z, al.w, ah.x, ah.y, ah.z, ah.w};
            const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int q = 0; q < 8; q++) acc[i][q] = fmaf(a[i], wv[q], acc[i][q]);
        }
    }
    cp_wait<0>();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int m = m0 + (i < 4 ? tx * 4 + i : MT / 2 + tx * 4 + (i - 4));
        if (m < pr.Min) {
            const int b = m / HW, rem = m % HW;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int cc = c0 + ty * 8 + q;
                const int c = j * pr.cb + cc;
                if (cc < pr.cb && c < pr.C) pr.ga[((size_t)b * pr.C + c) * HW + rem] = acc[i][q];
            }
        }
    }
}

int grid1d(long long total) {
    long long blocks = (total + 255) / 256;
    return (int)(blocks < sm_count() * 16 ? (blocks > 0 ? blocks : 1) : sm_count() * 16);
}

// ---- buffer plan -------------------------------------------------------------------------------------
struct GuidePlan {
    size_t d_bytes, apad_bytes, aoff_bytes, wf_bytes, wd_bytes, partial_bytes, mma_bytes;
    int S, slice_len, KT;
    size_t total() const { return d_bytes + apad_bytes + aoff_bytes + wf_bytes + wd_bytes + partial_bytes + mma_bytes; }
};

GuidePlan guide_plan(const GuideDims &d, const Geometry &g) {
    GuidePlan p;
    p.mma_bytes = mma_scratch_bytes(g);
    p.d_bytes = align_up((size_t)d.G * d.N2 * d.M * 4, 256);
    p.apad_bytes = align_up((size_t)d.B * d.C * d.Hp * d.Wp * 4, 256);
    p.aoff_bytes = align_up((size_t)d.G * d.K * 4, 256);
    p.wf_bytes = align_up((size_t)d.G * d.K * d.Opad * 2 * 4, 256);
    p.wd_bytes = align_up((size_t)d.J * d.K2 * d.K3 * d.N2 * d.cbpad * 4, 256);
    // member tile: 16 (dedicated small-group kernel) or the multiple of 32 up to 192 that wastes
    // the fewest rows (ties to the larger tile)
    if (d.K <= 16) {
        p.KT = 16;
    } else {
        long long best = -1;
        for (int kt = 32; kt <= 192; kt += 32) {
            const long long rows = (long long)((d.K + kt - 1) / kt) * kt;
            if (best < 0 || rows <= best) { best = rows; p.KT = kt; }
        }
    }
    const long long tiles = (long long)d.G * ((d.K + p.KT - 1) / p.KT) * ((d.N2 + WNT - 1) / WNT);
    long long S = ((long long)sm_count() * 6 + tiles - 1) / tiles;
    const long long maxS = (d.M + WMC - 1) / WMC;
    if (S > maxS) S = maxS;
    if (S < 1) S = 1;
    long long len = (d.M + S - 1) / S;
    len = (len + WMC - 1) / WMC * WMC;
    p.slice_len = (int)len;
    p.S = (int)((d.M + len - 1) / len);
    p.partial_bytes = align_up((size_t)p.S * d.G * d.K * d.N2 * 4, 256);
    return p;
}

// Raises the dynamic shared-memory limit of a kernel once per device (not on every launch, so
// that steady-state calls contain nothing but launches and can be captured into a CUDA graph).
template <typename Kern>
int set_smem(Kern kern, size_t bytes, bool *done) {   // `done`: one 64-entry array per kernel
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

template <int NT, int NTHREADS>
int launch_guide_fwd(const GuideDims &d, const FwdParams &pr, cudaStream_t s) {
    constexpr int TY = NT / 4, TX = NTHREADS / TY, MT = TX * 8;
    constexpr size_t smem = (size_t)FSTAGE * (FKC * MT + FKC * NT * 2) * 4;
    static bool done[64] = {};
    int rc = set_smem(guide_forward_kernel<NT, NTHREADS>, smem, done);
    if (rc) return rc;
    dim3 grid((d.M + MT - 1) / MT, d.Opad / NT, d.G);
    guide_forward_kernel<NT, NTHREADS><<<grid, NTHREADS, smem, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

template <int KT>
int launch_guide_wgrad(const GuideDims &d, const GuidePlan &p, const WgradParams &pr, cudaStream_t s) {
    constexpr size_t smem = (size_t)WSTAGE * (KT * WRS + WNT * WRS) * 4;
    static bool done[64] = {};
    int rc = set_smem(guide_wgrad_kernel<KT>, smem, done);
    if (rc) return rc;
    dim3 grid(p.S, (d.K + KT - 1) / KT, d.G * ((d.N2 + WNT - 1) / WNT));
    guide_wgrad_kernel<KT><<<grid, KT, smem, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

template <int NT, int NTHREADS>
int launch_guide_dgrad(const GuideDims &d, const DgradParams &pr, cudaStream_t s) {
    constexpr int TY = NT / 8, TX = NTHREADS / TY, MT = TX * 8;
    constexpr size_t smem = (size_t)DSTAGE * (DKC * MT + DKC * NT) * 4;
    static bool done[64] = {};
    int rc = set_smem(guide_dgrad_kernel<NT, NTHREADS>, smem, done);
    if (rc) return rc;
    dim3 grid((d.Min + MT - 1) / MT, d.cbpad / NT, d.J);
    guide_dgrad_kernel<NT, NTHREADS><<<grid, NTHREADS, smem, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

}  // namespace

}  // namespace geo

using namespace geo;

namespace geo {
namespace {
// Geometry the guide works on.  full_bin has no OR: its guide is the plain convolution
// (utils_functional.py:617-619), i.e. the full_or guide (one group with all members) without the exp.
int guide_geometry(const geo_sc_conv_desc *desc, Geometry *g) {
    if (desc && desc->mode == GEO_SC_MODE_FULL_BIN) {
        geo_sc_conv_desc d2 = *desc;
        d2.mode = GEO_SC_MODE_FULL_OR;
        int rc = make_geometry(&d2, g);
        if (rc) return rc;
        g->guide_linear = 1;
        return GEO_SC_OK;
    }
    return make_geometry(desc, g);
}
}  // namespace
}  // namespace geo

extern "C" {

int geo_sc_guide_backward_bytes(const geo_sc_conv_desc *desc, size_t *scratch_bytes) {
    Geometry g;
    int rc = guide_geometry(desc, &g);
    if (rc) return rc;
    const GuideDims d = guide_dims(g);
    if ((long long)d.G * d.N2 * d.M > (1LL << 31) - 1 || (long long)d.J * d.K2 * d.K3 * d.N2 * d.cbpad > (1LL << 31) - 1)
        return fail(GEO_SC_ERR_TOO_LARGE, "guide tensors exceed 31-bit indexing (groups %d x channels %d x positions %d)",
                    d.G, d.N2, d.M);
    if (!scratch_bytes) return fail(GEO_SC_ERR_NULL, "scratch_bytes is NULL");
    *scratch_bytes = guide_plan(d, g).total();
    return GEO_SC_OK;
}

}  // extern "C"

namespace geo {
namespace {

// Overwrites the gradients with NaN when the caller's promise of bf16-exact inputs did not hold.
__global__ void guide_poison_kernel(float *ga, long long na, float *gw, long long nw, const int *inexact) {
    if (!*inexact) return;
    const float nan = __int_as_float(0x7fc00000);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < na + nw; i += stride) {
        if (i < na) ga[i] = nan;
        else gw[i - na] = nan;
    }
}

int guide_backward_impl(const geo_sc_conv_desc *desc, const float *act, const float *weight, const float *grad_out,
                        float *grad_act, float *grad_weight, void *scratch, size_t scratch_bytes, void *stream,
                        bool promised_exact) {
    Geometry g;
    int rc = guide_geometry(desc, &g);
    if (rc) return rc;
    if (!act || !weight || !grad_out || !scratch) return fail(GEO_SC_ERR_NULL, "act, weight, grad_out or scratch is NULL");
    const GuideDims d = guide_dims(g);
    if ((long long)d.G * d.N2 * d.M > (1LL << 31) - 1 || (long long)d.J * d.K2 * d.K3 * d.N2 * d.cbpad > (1LL << 31) - 1)
        return fail(GEO_SC_ERR_TOO_LARGE, "guide tensors exceed 31-bit indexing");
    const GuidePlan p = guide_plan(d, g);
    if (scratch_bytes < p.total() || ((uintptr_t)scratch & 255))
        return fail(GEO_SC_ERR_WORKSPACE, "guide scratch holds %zu bytes, %zu needed (256-byte aligned)", scratch_bytes,
                    p.total());
    if (!grad_act && !grad_weight) return GEO_SC_OK;
    cudaStream_t s = (cudaStream_t)stream;
    char *base = (char *)scratch;
    float *D = (float *)base;
    float *apad = (float *)(base + p.d_bytes);
    int *aoff = (int *)(base + p.d_bytes + p.apad_bytes);
    float *wf = (float *)(base + p.d_bytes + p.apad_bytes + p.aoff_bytes);
    float *wd = (float *)(base + p.d_bytes + p.apad_bytes + p.aoff_bytes + p.wf_bytes);
    float *partial = (float *)(base + p.d_bytes + p.apad_bytes + p.aoff_bytes + p.wf_bytes + p.wd_bytes);
    void *mma_scratch = base + p.d_bytes + p.apad_bytes + p.aoff_bytes + p.wf_bytes + p.wd_bytes + p.partial_bytes;

    // Tensor-core path: does the whole backward pass when every input is bf16-exact, which is
    // decided on the device; the FFMA kernels below then return at once (and vice versa).
    int *inexact = nullptr;
    if (mma_eligible(g)) {
        rc = launch_mma_backward(g, act, weight, grad_out, grad_act, grad_weight, mma_scratch, &inexact, s);
        if (rc) return rc;
        if (promised_exact) {
            const long long na = grad_act ? (long long)d.B * d.C * d.H * d.W : 0;
            const long long nw = grad_weight ? (long long)d.O * d.C * d.K2 * d.K3 : 0;
            guide_poison_kernel<<<sm_count(), 256, 0, s>>>(grad_act, na, grad_weight, nw, inexact);
            GEO_CUDA_CHECK(cudaGetLastError());
            return GEO_SC_OK;
        }
    }
    pad_act_kernel<<<grid1d((long long)d.B * d.C * d.Hp * d.Wp), 256, 0, s>>>(d, act, apad);
    guide_prep_fwd_kernel<<<grid1d((long long)d.G * d.K * d.Opad), 256, 0, s>>>(d, weight, wf, aoff);
    GEO_CUDA_CHECK(cudaGetLastError());
    FwdParams fp;
    fp.apad = apad; fp.wf = wf; fp.aoff = aoff; fp.gout = grad_out; fp.D = D;
    fp.M = d.M; fp.O = d.O; fp.Opad = d.Opad; fp.HoWo = d.HoWo; fp.Wo = d.Wo; fp.Wp = d.Wp;
    fp.K = g.guide_linear ? 0 : d.K;   // no members: y = 0 and D = gout * exp(-0) = gout, the linear guide
    fp.img = d.C * d.Hp * d.Wp;
    fp.inexact = inexact;
    fp.vec_ok = (d.M % 4 == 0) && (d.HoWo % 4 == 0) && (((uintptr_t)grad_out & 15) == 0);
    switch (g.NT) {
    case 16: rc = launch_guide_fwd<16, 128>(d, fp, s); break;
    case 32: rc = launch_guide_fwd<32, 256>(d, fp, s); break;
    default: rc = launch_guide_fwd<64, 256>(d, fp, s); break;
    }
    if (rc) return rc;

    // 2. weight gradient
    if (grad_weight) {
        WgradParams pr;
        pr.apad = apad; pr.D = D; pr.aoff = aoff; pr.partial = partial;
        pr.M = d.M; pr.N2 = d.N2; pr.HoWo = d.HoWo; pr.Wo = d.Wo; pr.Wp = d.Wp; pr.K = d.K; pr.G = d.G;
        pr.img = d.C * d.Hp * d.Wp; pr.slice_len = p.slice_len;
        pr.inexact = inexact;
        switch (p.KT) {
        case 16: {
            constexpr size_t smem = (size_t)WSTAGE * (16 * WRS + WNT * WRS) * 4;
            dim3 grid(p.S, d.G, (d.N2 + WNT - 1) / WNT);
            guide_wgrad_smallk_kernel<<<grid, 128, smem, s>>>(pr);
            GEO_CUDA_CHECK(cudaGetLastError());
            break;
        }
        case 32: rc = launch_guide_wgrad<32>(d, p, pr, s); break;
        case 64: rc = launch_guide_wgrad<64>(d, p, pr, s); break;
        case 96: rc = launch_guide_wgrad<96>(d, p, pr, s); break;
        case 128: rc = launch_guide_wgrad<128>(d, p, pr, s); break;
        case 160: rc = launch_guide_wgrad<160>(d, p, pr, s); break;
        default: rc = launch_guide_wgrad<192>(d, p, pr, s); break;
        }
        if (rc) return rc;
        guide_wgrad_reduce_kernel<<<grid1d((long long)d.G * d.K * d.O), 256, 0, s>>>(d, p.S, partial, weight, grad_weight, inexact);
        GEO_CUDA_CHECK(cudaGetLastError());
    }
    // 3. activation gradient
    if (grad_act) {
        guide_prep_dgrad_kernel<<<grid1d((long long)d.J * d.K2 * d.K3 * d.N2 * d.cbpad), 256, 0, s>>>(d, weight, wd);
        GEO_CUDA_CHECK(cudaGetLastError());
        DgradParams pr;
        pr.D = D; pr.wd = wd; pr.ga = grad_act;
        pr.M = d.M; pr.N2 = d.N2; pr.Ho = d.Ho; pr.Wo = d.Wo; pr.H = d.H; pr.W = d.W; pr.C = d.C; pr.ph = d.ph; pr.pw = d.pw;
        pr.K2 = d.K2; pr.K3 = d.K3; pr.mode = d.mode; pr.cb = d.cb; pr.cbpad = d.cbpad; pr.Min = d.Min;
        pr.R = d.K2 * d.K3 * d.N2;
        pr.inexact = inexact;
        if (d.cbpad == 8) rc = launch_guide_dgrad<8, 64>(d, pr, s);
        else if (d.cbpad == 16) rc = launch_guide_dgrad<16, 128>(d, pr, s);
        else if (d.cbpad == 32) rc = launch_guide_dgrad<32, 128>(d, pr, s);
        else rc = launch_guide_dgrad<64, 256>(d, pr, s);
        if (rc) return rc;
    }
    return GEO_SC_OK;
}

}  // namespace
}  // namespace geo

extern "C" {

int geo_sc_guide_backward(const geo_sc_conv_desc *desc, const float *act, const float *weight, const float *grad_out,
                          float *grad_act, float *grad_weight, void *scratch, size_t scratch_bytes, void *stream) {
    return guide_backward_impl(desc, act, weight, grad_out, grad_act, grad_weight, scratch, scratch_bytes, stream, false);
}

int geo_sc_guide_backward_quantized(const geo_sc_conv_desc *desc, const float *act, const float *weight,
                                    const float *grad_out, float *grad_act, float *grad_weight, void *scratch,
                                    size_t scratch_bytes, void *stream) {
    return guide_backward_impl(desc, act, weight, grad_out, grad_act, grad_weight, scratch, scratch_bytes, stream, true);
}

}  // extern "C"
