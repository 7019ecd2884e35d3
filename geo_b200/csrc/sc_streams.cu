// LFSR bit-stream generation for weights and activations.
//
// The reference runs the LFSR bit by bit for every element (sc_cuda_kernel.cu:151-168,
// 678-690).  All six LFSRs are maximal length, so every seed is a phase into one state
// sequence s_0=1, s_1, ... of period L-1, and the stream of a value v seeded at phase f is
// the L-bit window starting at bit f+1 of the periodic pattern [v > s_j].  The patterns for
// all v are precomputed once per device ("pattern table", doubled so that a window never
// wraps) and a stream word becomes one funnel shift of two table words.  Progressive
// loading (sc_cuda_kernel.cu:156-160) only changes which truncation of v is visible
// during which bits; it is applied by merging the windows of the truncated values under
// constant bit masks.
#include <mutex>
#include <vector>

#include "sc_common.h"
#include "sc_pool.h"

namespace geo {

// ---- pattern tables ---------------------------------------------------------------------
// For stream length L: L rows (one per value) of RW(L) = max(2, 2*L/32) words holding two
// periods of [v > s_j], bit j at word j/32, bit 31-(j%32); and q0[seed] = (phase(seed)+1) mod (L-1).
constexpr int kNumL = 6;
__host__ __device__ constexpr int row_words(int L) { return L >= 32 ? 2 * (L / 32) : 2; }
constexpr int kTableWords = 8 * 2 + 16 * 2 + 32 * 2 + 64 * 4 + 128 * 8 + 256 * 16;

__device__ uint32_t g_pattern[kTableWords];
__device__ uint16_t g_q0[kNumL][256];

__host__ __device__ inline int l_index(int L) {  // 8->0 ... 256->5
    return L == 8 ? 0 : L == 16 ? 1 : L == 32 ? 2 : L == 64 ? 3 : L == 128 ? 4 : 5;
}
__host__ __device__ inline int table_offset(int L) {
    int off = 0;
    for (int l = 8; l < L; l *= 2) off += l * row_words(l);
    return off;
}

// One LFSR step (sc_cuda_kernel.cu:18-40 written with shifts): feedback = xor of the tap
// bits, shifted in at the bottom, top bit dropped.
static int lfsr_step_host(int v, int n) {
    static const int taps[9][4] = {{-1}, {-1}, {-1}, {2, 1, -1, -1}, {3, 2, -1, -1}, {4, 2, -1, -1},
                                   {5, 4, -1, -1}, {6, 5, -1, -1}, {7, 5, 4, 3}};
    int fb = 0;
    for (int i = 0; i < 4; i++)
        if (taps[n][i] >= 0) fb ^= (v >> taps[n][i]) & 1;
    return fb + 2 * (v & ((1 << (n - 1)) - 1));
}

static std::mutex g_table_mutex;
static bool g_table_ready[64] = {};
static std::vector<uint32_t> g_host_pattern;
static std::vector<uint16_t> g_host_q0;

// Builds the host copy of the tables (once per process).
static void build_host_tables() {
    if (!g_host_pattern.empty()) return;
    std::vector<uint32_t> pat(kTableWords, 0u);
    std::vector<uint16_t> q0(kNumL * 256, 0);
    for (int n = 3; n <= 8; n++) {
        const int L = 1 << n, period = L - 1, RW = row_words(L);
        std::vector<int> seq(period);
        int s = 1;
        for (int j = 0; j < period; j++) {
            seq[j] = s;
            q0[l_index(L) * 256 + s] = (uint16_t)((j + 1) % period);
            s = lfsr_step_host(s, n);
        }
        uint32_t *tab = pat.data() + table_offset(L);
        for (int v = 0; v < L; v++)
            for (int j = 0; j < 2 * period; j++)
                if (v > seq[j % period]) tab[v * RW + (j >> 5)] |= 1u << (31 - (j & 31));
    }
    g_host_q0.swap(q0);
    g_host_pattern.swap(pat);
}

int ensure_tables() {
    int dev = 0;
    GEO_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(GEO_SC_ERR_UNSUPPORTED, "device index %d", dev);
    std::lock_guard<std::mutex> lock(g_table_mutex);
    if (g_table_ready[dev]) return GEO_SC_OK;
    build_host_tables();
    GEO_CUDA_CHECK(cudaMemcpyToSymbol(g_pattern, g_host_pattern.data(), g_host_pattern.size() * sizeof(uint32_t)));
    GEO_CUDA_CHECK(cudaMemcpyToSymbol(g_q0, g_host_q0.data(), g_host_q0.size() * sizeof(uint16_t)));
    g_table_ready[dev] = true;
    return GEO_SC_OK;
}

// ---- device helpers -----------------------------------------------------------------------
struct GenParams {
    int B, C, H, W, pad_h, pad_w, Hp, Wp;
    int O, K2, K3;
    int L, P, mode, z, G, K, Kp, Opad;
    int RW;    // words per pattern row in the global table
    int RWS;   // ... in shared memory: odd, so that the rows of different values fall into different banks
    // activation-stream image: word(b, p, c, yx) = b * img_stride + p * pack_stride + (c * Hp * Wp + yx) * pix_stride
    // ([batch][pack][c][Hp][Wp], or batch-innermost [pack][c][Hp][Wp][Bp]: see act_img_words)
    int batch_fast, Bp;
    unsigned img_stride, pack_stride, pix_stride;
};

static GenParams gen_params(const Geometry &g) {
    GenParams p;
    p.B = g.B; p.C = g.C; p.H = g.H; p.W = g.W; p.pad_h = g.pad_h; p.pad_w = g.pad_w; p.Hp = g.Hp; p.Wp = g.Wp;
    p.O = g.O; p.K2 = g.K2; p.K3 = g.K3;
    p.L = g.L; p.P = g.P; p.mode = g.mode; p.z = g.z; p.G = g.G; p.K = g.K; p.Kp = g.Kp; p.Opad = g.Opad;
    p.RW = row_words(g.L);
    p.RWS = p.RW | 1;
    p.batch_fast = g.batch_fast;
    p.Bp = g.Bp;
    p.img_stride = (unsigned)act_img_words(g);
    p.pack_stride = (unsigned)act_pack_words(g);
    p.pix_stride = (unsigned)act_pixel_stride(g);
    return p;
}

// Copies the pattern table and phase table for stream length L into shared memory.
__device__ __forceinline__ void load_tables(uint32_t *s_pat, uint16_t *s_q0, int L, int RW, int RWS) {
    const uint32_t *src = g_pattern + table_offset(L);
    for (int i = threadIdx.x; i < L * RW; i += blockDim.x) s_pat[(i / RW) * RWS + i % RW] = src[i];
    const uint16_t *q = g_q0[l_index(L)];
    for (int i = threadIdx.x; i < L; i += blockDim.x) s_q0[i] = q[i];
    __syncthreads();
}

__host__ __device__ __forceinline__ uint32_t funnel_left(uint32_t lo, uint32_t hi, int sh) {
#ifdef __CUDA_ARCH__
    return __funnelshift_l(lo, hi, sh);
#else
    return sh ? (hi << sh) | (lo >> (32 - sh)) : hi;
#endif
}

// Stream word `p` of value V whose generator starts at window offset q0.
__host__ __device__ __forceinline__ uint32_t stream_word(const uint32_t *s_pat, int RW, int L, int V, int q0, int p,
                                                         const LoadPlan &plan) {
    uint32_t word = 0;
    const int q = q0 + 32 * p;
    const int i = q >> 5, sh = q & 31;
    const int n = plan.nact[p];
    for (int e = 0; e < n; e++) {
        const int j = plan.act[p][e];
        const int vj = (V >> plan.shift[j]) << plan.shift[j];
        const uint32_t *row = s_pat + vj * RW;
        uint32_t w32 = funnel_left(row[i + 1], row[i], sh);
        if (L < 32) w32 >>= (32 - L);
        word |= w32 & plan.mask[p][j];
    }
    return word;
}

// Filter coordinates (c, ky, kx) and LFSR generator index of member k of group g.
__device__ __forceinline__ void decode_weight_member(const GenParams &gp, int g, int k, int *c, int *ky, int *kx, int *sidx) {
    switch (gp.mode) {
    case GEO_SC_MODE_1D: *kx = g; *c = k / gp.K2; *ky = k % gp.K2; *sidx = k; break;
    case GEO_SC_MODE_Z: *c = g; *ky = k / gp.K3; *kx = k % gp.K3; *sidx = k; break;
    case GEO_SC_MODE_YZ: {
        const int zp = g / gp.K3;
        *kx = g % gp.K3;
        *c = zp * gp.z + k / gp.K2;
        *ky = k % gp.K2;
        *sidx = k;
        break;
    }
    case GEO_SC_MODE_2D: *ky = g / gp.K3; *kx = g % gp.K3; *c = k; *sidx = k; break;   // generators indexed by channel
    case GEO_SC_MODE_FULL_BIN:   // every filter element is a group of its own; generators as in full_or
        *c = g / (gp.K2 * gp.K3); *ky = (g / gp.K3) % gp.K2; *kx = g % gp.K3; *sidx = g;
        break;
    default: *c = k / (gp.K2 * gp.K3); *ky = (k / gp.K3) % gp.K2; *kx = k % gp.K3; *sidx = k; break;
    }
}

// ---- weight streams -----------------------------------------------------------------------
// One thread per (group, member, padded c_out); writes the positive and negative stream words
// of every pack as one 8-byte store, layout [pack][group][member][c_out_padded][2], and the
// activation offset of each (group, member).
__global__ void __launch_bounds__(256) prepare_weights_kernel(GenParams gp, LoadPlan plan, const float *__restrict__ w,
                                                              uint32_t *__restrict__ ws, int32_t *__restrict__ aoff) {
    extern __shared__ uint32_t smem[];
    uint32_t *s_pat = smem;
    uint16_t *s_q0 = (uint16_t *)(smem + gp.L * gp.RWS);
    load_tables(s_pat, s_q0, gp.L, gp.RW, gp.RWS);

    // 32-bit index arithmetic: the geometry check bounds the prepared streams by 2^31 words
    const unsigned total = (unsigned)gp.G * (unsigned)gp.Kp * (unsigned)gp.Opad;
    const float fL = (float)gp.L;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int o = (int)(idx % (unsigned)gp.Opad);
        const int gk = (int)(idx / (unsigned)gp.Opad);
        const int k = gk % gp.Kp, g = gk / gp.Kp;   // k >= K: padding member, zero streams
        int c, ky, kx, sidx;
        decode_weight_member(gp, g, k, &c, &ky, &kx, &sidx);
        const bool valid = c < gp.C && k < gp.K;
        if (o == 0) aoff[gk] = valid ? (c * gp.Hp + ky) * gp.Wp + kx : 0;
        int Vp = 0, Vn = 0;
        if (valid && o < gp.O) {
            const float x = w[(((size_t)o * gp.C + c) * gp.K2 + ky) * gp.K3 + kx] * fL;
            Vp = (int)ceilf(fminf(fmaxf(x, 0.0f), fL - 1.0f));
            Vn = (int)ceilf(-fminf(fmaxf(x, 1.0f - fL), 0.0f));
        }
        const int qp = s_q0[(67 + sidx) % (gp.L - 1) + 1];
        const int qn = s_q0[(37 + sidx) % (gp.L - 1) + 1];
        for (int p = 0; p < gp.P; p++) {
            uint2 v;
            v.x = Vp ? stream_word(s_pat, gp.RWS, gp.L, Vp, qp, p, plan) : 0u;
            v.y = Vn ? stream_word(s_pat, gp.RWS, gp.L, Vn, qn, p, plan) : 0u;
            *(uint2 *)(ws + ((((size_t)p * gp.G + g) * gp.Kp + k) * gp.Opad + o) * 2) = v;
        }
    }
}

// ---- activation streams ---------------------------------------------------------------------
// One thread per element of the padded image; fuses zero padding and the float -> level
// quantisation (sc_cuda.cpp:50-51).  Layout [batch][pack][c][Hp][Wp].
// 32-bit index arithmetic: the geometry check bounds the padded tensor by 2^31 elements, and 64-bit
// divisions would cost several times the stream generation itself.
__global__ void __launch_bounds__(256) act_streams_kernel(GenParams gp, LoadPlan plan, const float *__restrict__ act,
                                                          uint32_t *__restrict__ as) {
    extern __shared__ uint32_t smem[];
    uint32_t *s_pat = smem;
    uint16_t *s_q0 = (uint16_t *)(smem + gp.L * gp.RWS);
    load_tables(s_pat, s_q0, gp.L, gp.RW, gp.RWS);

    const unsigned plane = (unsigned)(gp.Hp * gp.Wp);
    const unsigned total = (unsigned)gp.B * gp.C * plane;
    const float fL = (float)gp.L;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const unsigned yx = idx % plane, bc = idx / plane;
        const unsigned c = bc % (unsigned)gp.C, b = bc / (unsigned)gp.C;
        const int y = (int)(yx / (unsigned)gp.Wp), x = (int)(yx % (unsigned)gp.Wp);
        const int yi = y - gp.pad_h, xi = x - gp.pad_w;
        int V = 0;
        if (yi >= 0 && yi < gp.H && xi >= 0 && xi < gp.W) {
            const float a = act[(((size_t)b * gp.C + c) * gp.H + yi) * gp.W + xi] * fL;
            V = (int)ceilf(fminf(fmaxf(a, 0.0f), fL - 1.0f));
        }
        const int cc = gp.mode == GEO_SC_MODE_YZ ? (int)c % gp.z : (int)c;
        const unsigned sidx = (unsigned)((cc * gp.Hp + y) * gp.Wp + x);
        const int q0 = s_q0[sidx % (unsigned)(gp.L - 1) + 1];
        uint32_t *dst = as + ((size_t)b * gp.P * gp.C + c) * plane + yx;
        for (int p = 0; p < gp.P; p++)
            dst[(size_t)p * gp.C * plane] = V ? stream_word(s_pat, gp.RWS, gp.L, V, q0, p, plan) : 0u;
    }
}

// The same for a batch-innermost stream image ([pack][c][Hp][Wp][Bp]): a CTA turns tiles of 32 images x 32
// elements of the padded image through shared memory, so that the activation reads run along an image row and the
// stream-word stores along the batch -- both consecutive.  Images past the batch are written as zeros.
__global__ void __launch_bounds__(256) act_streams_batch_kernel(GenParams gp, LoadPlan plan, const float *__restrict__ act,
                                                                uint32_t *__restrict__ as) {
    extern __shared__ uint32_t smem[];
    uint32_t *s_pat = smem;
    uint16_t *s_q0 = (uint16_t *)(smem + gp.L * gp.RWS);
    __shared__ uint16_t s_level[32][33];
    load_tables(s_pat, s_q0, gp.L, gp.RW, gp.RWS);

    const unsigned plane = (unsigned)(gp.Hp * gp.Wp);
    const unsigned E = (unsigned)gp.C * plane;   // elements of one padded image
    const unsigned nbt = ((unsigned)gp.Bp + 31) / 32, net = (E + 31) / 32;
    const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const float fL = (float)gp.L;
    for (unsigned tile = blockIdx.x; tile < nbt * net; tile += gridDim.x) {
        const unsigned b0 = (tile % nbt) * 32, e0 = (tile / nbt) * 32;
        {   // lanes along the elements: the level of element e0 + tx in images b0 + ty, + 8, ...
            const unsigned e = e0 + tx, c = e / plane, yx = e % plane;
            const int yi = (int)(yx / (unsigned)gp.Wp) - gp.pad_h, xi = (int)(yx % (unsigned)gp.Wp) - gp.pad_w;
            const bool inside = e < E && yi >= 0 && yi < gp.H && xi >= 0 && xi < gp.W;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const unsigned b = b0 + ty + 8 * k;
                int V = 0;
                if (inside && b < (unsigned)gp.B) {
                    const float a = act[(((size_t)b * gp.C + c) * gp.H + yi) * gp.W + xi] * fL;
                    V = (int)ceilf(fminf(fmaxf(a, 0.0f), fL - 1.0f));
                }
                s_level[ty + 8 * k][tx] = (uint16_t)V;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; k++) {   // lanes along the batch: the stream words of element e0 + ty + 8k in image b0 + tx
            const unsigned e = e0 + ty + 8 * k, b = b0 + tx;
            if (e < E && b < (unsigned)gp.Bp) {
                const int V = s_level[tx][ty + 8 * k];
                const unsigned c = e / plane, yx = e % plane;
                const unsigned sidx = gp.mode == GEO_SC_MODE_YZ ? (c % (unsigned)gp.z) * plane + yx : e;
                const int q0 = s_q0[sidx % (unsigned)(gp.L - 1) + 1];
                uint32_t *dst = as + (size_t)e * gp.pix_stride + b;
                for (int p = 0; p < gp.P; p++)
                    dst[(size_t)p * gp.pack_stride] = V ? stream_word(s_pat, gp.RWS, gp.L, V, q0, p, plan) : 0u;
            }
        }
        __syncthreads();
    }
}

// ---- fused layer epilogue ---------------------------------------------------------------------
// What lies between two SC layers of the reference (network.py:165-184, utils_class.py:32-33,37-65), from the
// bit counts of one layer to the packed streams of the next in one pass: x = counts / L, batch norm with the
// folded 7-bit scale and shift, 2x2 average pool, hardtanh(0, 1), fixed-point rounding of the activation
// (utils_functional.py:33-39), float -> level (sc_cuda.cpp:50-51) and the stream words of every pack, written
// into the next layer's padded stream image [batch][pack][c][Hp][Wp] (whose border the launcher has zeroed).
// The rounded activation is also written as fp32: the backward pass of the next layer reads it.
// A thread owns two horizontally adjacent pooled values = one 16-byte load from each of two input rows.
// `gp` describes the NEXT layer: C, H, W are the pooled tensor's dimensions.
__global__ void __launch_bounds__(256) epilogue_streams_kernel(GenParams gp, LoadPlan plan, XSource xs,
                                                               const float *__restrict__ wq, const float *__restrict__ bq,
                                                               float qlevels, float qinv, float *__restrict__ act_out,
                                                               uint32_t *__restrict__ as) {
    extern __shared__ uint32_t smem[];
    uint32_t *s_pat = smem;
    uint16_t *s_q0 = (uint16_t *)(smem + gp.L * gp.RWS);
    load_tables(s_pat, s_q0, gp.L, gp.RW, gp.RWS);

    const unsigned Wx = 2u * (unsigned)gp.W;                 // width of the counts
    const unsigned q = Wx >> 2, rows = (unsigned)gp.B * gp.C * gp.H, total = rows * q;
    const float fL = (float)gp.L;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const unsigned r = i / q, j = i % q;                 // r = (b * C + c) * H + oy
        const unsigned oy = r % (unsigned)gp.H, bc = r / (unsigned)gp.H;
        const unsigned c = bc % (unsigned)gp.C, b = bc / (unsigned)gp.C;
        const float w = wq[c], sh = bq[c];
        const float4 t = load_x4(xs, ((size_t)(2 * r) * Wx >> 2) + j);
        const float4 u = load_x4(xs, ((size_t)(2 * r + 1) * Wx >> 2) + j);
        float v[2] = {pooled_value(t.x, t.y, u.x, u.y, w, sh), pooled_value(t.z, t.w, u.z, u.w, w, sh)};
#pragma unroll
        for (int e = 0; e < 2; e++) v[e] = quantize_value(fminf(fmaxf(v[e], 0.0f), 1.0f), qlevels, qinv);
        ((float2 *)(act_out + (size_t)r * gp.W))[j] = make_float2(v[0], v[1]);
        const int cc = gp.mode == GEO_SC_MODE_YZ ? (int)c % gp.z : (int)c;
        const unsigned y = oy + (unsigned)gp.pad_h;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const unsigned x = 2 * j + e + (unsigned)gp.pad_w;
            const int V = (int)ceilf(fminf(fmaxf(v[e] * fL, 0.0f), fL - 1.0f));
            const unsigned sidx = (unsigned)((cc * gp.Hp + (int)y) * gp.Wp + (int)x);
            const int q0 = s_q0[sidx % (unsigned)(gp.L - 1) + 1];
            uint32_t *dst = as + (size_t)b * gp.img_stride + ((size_t)c * (unsigned)(gp.Hp * gp.Wp) + y * (unsigned)gp.Wp + x) * gp.pix_stride;
            for (int p = 0; p < gp.P; p++)
                dst[(size_t)p * gp.pack_stride] = V ? stream_word(s_pat, gp.RWS, gp.L, V, q0, p, plan) : 0u;
        }
    }
}

// The same pass for a batch-innermost stream image ([pack][c][Hp][Wp][Bp]).  A CTA turns tiles of 32 images x 32
// pooled elements through shared memory: with the lanes along the elements it reads the counts (8 bytes per lane
// and input row, consecutive), evaluates batch norm, pool, hardtanh and rounding and writes the fp32 activation
// (consecutive); with the lanes along the batch it writes the stream words (consecutive).  (With one image per thread
// and no turn every stream word was a 4-byte store into a sector of its own: 5 % of the VGG-11-style step at 2048
// images.)
__global__ void __launch_bounds__(256) epilogue_streams_batch_kernel(GenParams gp, LoadPlan plan, XSource xs,
                                                                     const float *__restrict__ wq, const float *__restrict__ bq,
                                                                     float qlevels, float qinv, float *__restrict__ act_out,
                                                                     uint32_t *__restrict__ as) {
    extern __shared__ uint32_t smem[];
    uint32_t *s_pat = smem;
    uint16_t *s_q0 = (uint16_t *)(smem + gp.L * gp.RWS);
    __shared__ uint16_t s_level[32][33];
    load_tables(s_pat, s_q0, gp.L, gp.RW, gp.RWS);

    const unsigned HW = (unsigned)(gp.H * gp.W), E = (unsigned)gp.C * HW;   // pooled elements of one image
    const unsigned plane = (unsigned)(gp.Hp * gp.Wp);
    const unsigned nbt = ((unsigned)gp.Bp + 31) / 32, net = (E + 31) / 32;
    const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const float fL = (float)gp.L;
    for (unsigned tile = blockIdx.x; tile < nbt * net; tile += gridDim.x) {
        const unsigned b0 = (tile % nbt) * 32, e0 = (tile / nbt) * 32;
        {   // lanes along the pooled elements
            const unsigned e = e0 + tx, c = e / HW, rem = e % HW, oy = rem / (unsigned)gp.W, ox = rem % (unsigned)gp.W;
            const float w = e < E ? wq[c] : 0.0f, sh = e < E ? bq[c] : 0.0f;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const unsigned b = b0 + ty + 8 * k;
                int V = 0;
                if (e < E && b < (unsigned)gp.B) {
                    const size_t r = ((size_t)b * gp.C + c) * gp.H + oy;             // pooled row; counts rows 2r, 2r + 1
                    const float2 t = load_x2(xs, (size_t)(2 * r) * gp.W + ox);       // counts are 2 W wide: W pairs per row
                    const float2 u = load_x2(xs, (size_t)(2 * r + 1) * gp.W + ox);
                    float v = pooled_value(t.x, t.y, u.x, u.y, w, sh);
                    v = quantize_value(fminf(fmaxf(v, 0.0f), 1.0f), qlevels, qinv);
                    act_out[(size_t)b * E + e] = v;
                    V = (int)ceilf(fminf(fmaxf(v * fL, 0.0f), fL - 1.0f));
                }
                s_level[ty + 8 * k][tx] = (uint16_t)V;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; k++) {   // lanes along the batch
            const unsigned e = e0 + ty + 8 * k, b = b0 + tx;
            if (e < E && b < (unsigned)gp.Bp) {
                const int V = s_level[tx][ty + 8 * k];
                const unsigned c = e / HW, rem = e % HW, oy = rem / (unsigned)gp.W, ox = rem % (unsigned)gp.W;
                const unsigned yx = (oy + (unsigned)gp.pad_h) * (unsigned)gp.Wp + ox + (unsigned)gp.pad_w;
                const unsigned sidx = (gp.mode == GEO_SC_MODE_YZ ? c % (unsigned)gp.z : c) * plane + yx;
                const int q0 = s_q0[sidx % (unsigned)(gp.L - 1) + 1];
                uint32_t *dst = as + ((size_t)c * plane + yx) * gp.pix_stride + b;
                for (int p = 0; p < gp.P; p++)
                    dst[(size_t)p * gp.pack_stride] = V ? stream_word(s_pat, gp.RWS, gp.L, V, q0, p, plan) : 0u;
            }
        }
        __syncthreads();
    }
}

// ---- "accurate" generator ---------------------------------------------------------------------------
// Sampling without replacement (utils_functional.py:157-176): with cur ones still to place and L - k bits
// left, bit k is one when cur * L / (L - k) exceeds a uniform integer below L -- so a stream of level V
// holds exactly V ones.  The reference draws the integers from a random generator; here they are a hash
// of (seed, generator id, bit index), so a seed reproduces its streams.  Every activation element and
// every weight has its own generator id.  Bits are packed like the LFSR streams (MSB first).
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352dU;
    x ^= x >> 15; x *= 0x846ca68bU;
    x ^= x >> 16;
    return x;
}

// Writes the packs of one stream through `put(pack, word)`.  RAND: independent bits, each one when the level
// exceeds a fresh uniform integer below L (utils_functional.py:92-102,148-150); `id` is then the shared
// generator index, so that streams that share a generator see the same integers.
template <bool RAND, typename Put>
__device__ __forceinline__ void acc_stream(uint32_t seed, uint32_t id, int V, int L, int P, Put put) {
    const uint32_t base = mix32(seed ^ mix32(id + 0x9E3779B9u));
    const int bits = L < 32 ? L : 32;
    int cur = V;
    for (int p = 0; p < P; p++) {
        uint32_t word = 0;
        for (int i = 0; i < bits; i++) {
            const int k = p * 32 + i;
            const uint32_t r = mix32(base + (uint32_t)k * 0x85EBCA6Bu) >> (32 - 8) & (uint32_t)(L - 1);   // L <= 256
            const uint32_t bit = RAND ? ((uint32_t)V > r ? 1u : 0u) : ((uint32_t)(cur * L) > r * (uint32_t)(L - k) ? 1u : 0u);
            cur -= (int)bit;
            word = (word << 1) | bit;
        }
        put(p, word);
    }
}

template <bool RAND>
__global__ void __launch_bounds__(256) act_streams_acc_kernel(GenParams gp, uint32_t seed, const float *__restrict__ act,
                                                              uint32_t *__restrict__ as) {
    const unsigned plane = (unsigned)(gp.Hp * gp.Wp);
    const unsigned nb = (unsigned)(gp.batch_fast ? gp.Bp : gp.B);
    const unsigned total = nb * gp.C * plane;
    const float fL = (float)gp.L;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        unsigned yx, uc, b;
        if (gp.batch_fast) { b = idx % nb; const unsigned r = idx / nb; yx = r % plane; uc = r / plane; }
        else { yx = idx % plane; const unsigned bc = idx / plane; uc = bc % (unsigned)gp.C; b = bc / (unsigned)gp.C; }
        const int c = (int)uc;
        const int y = (int)(yx / (unsigned)gp.Wp), x = (int)(yx % (unsigned)gp.Wp);
        const int yi = y - gp.pad_h, xi = x - gp.pad_w;
        int V = 0;
        if (yi >= 0 && yi < gp.H && xi >= 0 && xi < gp.W && b < (unsigned)gp.B) {
            const float a = act[(((size_t)b * gp.C + c) * gp.H + yi) * gp.W + xi] * fL;
            V = (int)ceilf(fminf(fmaxf(a, 0.0f), fL - 1.0f));
        }
        uint32_t *dst = as + (size_t)b * gp.img_stride + ((size_t)c * plane + yx) * gp.pix_stride;
        const size_t pstride = gp.pack_stride;
        // ACC: one generator per element; RAND: one per (channel, y, x), shared over the batch like the LFSR seeds
        const int cc = gp.mode == GEO_SC_MODE_YZ ? c % gp.z : c;
        const uint32_t id = RAND ? (uint32_t)(cc * (int)plane) + yx : ((uint32_t)b * (uint32_t)gp.C + (uint32_t)c) * plane + yx;
        acc_stream<RAND>(seed, id, V, gp.L, gp.P, [&](int p, uint32_t w) { dst[(size_t)p * pstride] = w; });
    }
}

// Weight streams of the accurate generator: same layout as prepare_weights_kernel; generator id =
// index of (polarity, c_out, c, ky, kx), offset so that it never meets an activation's id.
template <bool RAND>
__global__ void __launch_bounds__(256) prepare_weights_acc_kernel(GenParams gp, uint32_t seed, const float *__restrict__ w,
                                                                  uint32_t *__restrict__ ws, int32_t *__restrict__ aoff) {
    const long long total = (long long)gp.G * gp.Kp * gp.Opad;
    const float fL = (float)gp.L;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int o = (int)(idx % gp.Opad);
        const int gk = (int)(idx / gp.Opad);
        const int k = gk % gp.Kp, g = gk / gp.Kp;
        int c, ky, kx, sidx;
        decode_weight_member(gp, g, k, &c, &ky, &kx, &sidx);
        const bool valid = c < gp.C && k < gp.K;
        if (o == 0) aoff[gk] = valid ? (c * gp.Hp + ky) * gp.Wp + kx : 0;
        int Vp = 0, Vn = 0;
        uint32_t id = 0;
        if (valid && o < gp.O) {
            const uint32_t e = (uint32_t)((((size_t)o * gp.C + c) * gp.K2 + ky) * gp.K3 + kx);
            const float x = w[e] * fL;
            Vp = (int)ceilf(fminf(fmaxf(x, 0.0f), fL - 1.0f));
            Vn = (int)ceilf(-fminf(fmaxf(x, 1.0f - fL), 0.0f));
            // ACC: one generator per weight and polarity; RAND: one per LFSR generator index and polarity
            id = 0x80000000u + 2u * (RAND ? (uint32_t)sidx : e);
        }
        uint32_t *dst = ws + ((size_t)g * gp.Kp + k) * gp.Opad * 2 + (size_t)o * 2;
        const size_t pstride = (size_t)gp.G * gp.Kp * gp.Opad * 2;
        acc_stream<RAND>(seed, id, Vp, gp.L, gp.P, [&](int p, uint32_t v) { dst[(size_t)p * pstride] = v; });
        acc_stream<RAND>(seed, id + 1, Vn, gp.L, gp.P, [&](int p, uint32_t v) { dst[(size_t)p * pstride + 1] = v; });
    }
}

static int grid_for(long long total) {
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    return (int)(blocks < cap ? blocks : cap);
}

int launch_prepare_weights(const Geometry &g, const float *w, uint32_t *wstream, int32_t *aoff, cudaStream_t s) {
    int rc = ensure_tables();
    if (rc) return rc;
    GenParams gp = gen_params(g);
    LoadPlan plan;
    make_load_plan(g.L, g.tw, g.lu, g.lw_w, &plan);
    const size_t smem = (size_t)g.L * gp.RWS * 4 + (size_t)g.L * 2;
    const long long total = (long long)g.G * g.Kp * g.Opad;
    if (g.generator == GEO_SC_GEN_ACC) prepare_weights_acc_kernel<false><<<grid_for(total), 256, 0, s>>>(gp, g.seed, w, wstream, aoff);
    else if (g.generator == GEO_SC_GEN_RAND) prepare_weights_acc_kernel<true><<<grid_for(total), 256, 0, s>>>(gp, g.seed, w, wstream, aoff);
    else prepare_weights_kernel<<<grid_for(total), 256, smem, s>>>(gp, plan, w, wstream, aoff);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_act_streams(const Geometry &g, const float *act, uint32_t *astream, cudaStream_t s) {
    int rc = ensure_tables();
    if (rc) return rc;
    GenParams gp = gen_params(g);
    LoadPlan plan;
    make_load_plan(g.L, g.tw, g.lu, g.lw_a, &plan);
    const size_t smem = (size_t)g.L * gp.RWS * 4 + (size_t)g.L * 2;
    const long long total = (long long)(g.batch_fast ? g.Bp : g.B) * g.C * g.Hp * g.Wp;
    if (g.generator == GEO_SC_GEN_ACC) act_streams_acc_kernel<false><<<grid_for(total), 256, 0, s>>>(gp, g.seed, act, astream);
    else if (g.generator == GEO_SC_GEN_RAND) act_streams_acc_kernel<true><<<grid_for(total), 256, 0, s>>>(gp, g.seed, act, astream);
    else if (g.batch_fast) {
        const long long tiles = (long long)((g.Bp + 31) / 32) * (((long long)g.C * g.Hp * g.Wp + 31) / 32);
        act_streams_batch_kernel<<<grid_for(tiles * 256), 256, smem, s>>>(gp, plan, act, astream);
    } else act_streams_kernel<<<grid_for(total), 256, smem, s>>>(gp, plan, act, astream);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_epilogue_streams(const Geometry &g, const XSource &xs, const float *wq, const float *bq, int prec, float *act_out,
                            uint32_t *astream, cudaStream_t s) {
    int rc = ensure_tables();
    if (rc) return rc;
    GenParams gp = gen_params(g);
    LoadPlan plan;
    make_load_plan(g.L, g.tw, g.lu, g.lw_a, &plan);
    const size_t smem = (size_t)g.L * gp.RWS * 4 + (size_t)g.L * 2;
    // the kernel writes the interior of every padded image; the border holds the all-zero streams of level 0
    if (g.pad_h || g.pad_w || (g.batch_fast && g.Bp != g.B)) GEO_CUDA_CHECK(cudaMemsetAsync(astream, 0, g.act_stream_words * 4, s));
    const float levels = (float)(1 << prec);
    if (g.batch_fast) {
        const long long tiles = (long long)((g.Bp + 31) / 32) * (((long long)g.C * g.H * g.W + 31) / 32);
        epilogue_streams_batch_kernel<<<grid_for(tiles * 256), 256, smem, s>>>(gp, plan, xs, wq, bq, levels, 1.0f / levels, act_out,
                                                                               astream);
    } else {
        const long long total = (long long)g.B * g.C * g.H * (g.W / 2);
        epilogue_streams_kernel<<<grid_for(total), 256, smem, s>>>(gp, plan, xs, wq, bq, levels, 1.0f / levels, act_out, astream);
    }
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

}  // namespace geo

// Host mirror of the device stream generator (same tables, same plan, same word function):
// the packed stream of integer level `value` for generator index `seed_index` and seed base
// `seed_base` (67 / 37 for positive / negative weights, 0 for activations).
extern "C" int geo_sc_host_stream(int bit_length, int value, int seed_base, int seed_index, int total_width,
                                  int load_width, int load_wait, uint32_t *words) {
    using namespace geo;
    if (!words) return fail(GEO_SC_ERR_NULL, "words is NULL");
    geo_sc_conv_desc d = {1, 1, 1, 1, 0, 0, 1, 1, 1, bit_length, GEO_SC_MODE_1D, 1, total_width, load_width,
                          load_wait, load_wait};
    Geometry g;
    int rc = make_geometry(&d, &g);
    if (rc) return rc;
    if (value < 0 || value >= bit_length) return fail(GEO_SC_ERR_SHAPE, "value %d outside [0,%d)", value, bit_length);
    if (seed_base < 0 || seed_index < 0) return fail(GEO_SC_ERR_SHAPE, "negative seed");
    {
        std::lock_guard<std::mutex> lock(g_table_mutex);
        build_host_tables();
    }
    LoadPlan plan;
    make_load_plan(g.L, g.tw, g.lu, load_wait, &plan);
    const int RW = row_words(g.L);
    const uint32_t *pat = g_host_pattern.data() + table_offset(g.L);
    const int seed = (int)(((long long)seed_base + seed_index) % (g.L - 1)) + 1;
    const int q0 = g_host_q0[l_index(g.L) * 256 + seed];
    for (int p = 0; p < g.P; p++) words[p] = value ? stream_word(pat, RW, g.L, value, q0, p, plan) : 0u;
    return GEO_SC_OK;
}
