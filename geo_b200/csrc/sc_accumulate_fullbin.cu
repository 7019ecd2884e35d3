// SC accumulation without OR (GEO_SC_MODE_FULL_BIN) as a binary GEMM on the tensor cores.
//
// full_bin counts every product bit: out[m][o] = sum over members k and packs p of
//     popc(A[m][k][p] & W+[k][o][p]) - popc(A[m][k][p] & W-[k][o][p]),
// which is a GEMM over bits with AND as the product and popcount as the sum -- exactly what
// mma.sync.m16n8k256.b1.and.popc computes (16 positions x 8 columns x 256 bits per instruction, s32
// accumulators).  It is the one accumulation mode of this path that a tensor-core instruction maps to:
// the OR modes need OR inside a group before anything is counted, and no MMA has that.
//
// Layout.  Columns are (polarity, channel) pairs; a CTA of four warps owns 128 positions x 64 columns =
// 32 channels x {+, -}, so that the subtraction of the two polarities happens in registers.  The reduction
// runs over words kw = member * packs + pack in stages of 32 words (four MMA k-steps).  An MMA thread
// (group g = lane / 4, t = lane % 4) needs words t and t + 4 of each 8-word k-step, for A rows g and g + 8 and
// for B column g; the four k-steps of a stage are stored so that these eight words are 32 consecutive bytes
// (word j of a stage sits at position (j % 4) * 8 + (j / 8) * 2 + (j % 8) / 4), read with two 16-byte loads.
// A and B use the same order, and AND/popcount does not care in which order bits are summed.
// Weights are packed into that order once, when they are prepared; activation words are gathered from the
// stream image with 4-byte cp.async through the member offset table (implicit im2col), three stages deep.
#include "sc_common.h"
#include "sc_fullbin.h"

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
__device__ __forceinline__ void mma_b1(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int FB_STAGE_WORDS = 32;   // words of the reduction per stage: four k-steps of 256 bits
constexpr int FB_NSTAGE = 3;
constexpr int FB_A_BYTES = 128 * FB_STAGE_WORDS * 4;   // 128 positions
constexpr int FB_B_BYTES = 64 * FB_STAGE_WORDS * 4;    // 64 columns
constexpr int FB_STAGE_BYTES = FB_A_BYTES + FB_B_BYTES;

// Position of word j (0..31) of a stage inside a row: see the file comment.
__host__ __device__ __forceinline__ int frag_pos(int j) { return (j & 3) * 8 + (j >> 3) * 2 + ((j >> 2) & 1); }
// Byte offset inside a 128-byte row, with odd rows shifted by one 16-byte chunk so that the two rows a quarter
// warp reads fall into different banks.
__device__ __forceinline__ uint32_t row_byte(int row, int byte) { return (uint32_t)(row * 128 + (byte ^ ((row & 1) << 4))); }

struct FullBinParams {
    const uint32_t *as;     // [B][P][C][Hp][Wp]
    const int32_t *aoff;    // [K][4]: entry 0 of each group is the member's activation offset
    const uint32_t *wb;     // [CT][NST][64 columns][32 words in fragment order]
    int32_t *out;           // [B][O][Ho][Wo]
    int M, O, HoWo, Wo, Wp;
    int P, K, KW, NST;      // K filter elements (members), KW = K * P words, NST = stages = ceil(KW / 32)
    int img_words, pack_words, aoff_mul;
    int splits;
};

__global__ void __launch_bounds__(128, 3) accumulate_fullbin_kernel(FullBinParams pr) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int m0 = blockIdx.x * 128, ct = blockIdx.y;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);

    // gather: lane = word of the stage, warp w copies rows w, w + 4, ...: the 32 lanes of a copy instruction write the
    // 32 words of one row (32 banks), where one row per lane would put the whole warp on two banks
    __shared__ int s_abase[128];
    {
        int m = m0 + t;
        if (m >= pr.M) m = pr.M - 1;
        const int b = m / pr.HoWo, rem = m % pr.HoWo;
        s_abase[t] = b * pr.img_words + ((rem / pr.Wo) * pr.Wp + (rem % pr.Wo)) * pr.aoff_mul;
    }
    __syncthreads();
    const int st0 = (int)((long long)pr.NST * blockIdx.z / pr.splits);
    const int st1 = (int)((long long)pr.NST * (blockIdx.z + 1) / pr.splits);
    int ld = st0;
    const uint32_t word_byte = (uint32_t)frag_pos(lane) * 4;
    auto issue = [&]() {
        if (ld < st1) {
            const uint32_t a_s = smem_base + (uint32_t)((ld - st0) % FB_NSTAGE) * FB_STAGE_BYTES, b_s = a_s + FB_A_BYTES;
            // this lane's word of the stage: member k, pack p; words past the last member read member 0 (weights zero)
            const int kw = ld * FB_STAGE_WORDS + lane;
            int k = kw / pr.P;
            const int p = kw - k * pr.P;
            if (k >= pr.K) k = 0;
            const uint32_t *src = pr.as + (size_t)p * pr.pack_words + (size_t)__ldg(pr.aoff + k * 4) * pr.aoff_mul;
#pragma unroll 8
            for (int i = 0; i < 32; i++) {
                const int row = warp + 4 * i;
                cp4(a_s + row_byte(row, word_byte), src + s_abase[row]);
            }
            const uint4 *wsrc = (const uint4 *)(pr.wb + ((size_t)ct * pr.NST + ld) * 64 * FB_STAGE_WORDS);
#pragma unroll
            for (int i = 0; i < 4; i++) {   // 64 rows x 8 chunks = 512 chunks of 16 bytes
                const int c = t + 128 * i, row = c >> 3, chunk = c & 7;
                cp16(b_s + row_byte(row, chunk * 16), wsrc + c);
            }
            ld++;
        }
        cp_commit();
    };
#pragma unroll
    for (int s = 0; s < FB_NSTAGE - 1; s++) issue();

    int acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[i][j][q] = 0;

    for (int s = st0; s < st1; s++) {
        cp_wait<FB_NSTAGE - 2>();
        __syncthreads();
        issue();
        const unsigned char *a_s = smem + (size_t)((s - st0) % FB_NSTAGE) * FB_STAGE_BYTES, *b_s = a_s + FB_A_BYTES;
        // A: rows warp * 32 + mt * 16 + g (+ 8); eight words = two 16-byte loads at byte tq * 32
        uint4 a[2][2][2];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int row = warp * 32 + mt * 16 + g + 8 * h;
                a[mt][h][0] = *(const uint4 *)(a_s + row_byte(row, tq * 32));
                a[mt][h][1] = *(const uint4 *)(a_s + row_byte(row, tq * 32 + 16));
            }
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const int row = nt * 8 + g;
            const uint4 b0 = *(const uint4 *)(b_s + row_byte(row, tq * 32));
            const uint4 b1 = *(const uint4 *)(b_s + row_byte(row, tq * 32 + 16));
            const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const uint32_t lo[8] = {a[mt][0][0].x, a[mt][0][0].y, a[mt][0][0].z, a[mt][0][0].w,
                                        a[mt][0][1].x, a[mt][0][1].y, a[mt][0][1].z, a[mt][0][1].w};
                const uint32_t hi[8] = {a[mt][1][0].x, a[mt][1][0].y, a[mt][1][0].z, a[mt][1][0].w,
                                        a[mt][1][1].x, a[mt][1][1].y, a[mt][1][1].z, a[mt][1][1].w};
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    mma_b1(acc[mt][nt], lo[2 * ks], hi[2 * ks], lo[2 * ks + 1], hi[2 * ks + 1], bw[2 * ks], bw[2 * ks + 1]);
            }
        }
    }
    cp_wait<0>();

    // columns: n-tiles 0..3 hold the positive streams of channels ct * 32 + nt * 8 + tq * 2 (+1), n-tiles 4..7
    // the negative streams of the same channels
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = m0 + warp * 32 + mt * 16 + g + 8 * h;
            if (m >= pr.M) continue;
            const int b = m / pr.HoWo, rem = m % pr.HoWo;
#pragma unroll
            for (int nt = 0; nt < 4; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int o = ct * 32 + nt * 8 + tq * 2 + e;
                    if (o >= pr.O) continue;
                    const int v = acc[mt][nt][h * 2 + e] - acc[mt][nt + 4][h * 2 + e];
                    int32_t *dst = pr.out + ((size_t)b * pr.O + o) * pr.HoWo + rem;
                    if (pr.splits > 1) atomicAdd(dst, v);
                    else *dst = v;
                }
        }
}

// Packs the dense prepared streams ws[P][G = K][4][Opad][2] (one real member per group) into the stage /
// fragment order the kernel copies with 16-byte chunks: wb[ct][stage][column][32 words], column = polarity * 32 +
// channel inside the tile, zero beyond the last word or channel.
__global__ void __launch_bounds__(256) fullbin_pack_kernel(const uint32_t *__restrict__ ws, int P, int K, int Opad, int NST,
                                                           int CT, uint32_t *__restrict__ wb) {
    const long long total = (long long)CT * NST * 64 * FB_STAGE_WORDS;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const int pos = (int)(i % FB_STAGE_WORDS);
        const int col = (int)((i / FB_STAGE_WORDS) % 64);
        const int st = (int)((i / (FB_STAGE_WORDS * 64)) % NST);
        const int ct = (int)(i / ((long long)FB_STAGE_WORDS * 64 * NST));
        // inverse of frag_pos: pos = t * 8 + ks * 2 + h  ->  j = ks * 8 + h * 4 + t
        const int tq = pos >> 3, ks = (pos >> 1) & 3, h = pos & 1;
        const int j = ks * 8 + h * 4 + tq;
        const long long kw = (long long)st * FB_STAGE_WORDS + j;
        const int k = (int)(kw / P), p = (int)(kw % P);
        const int pol = col >> 5, o = ct * 32 + (col & 31);
        uint32_t v = 0;
        if (k < K && o < Opad) v = ws[((((size_t)p * K + k) * 4 + 0) * Opad + o) * 2 + pol];
        wb[i] = v;
    }
}

}  // namespace

FullBinPlan fullbin_plan(const Geometry &g) {
    FullBinPlan fp = {};
    fp.layout = g.mode == GEO_SC_MODE_FULL_BIN && g.K == 1 && g.Kp == 4 && (long long)g.G * g.P < (1LL << 30);
    if (!fp.layout) return fp;
    fp.KW = g.G * g.P;   // full_bin: every filter element is a group of one member
    fp.NST = (fp.KW + FB_STAGE_WORDS - 1) / FB_STAGE_WORDS;
    fp.CT = (g.O + 31) / 32;
    fp.bytes = align_up((size_t)fp.CT * fp.NST * 64 * FB_STAGE_WORDS * 4, 256);
    return fp;
}

int launch_fullbin_pack(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s) {
    const FullBinPlan fp = fullbin_plan(g);
    const long long total = (long long)fp.CT * fp.NST * 64 * FB_STAGE_WORDS;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    fullbin_pack_kernel<<<(unsigned)blocks, 256, 0, s>>>(wstream, g.P, g.G, g.Opad, fp.NST, fp.CT, (uint32_t *)section);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

int launch_accumulate_fullbin(const Geometry &g, const uint32_t *astream, const int32_t *aoff, const void *section,
                              int32_t *out, cudaStream_t s) {
    const FullBinPlan fp = fullbin_plan(g);
    FullBinParams pr;
    pr.as = astream; pr.aoff = aoff; pr.wb = (const uint32_t *)section; pr.out = out;
    pr.M = (int)g.M; pr.O = g.O; pr.HoWo = g.Ho * g.Wo; pr.Wo = g.Wo; pr.Wp = g.Wp;
    pr.P = g.P; pr.K = g.G; pr.KW = fp.KW; pr.NST = fp.NST;
    pr.pack_words = act_pack_words(g);
    pr.img_words = act_img_words(g);
    pr.aoff_mul = act_pixel_stride(g);
    static PerDeviceOnce once;
    int rc = per_device_once(once, []() -> int {
        GEO_CUDA_CHECK(cudaFuncSetAttribute(accumulate_fullbin_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            FB_NSTAGE * FB_STAGE_BYTES));
        return GEO_SC_OK;
    });
    if (rc) return rc;
    dim3 grid((unsigned)((g.M + 127) / 128), (unsigned)fp.CT, 1);
    // split the reduction over grid.z while the tiles alone leave SMs idle (three CTAs per SM)
    const long long tiles = (long long)grid.x * grid.y, slots = (long long)sm_count() * 3;
    long long splits = 1;
    while (tiles * splits < slots && splits * 2 <= fp.NST && splits < 64) splits *= 2;
    pr.splits = (int)splits;
    grid.z = (unsigned)splits;
    if (splits > 1) GEO_CUDA_CHECK(cudaMemsetAsync(out, 0, (size_t)g.M * g.O * sizeof(int32_t), s));
    accumulate_fullbin_kernel<<<grid, 128, FB_NSTAGE * FB_STAGE_BYTES, s>>>(pr);
    GEO_CUDA_CHECK(cudaGetLastError());
    return GEO_SC_OK;
}

}  // namespace geo
