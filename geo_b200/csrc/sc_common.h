// Internal declarations shared by the translation units of libgeo_sc.so.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <mutex>

#include "../../include/geo_sc.h"

namespace geo {

// Records a thread-local error detail and returns `status`.
int fail(int status, const char *fmt, ...);

// Everything the kernels need to know about one convolution, derived once on the host.
struct Geometry {
    int B, C, H, W;          // activation dims, unpadded
    int pad_h, pad_w;
    int Hp, Wp;              // padded image
    int O, K2, K3;           // filter dims (K2 = dim 2, K3 = dim 3)
    int Ho, Wo;
    int L, P;                // stream length, 32-bit packs per stream
    int nbits;               // LFSR width
    int mode;
    int z;                   // OR-group width in channels (yz mode)
    int G, K;                // binary-accumulated groups, OR-accumulated members per group
    int Kp;                  // members per group as laid out: K rounded up to 4 (K <= 16) or 16, zero streams
    int NT;                  // c_out tile of the accumulate kernel
    int Opad;                // c_out rounded up to NT
    int tw, lu, lw_w, lw_a;  // progressive loading
    int guide_linear;        // guide without the exp(-y) factor (full_bin: the guide is the plain convolution)
    int batch_fast;          // the stream image has the batch innermost (see act_img_words)
    int Bp;                  // batch rounded up to a multiple of 4: the batch extent of a batch-innermost image
    int generator;           // GEO_SC_GEN_*
    uint32_t seed;           // GEO_SC_GEN_ACC
    long long M;             // output positions B*Ho*Wo
    size_t act_stream_words; // B*P*C*Hp*Wp
    size_t w_stream_words;   // P*G*K*Opad*2
    size_t aoff_entries;     // G*K
};

int make_geometry(const geo_sc_conv_desc *d, Geometry *g);

// Layout of the activation-stream image.  In general [batch][pack][c][Hp][Wp]: a member (c, ky, kx) of a group is a
// fixed word offset from an output position's origin, and consecutive positions of an output row are consecutive
// words.  The batch-innermost form [pack][c][Hp][Wp][Bp] (Bp = batch rounded up to 4, images past the batch all
// zero) makes the same pixel of consecutive images consecutive words: linear layers (1x1 padded images), whose
// positions are the images, and the layers of sc_accumulate_taps.cu, whose tiles hold one pixel of many images.
// Both are one formula: word(b, p, c, y, x) = b * img + p * pack + ((c * Hp + y) * Wp + x) * pixel_stride.
inline int act_img_words(const Geometry &g) { return g.batch_fast ? 1 : g.P * g.C * g.Hp * g.Wp; }
inline int act_pack_words(const Geometry &g) { return g.C * g.Hp * g.Wp * (g.batch_fast ? g.Bp : 1); }
inline int act_pixel_stride(const Geometry &g) { return g.batch_fast ? g.Bp : 1; }   // also scales the member offset table

// Progressive-loading plan: the distinct right-shifts applied to a value and, per pack,
// the stream bits (MSB-first masks) during which each shift is in force.
constexpr int kMaxLevels = 16;
constexpr int kMaxPacks = 8;
struct LoadPlan {
    int nlev;
    int shift[kMaxLevels];
    uint32_t mask[kMaxPacks][kMaxLevels];
    // per pack, the levels whose mask is not empty (with progressive loading only the first pack
    // sees more than one): the generators loop over these instead of all nlev levels
    unsigned char nact[kMaxPacks];
    unsigned char act[kMaxPacks][kMaxLevels];
};
void make_load_plan(int L, int tw, int lu, int lw, LoadPlan *plan);

// Stream generation (sc_streams.cu)
int ensure_tables();
int launch_prepare_weights(const Geometry &g, const float *w, uint32_t *wstream, int32_t *aoff, cudaStream_t s);
int launch_act_streams(const Geometry &g, const float *act, uint32_t *astream, cudaStream_t s);

// Fused layer epilogue (sc_streams.cu): bit counts of one layer -> batch norm (folded scale / shift) -> 2x2 average
// pool -> hardtanh(0, 1) -> fixed-point rounding -> packed activation streams of the next layer `g`.
struct XSource;
int launch_epilogue_streams(const Geometry &g, const XSource &xs, const float *wq, const float *bq, int prec, float *act_out,
                            uint32_t *astream, cudaStream_t s);

// Accumulation (sc_accumulate.cu)
int launch_accumulate(const Geometry &g, const uint32_t *astream, const uint32_t *wstream, const int32_t *aoff,
                      int32_t *out, cudaStream_t s);

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Streaming multiprocessors of the current device (queried once per device, then cached): the unit
// in which grids and split counts are sized.
int sm_count();

// Runs `f` (a callable returning a geo_sc_status) once per device and caller-owned state, under a
// lock: per-device launch configuration (shared-memory opt-ins) from any number of host threads.
struct PerDeviceOnce {
    std::mutex m;
    bool done[64] = {};
};
template <typename F>
int per_device_once(PerDeviceOnce &st, F f) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(GEO_SC_ERR_CUDA, "cudaGetDevice failed");
    if (dev < 0 || dev >= 64) return f();   // beyond the table: configure every time
    std::lock_guard<std::mutex> lock(st.m);
    if (st.done[dev]) return GEO_SC_OK;
    int rc = f();
    if (rc == GEO_SC_OK) st.done[dev] = true;
    return rc;
}

#define GEO_CUDA_CHECK(expr)                                                                       \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return ::geo::fail(GEO_SC_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));   \
    } while (0)

}  // namespace geo
