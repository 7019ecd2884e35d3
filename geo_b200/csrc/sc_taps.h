// Sign-sorted accumulation on tap tiles (sc_accumulate_taps.cu): plan and layout of the section of the
// prepared-weight buffer that this kernel reads, and the geometry helpers its host and device sides share.
#pragma once

#include "sc_common.h"

namespace geo {

constexpr int kTapsThreads = 512;       // 16 warps: NQ channel quads x NH position halves
constexpr int kTapsMaxCtas = 160;       // persistent CTAs at most (one per SM); their first items travel as kernel arguments
constexpr size_t kTapsSmemBudget = 232448 - 1024;

// A "tap" is one filter element (ky, kx).  A group's members are walked tap by tap, the channels of a tap in chunks
// of at most UCH: chunk ch of a group = (tap ch / NCS, channels [ch % NCS * UCH, ...)).  An output pixel near the
// border sees only some taps inside the image; the others meet the all-zero streams of the padding and add nothing,
// so a tile whose positions all lie on the same border class skips their chunks.
struct TapsPlan {
    bool layout;      // the prepared-weight buffer carries this section, and the stream image is batch-innermost:
                      // decided by the layer's geometry, never the batch
    bool eligible;    // this launch runs on the tap-tile kernel (layout present, enough runs for one tile)
    int NQ, NH;       // channel quads and position halves (of 256 positions) per CTA
    int TG;           // taps per group: K2 (1d_bin), K2*K3 (full_or), 1 (2d_bin)
    int UCH, NCS;     // channels per chunk, chunks per tap
    int NCH;          // chunks per group: TG * NCS
    int SL;           // list slots per (group, chunk, quad): UCH rounded up to a multiple of 4
    int Q;            // quads in all
    size_t sw_bytes, soff_bytes, sbeg_bytes, moff_bytes, pix_bytes;   // sections, each 256-byte aligned
    size_t stage_bytes;
    size_t total() const { return layout ? sw_bytes + soff_bytes + sbeg_bytes + moff_bytes + pix_bytes : 0; }
};

TapsPlan taps_plan(const Geometry &g);
int launch_sort_taps(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s);
int launch_accumulate_taps(const Geometry &g, const uint32_t *astream, const void *section, int32_t *out, cudaStream_t s);

// ---- geometry shared by host and device ------------------------------------------------------------------
// Border class of an output coordinate: the range [lo, hi) of filter offsets whose input coordinate lies inside
// the unpadded image, as one number.
__host__ __device__ inline int taps_border_class(int o, int pad, int k, int n) {
    const int lo = pad - o > 0 ? pad - o : 0;
    const int hi = n + pad - o < k ? n + pad - o : k;
    return lo * (k + 1) + (hi > lo ? hi : lo);
}
// Bit (ky * K3 + kx) set: tap (ky, kx) of output pixel (oy, ox) reads inside the image.
__host__ __device__ inline unsigned long long taps_live_mask(int oy, int ox, int K2, int K3, int pad_h, int pad_w, int H,
                                                             int W) {
    unsigned long long m = 0;
    for (int ky = 0; ky < K2; ky++) {
        const int y = oy + ky - pad_h;
        if (y < 0 || y >= H) continue;
        for (int kx = 0; kx < K3; kx++) {
            const int x = ox + kx - pad_w;
            if (x >= 0 && x < W) m |= 1ull << (ky * K3 + kx);
        }
    }
    return m;
}
// Tap (ky * K3 + kx) of chunk-tap index `tap` of group g.
__host__ __device__ inline int taps_tap_of(int mode, int g, int tap, int K3) {
    switch (mode) {
    case GEO_SC_MODE_1D: return tap * K3 + g;   // group = filter column, taps = filter rows
    case GEO_SC_MODE_2D: return g;              // group = tap
    default: return tap;                        // full_or: one group, every tap
    }
}

}  // namespace geo
