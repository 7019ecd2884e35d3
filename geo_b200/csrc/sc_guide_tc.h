// tcgen05 / TMEM / TMA kernels of the float guide for wide layers (sc_guide_tc.cu).
#pragma once

#include "sc_common.h"
#include "sc_guide_mma.h"

namespace geo {

struct TcTile {
    int bw, bh, nb;   // pixel tile of a CTA: nb images x bh rows x bw columns = 128 pixels
};

// Whether the activation-gradient GEMM of this layer runs on tcgen05 (wide layers: at least 128 input channels
// padded to a multiple of 128, column count a multiple of 64, image width a power of two).
bool tc_dgrad_plan(const MmaDims &d, int Cn, TcTile *tile);
int launch_tc_dgrad(const MmaDims &d, int Cn, const void *Dh, const void *wd, float *grad_act, const int *flag,
                    cudaStream_t s);
// Whether the forward product (and D = gout * exp(-y)) of this layer runs on tcgen05: input channels a multiple of
// 64, column count a multiple of 128, output width a power of two.
bool tc_forward_plan(const MmaDims &d, TcTile *tile);
int launch_tc_forward(const MmaDims &d, const void *apad, const void *wb, const float *gout, void *Dh, const int *flag,
                      cudaStream_t s);
// Whether the weight-gradient GEMM runs on tcgen05: input channels a multiple of 128, column count a multiple of
// 128, output width a power of two up to 64, slices of whole 64-position blocks.
bool tc_wgrad_plan(const MmaDims &d, int slice_len, TcTile *tile);
int launch_tc_wgrad(const MmaDims &d, const void *apad, const void *Dh, float *partial, int S, int slice_len, const int *flag,
                    cudaStream_t s);
// Bounded mbarrier waits that ran out since the library was loaded (0 in a healthy run).
int tc_error_count(int *count);

}  // namespace geo
