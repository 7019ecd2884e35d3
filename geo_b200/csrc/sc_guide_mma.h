// Internal interface of the tensor-core guide path (sc_guide_mma.cu).
#pragma once

#include "sc_common.h"

namespace geo {

struct MmaDims {
    int B, C, H, W, ph, pw, Hp, Wp, O, K2, K3, Ho, Wo, HoWo;
    int mode, G, Opad, N2, M;
    int Cp;     // channels rounded up to 8
    int taps;   // filter taps per group
    int Kp;     // members per group, taps * Cp rounded up to the stage size
    int linear; // guide without the exp(-y) factor: the forward product is skipped and D = gout
};

bool mma_eligible(const Geometry &g);
MmaDims mma_dims(const Geometry &g);
size_t mma_scratch_bytes(const Geometry &g);
int launch_mma_backward(const Geometry &g, const float *act, const float *weight, const float *gout, float *grad_act,
                        float *grad_weight, void *scratch, int **flag_out, cudaStream_t s);

}  // namespace geo
