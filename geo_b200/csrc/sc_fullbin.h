// Binary-GEMM accumulation of GEO_SC_MODE_FULL_BIN (sc_accumulate_fullbin.cu): plan and the section of the
// prepared-weight buffer that its kernel reads.
#pragma once

#include "sc_common.h"

namespace geo {

struct FullBinPlan {
    bool layout;   // the descriptor is full_bin: the prepared-weight buffer carries the packed section
    int KW;        // words of the reduction: members * packs
    int NST;       // stages of 32 words
    int CT;        // tiles of 32 output channels
    size_t bytes;  // size of the section (256-byte aligned)
};

FullBinPlan fullbin_plan(const Geometry &g);
int launch_fullbin_pack(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s);
int launch_accumulate_fullbin(const Geometry &g, const uint32_t *astream, const int32_t *aoff, const void *section,
                              int32_t *out, cudaStream_t s);

}  // namespace geo
