// Sign-sorted accumulation for short OR groups (sc_accumulate_short.cu): plan and layout of the section of the
// prepared-weight buffer that this kernel reads.  It serves the layers whose groups are too short for the
// sign-sorted kernels of sc_accumulate_rows.cu / sc_accumulate_sorted.cu (fewer than 64 members as laid out) or
// whose padded c_out is 16.
#pragma once

#include "sc_common.h"

namespace geo {

constexpr int kShortMetaBytes = 32;   // per (group, chunk, quad): 16 row indices, then the end slot of each pattern

struct ShortPlan {
    bool layout;     // the prepared-weight buffer carries this section: decided by the layer's geometry, never the batch
    bool eligible;   // this launch runs on this kernel (layout present, most of one 256-position tile filled)
    int KC, NCH;     // members per chunk (= stage): 4, 8, 12 or 16; chunks per group
    int Q;           // channel quads: c_out_padded / 4
    // wl[P][G][NCH][Q][KC] uint4: the non-zero stream words of a chunk's members, four channels each, sorted by pattern
    // meta[G][NCH][Q][32] bytes: row (member of the chunk) of each sorted slot, then for patterns 0..15 the slot
    //                            after the pattern's last member
    size_t wl_bytes, meta_bytes;
    size_t total() const { return layout ? wl_bytes + meta_bytes : 0; }
};

ShortPlan short_plan(const Geometry &g);
int launch_sort_short(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s);
int launch_accumulate_short(const Geometry &g, const uint32_t *astream, const int32_t *aoff, const void *section,
                            int32_t *out, cudaStream_t s);

}  // namespace geo
