// Sign-sorted accumulation (sc_accumulate_sorted.cu): layout of the sorted weight section that follows
// the dense prepared streams and the member offset table in the prepared-weight buffer.
#pragma once

#include "sc_common.h"

namespace geo {

constexpr int kSortChunkMax = 160;   // members of a chunk: 80 KB of activation words + 23 KB of sorted lists, two CTAs per SM

struct SortedPlan {
    // `layout`: the prepared-weight buffer carries the sorted section.  Decided from the group length and the
    // padded c_out alone, never from the batch, so that weights prepared once serve every batch size.
    // `eligible`: this launch runs on the sorted kernel (layout present and at least one full position tile).
    bool layout, eligible;
    int NCH, KCH, SL, Q;   // chunks per group, members per chunk, slots per (group, chunk, quad), quads
    size_t sw_bytes, srow_bytes, sbeg_bytes;
    size_t total() const { return layout ? sw_bytes + srow_bytes + sbeg_bytes : 0; }
};

SortedPlan sorted_plan(const Geometry &g);
int launch_sort_members(const Geometry &g, const uint32_t *wstream, void *sorted, cudaStream_t s);
int launch_accumulate_sorted(const Geometry &g, const uint32_t *astream, const int32_t *aoff, const void *sorted,
                             int32_t *out, cudaStream_t s);

}  // namespace geo
