// Sign-sorted accumulation on row tiles (sc_accumulate_rows.cu): plan and layout of the section of the
// prepared-weight buffer that this kernel reads.
#pragma once

#include "sc_common.h"

namespace geo {

constexpr int kRowsThreads = 512;        // 16 warps: NQ channel quads x NH position halves
constexpr int kRowsSlotsMax = 1024;      // members of a chunk at most (shared arrays of the sorting kernel)
constexpr int kRowsGatherSlots = 4;      // words of one plane that a thread copies, at most
constexpr size_t kRowsSmemBudget = 232448 - 1024;   // dynamic shared memory of one CTA (227 KB) less a margin

// A "plane" is the part of one activation channel, shifted by one filter column, that a position tile
// can touch: the tile's output rows plus K2 - 1 halo rows per image, all W_out columns.  The members
// (c, ky, kx) of a group that differ only in ky read the same plane at row offsets ky, so a plane is
// loaded once where an im2col tile would hold K2 copies.  A "unit" is the smallest run of consecutive
// members that holds whole planes (1d_bin, yz_bin: the K2 members of a channel = 1 plane; full_or, z_bin:
// K2*K3 members = K3 planes; 2d_bin: 1 member = 1 plane); chunks are whole units.
struct RowsPlan {
    bool layout;     // the prepared-weight buffer carries this section: decided by the layer's geometry, never the batch
    bool eligible;   // this launch runs on the row-tile kernel (layout present, at least one full position tile)
    int NQ, NH;      // channel quads and position halves (of 256 positions) per CTA; NQ * NH = 16 warps
    int U, PU;       // members and planes per unit
    int units;       // units per group
    int UCH, NCH;    // units per chunk, chunks per group
    int SL;          // list slots per (group, chunk, quad): members per chunk rounded up to a multiple of 4
    int NPL;         // planes per chunk
    int CG;          // row-quads (4 consecutive output columns) per output row
    int H;           // halo rows per image in a tile: K2 - 1
    int RT, PL;      // rows of a plane in shared memory at most, words of a plane (RT * W_out)
    int NS;          // gather slots per thread: ceil(PL / 512)
    int Q;           // quads in all: c_out_padded / 4
    size_t sw_bytes, soff_bytes, sbeg_bytes, pgoff_bytes;   // sections, each 256-byte aligned
    size_t stage_bytes;                                     // shared memory of one pipeline stage
    size_t total() const { return layout ? sw_bytes + soff_bytes + sbeg_bytes + pgoff_bytes : 0; }
};

RowsPlan rows_plan(const Geometry &g);
int launch_sort_rows(const Geometry &g, const uint32_t *wstream, void *section, cudaStream_t s);
int launch_accumulate_rows(const Geometry &g, const uint32_t *astream, const void *section, int32_t *out,
                           cudaStream_t s);

}  // namespace geo
