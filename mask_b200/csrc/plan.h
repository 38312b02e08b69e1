// Execution plan: fragments of consecutive tiles, grouped per thread block.
#pragma once

#include <cstdint>
#include <vector>

#include "mask_b200.h"

// Fragment f covers tiles [frag_off[f], frag_off[f+1]) of window frag_win[f]; fragments are in
// window order, so tile ranges are contiguous and windows without tiles appear as empty
// fragments (their rows of C must still be written).  frag_slot[f] is -1 when the fragment is
// its whole window (direct store to C) and otherwise the index of its 16xN partial tile in
// scratch.  Thread block g processes fragments [group_off[g], group_off[g+1]).  head_frag lists
// the first fragment of every split window for the fix-up pass.
struct mask_plan {
    int32_t M = 0;
    int32_t W = 0;
    int64_t T = 0;
    int policy = 0;
    int32_t group_tiles = 0;
    int64_t F = 0;  // fragments
    int64_t G = 0;  // groups (thread blocks)
    int64_t P = 0;  // fragments that are part of a split window
    int64_t H = 0;  // split windows
    int32_t max_group_tiles = 0;  // most tiles any thread block gets
    int32_t nslab = 0;  // persistent kernel: 128-column slabs per column block (0 = the widest N fills)
    std::vector<int32_t> h_frag_off, h_frag_win, h_frag_slot, h_group_off, h_head_frag, h_group_tile;
    int32_t* d_frag_off = nullptr;
    int32_t* d_frag_win = nullptr;
    int32_t* d_frag_slot = nullptr;
    int32_t* d_group_off = nullptr;
    int32_t* d_head_frag = nullptr;
    int32_t* d_group_tile = nullptr;  // first tile of every group, then T
    const int32_t* d_row_map = nullptr;  // optional, not owned: output row of packed row i (a row reorder's order[])
    float* const* d_peer_out = nullptr;  // optional, not owned: device array of n_peer_out extra output bases
    int32_t n_peer_out = 0;
    mask_column_features col_features = {};   // set by mask_plan_autotune
    int32_t has_col_features = 0;
    float* d_vals_tf32 = nullptr;        // owned: val_block_val rounded to TF32 (mask_plan_prepare_values), for the TMA kernel
    const float* vals_src = nullptr;     // the array d_vals_tf32 was made from
    int32_t* d_status = nullptr;  // device status word: non-zero after a kernel gave up on a bounded wait
};
