// Test infrastructure, not product code.
//
// Exposes the reference project's strict load-balance task planner
// (strict_load_balance, examples/src_fp32/sr_bcrs/testbed/main_strict_lb_16x8.cu:208-256)
// by including that translation unit unmodified from a checkout of the reference project.
#define main ref_main_unused_slb
#include "sr_bcrs/testbed/main_strict_lb_16x8.cu"
#undef main

#include <cstring>

template <int T_M, int T_N, int T_K>
void sr_bcrs_test_tf32_strict_lb(int, int, int, int, int*, int*, DTYPEAB*, DTYPEAB*,
                                 const vector<int>&, const vector<int>&, const vector<int>&, float*,
                                 bool, int, int) {}

namespace {
vector<int> g_rbo, g_rb2w, g_tbo;
}

extern "C" {

// Plans fragments for `val_soff` (W+1 entries) with `workload` tiles per group; returns the
// number of fragments and writes the number of groups.
int ref_strict_lb_plan(int M, int T, int* val_soff, int workload, int* n_groups) {
    strict_load_balance(M, T, val_soff, workload, g_rbo, g_rb2w, g_tbo);
    *n_groups = (int)g_tbo.size() - 1;
    return (int)g_rb2w.size();
}

// row_block_offset: fragments+1, row_block_to_row_window_id: fragments, slb_tb_offset: groups+1
void ref_strict_lb_fetch(int* row_block_offset, int* row_block_to_row_window_id, int* slb_tb_offset) {
    std::memcpy(row_block_offset, g_rbo.data(), sizeof(int) * g_rbo.size());
    std::memcpy(row_block_to_row_window_id, g_rb2w.data(), sizeof(int) * g_rb2w.size());
    std::memcpy(slb_tb_offset, g_tbo.data(), sizeof(int) * g_tbo.size());
}

}  // extern "C"
