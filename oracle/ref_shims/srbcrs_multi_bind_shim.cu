// Test infrastructure, not product code.
//
// Exposes the reference project's multi-binding task planner
// (multi_binding_load_balance, examples/src_fp32/sr_bcrs/testbed/main_multi_bind_16x8.cu:207-271)
// by including that translation unit unmodified from a checkout of the reference project.
#define main ref_main_unused_mb
#include "sr_bcrs/testbed/main_multi_bind_16x8.cu"
#undef main

#include <cstring>

template <int T_M, int T_N, int T_K>
void sr_bcrs_test_tf32_multi_bind(int, int, int, int, int*, const vector<int>&, DTYPEAB*,
                                  DTYPEAB*, const vector<int>&, const vector<int>&, float*, bool,
                                  int, int) {}

namespace {
vector<int> g_binding, g_split, g_soff;
}

extern "C" {

// Returns the number of bound tasks.
int ref_multi_bind_plan(int M, int T, int* val_soff) {
    int n_tasks = 0;
    multi_binding_load_balance(M, T, val_soff, n_tasks, g_binding, g_split, g_soff);
    return n_tasks;
}

// row_window_binding: tasks, row_window_split: W, row_window_val_soff: tasks+1
void ref_multi_bind_fetch(int* row_window_binding, int* row_window_split, int* row_window_val_soff) {
    std::memcpy(row_window_binding, g_binding.data(), sizeof(int) * g_binding.size());
    std::memcpy(row_window_split, g_split.data(), sizeof(int) * g_split.size());
    std::memcpy(row_window_val_soff, g_soff.data(), sizeof(int) * g_soff.size());
}

}  // extern "C"
