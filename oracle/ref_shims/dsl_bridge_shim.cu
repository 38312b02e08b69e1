// Test infrastructure, not product code.
//
// Exposes the host-side row reorders of the reference project's Format-DSL bridge
// (reverse_cuthill_mckee, first_column_order, jaccard_greedy_order;
// examples/src_fp32/acc/testbed/custom_format_e2e.cu:163-347) by including that translation unit
// unmodified from a checkout of the reference project, configured as the SR-BCRS backend
// (packing mode 2, 16x8) with a stub operator include.
#define main ref_main_unused_bridge
#include "acc/testbed/custom_format_e2e.cu"
#undef main

#include <cstring>

extern "C" {

// kind: 1 = row_rcm, 2 = first_col_sort, 3 = jaccard_greedy.  order[new_row] = original_row.
int ref_reorder_rows(int kind, int m, int k, const int* row_ptr, const int* col_idx, int* order) {
    std::vector<int> o;
    try {
        if (kind == 1) o = sparsene_custom_e2e::reverse_cuthill_mckee(m, k, row_ptr, col_idx);
        else if (kind == 2) o = sparsene_custom_e2e::first_column_order(m, k, row_ptr, col_idx);
        else if (kind == 3) o = sparsene_custom_e2e::jaccard_greedy_order(m, k, row_ptr, col_idx);
        else return 1;
    } catch (const std::exception&) {
        return 2;
    }
    if ((int)o.size() != m) return 3;
    std::memcpy(order, o.data(), sizeof(int) * (size_t)m);
    return 0;
}

}  // extern "C"
