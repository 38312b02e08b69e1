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

// The bridge's own packer (convert_to_mco, custom_format_e2e.cu:478-800) for whatever packing mode
// this shim was compiled with: mode 0 ("column_condensed") yields the MCO bitmap leaf.  Two-call
// protocol: with NULL arrays only the sizes are returned.
extern "C" int ref_bridge_pack(int m, int k, const int* row_ptr, const int* col_idx, const float* vals, int* tiles,
                               long long* n_values, int* row_offsets, int* sparse_columns, int* value_offsets,
                               unsigned long long* masks, float* values) {
    try {
        const sparsene_custom_e2e::PackedMco p =
            sparsene_custom_e2e::convert_to_mco(m, k, row_ptr, col_idx, vals, 32, "row", 64);
        *tiles = p.tiles;
        *n_values = (long long)p.values.size();
        if (row_offsets) std::memcpy(row_offsets, p.row_offsets.data(), sizeof(int) * p.row_offsets.size());
        if (sparse_columns) std::memcpy(sparse_columns, p.sparse_columns.data(), sizeof(int) * p.sparse_columns.size());
        if (value_offsets) std::memcpy(value_offsets, p.value_offsets.data(), sizeof(int) * p.value_offsets.size());
        if (masks && !p.masks.empty()) std::memcpy(masks, p.masks.data(), sizeof(uint64_t) * p.masks.size());
        if (values && !p.values.empty()) std::memcpy(values, p.values.data(), sizeof(float) * p.values.size());
    } catch (const std::exception&) {
        return 2;
    }
    return 0;
}
