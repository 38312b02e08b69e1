// Test infrastructure, not product code.
//
// Exposes the reference project's ME-TCF host packer (buildMETCFMetadata,
// examples/src_fp32/dtc/testbed/main.cu:352-520) by including that translation unit
// unmodified from a checkout of the reference project.  The GPU launch template the unit
// declares is given an empty body: nothing in this library touches a GPU.
#define main ref_main_unused_metcf
#include "dtc/testbed/main.cu"
#undef main

#include <cstring>

template <int TILE_B>
void dtc_spmm_test_val_sidx_bind_reorder(int, int, int, int, int, int*, int*, float*, int*, float*,
                                         int*, float*, bool, int, int) {}
template void dtc_spmm_test_val_sidx_bind_reorder<64>(int, int, int, int, int, int*, int*, float*,
                                                      int*, float*, int*, float*, bool, int, int);
template void dtc_spmm_test_val_sidx_bind_reorder<32>(int, int, int, int, int, int*, int*, float*,
                                                      int*, float*, int*, float*, bool, int, int);
template void dtc_spmm_test_val_sidx_bind_reorder<16>(int, int, int, int, int, int*, int*, float*,
                                                      int*, float*, int*, float*, bool, int, int);

namespace {
METCFMetadata g_meta;
}

extern "C" {

// Runs the reference packer; returns T and writes nnz_pad.
int ref_metcf_pack(int M, int K, const int* rowptr, const int* colind, const float* values,
                   int* nnz_pad) {
    g_meta = buildMETCFMetadata(M, K, rowptr, colind, values);
    *nnz_pad = g_meta.nnz_pad;
    return g_meta.total_TCBlock_num;
}

// val_soff: W+1, val_sidx: 8T, val_coo_off: 2T+1, val_coo_idx / val_coo_val: nnz_pad
void ref_metcf_fetch(int* val_soff, int* val_sidx, int* val_coo_off, int* val_coo_idx,
                     float* val_coo_val) {
    std::memcpy(val_soff, g_meta.val_soff.data(), sizeof(int) * g_meta.val_soff.size());
    std::memcpy(val_sidx, g_meta.val_sidx.data(), sizeof(int) * g_meta.val_sidx.size());
    std::memcpy(val_coo_off, g_meta.val_coo_off.data(), sizeof(int) * g_meta.val_coo_off.size());
    std::memcpy(val_coo_idx, g_meta.val_coo_idx.data(), sizeof(int) * g_meta.val_coo_idx.size());
    std::memcpy(val_coo_val, g_meta.val_coo_val.data(), sizeof(float) * g_meta.val_coo_val.size());
}

// Writes the checkpoint of the last ref_metcf_pack result with the reference's own storeCheckpoint
// (main.cu:232-285) into the directory named by SPARSENE_MTX_CACHE_DIR; returns its 0/1.
int ref_metcf_store_checkpoint(const char* matrix_file_path, int M, int K) {
    return storeCheckpoint(std::string(matrix_file_path), M, K, 0.0f, g_meta.val_sidx, g_meta.val_soff, g_meta.val_coo_idx,
                           g_meta.val_coo_val, g_meta.val_coo_off, g_meta.total_TCBlock_num, g_meta.nnz_pad);
}

// Loads a checkpoint with the reference's own loadCheckpoint (main.cu:287-340) into the capture slot.
int ref_metcf_load_checkpoint(const char* matrix_file_path, int M, int K, int* T, int* nnz_pad) {
    g_meta = METCFMetadata();
    const int ok = loadCheckpoint(std::string(matrix_file_path), M, K, 0.0f, g_meta.val_sidx, g_meta.val_soff, g_meta.val_coo_idx,
                                  g_meta.val_coo_val, g_meta.val_coo_off, g_meta.total_TCBlock_num, g_meta.nnz_pad);
    *T = g_meta.total_TCBlock_num;
    *nnz_pad = g_meta.nnz_pad;
    return ok;
}

// The file name the reference derives from a matrix path and sparsity (main.cu:205-230).
int ref_metcf_checkpoint_stem(const char* matrix_file_path, int M, int K, float sparsity, char* out, int out_len) {
    const std::string stem = buildCheckpointStem(std::string(matrix_file_path), M, K, sparsity);
    if ((int)stem.size() + 1 > out_len) return 0;
    std::memcpy(out, stem.c_str(), stem.size() + 1);
    return 1;
}

}  // extern "C"
