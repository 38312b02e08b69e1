// Test infrastructure, not product code.
//
// Builds the reference project's own SR-BCRS 16x8 host packer (convertToSRBCRS,
// examples/src_fp32/sr_bcrs/testbed/main_16x8.cu:196-328) into a shared library by
// including that translation unit, unmodified, from where it lies in a checkout of the
// reference project (include path given on the compiler command line).  The packer hands
// its result to an extern template `sr_bcrs_test_tf32<16,64,8>` (main_16x8.cu:32-44), which
// in the reference launches the GPU kernel; here that template is defined to copy the
// packed arrays out instead, so nothing in this library touches a GPU.
#define main ref_main_unused_srbcrs
#include "sr_bcrs/testbed/main_16x8.cu"
#undef main

#include <cstdint>
#include <cstring>

namespace {
struct Capture {
    int T = 0;
    int W = 0;
    int* soff = nullptr;
    int* sidx = nullptr;
    float* blk = nullptr;
} g_cap;
}  // namespace

template <int T_M, int T_N, int T_K>
void sr_bcrs_test_tf32(int M, int, int, int TCBlock_num, int* val_sidx, int* val_soff, DTYPEAB*,
                       DTYPEAB* val_block_val, float*, bool, int, int) {
    g_cap.T = TCBlock_num;
    g_cap.W = (M + T_M - 1) / T_M;
    g_cap.soff = val_soff;
    g_cap.sidx = val_sidx;
    g_cap.blk = val_block_val;
}

extern "C" {

// Runs the reference packer on a CSR matrix and leaves the result in library-owned buffers.
// Returns T (number of 16x8 tiles).  Not thread-safe (one capture slot).
int ref_srbcrs_pack(int M, int K, int nnz, int* rowptr, int* colind, float* values) {
    g_cap = Capture();
    convertToSRBCRS(M, /*N=*/64, K, nnz, rowptr, colind, values, nullptr, nullptr, false, 0, 0);
    return g_cap.T;
}

// Copies the captured arrays into caller buffers of W+1, 8T and 128T elements, then frees them.
void ref_srbcrs_fetch(int* val_soff, int* val_sidx, float* val_block_val) {
    std::memcpy(val_soff, g_cap.soff, sizeof(int) * (size_t)(g_cap.W + 1));
    if (g_cap.T > 0) {
        std::memcpy(val_sidx, g_cap.sidx, sizeof(int) * (size_t)g_cap.T * 8);
        std::memcpy(val_block_val, g_cap.blk, sizeof(float) * (size_t)g_cap.T * 128);
    }
    free(g_cap.soff);
    free(g_cap.sidx);
    free(g_cap.blk);
    g_cap = Capture();
}

}  // extern "C"
