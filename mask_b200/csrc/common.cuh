// Shared helpers of the mask_b200 library: status reporting and small device utilities.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "mask_b200.h"

namespace mask {

// Per-thread message for the last failure, returned by mask_last_error().
void set_error(const char* fmt, ...);

inline int fail(int status, const char* what) {
    set_error("%s", what);
    return status;
}

#define MASK_CUDA_TRY(expr)                                                              \
    do {                                                                                 \
        cudaError_t e_ = (expr);                                                         \
        if (e_ != cudaSuccess) {                                                         \
            mask::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_),      \
                            __FILE__, __LINE__);                                         \
            return MASK_ERR_CUDA;                                                        \
        }                                                                                \
    } while (0)

#define MASK_REQUIRE(cond, msg)                                      \
    do {                                                             \
        if (!(cond)) return mask::fail(MASK_ERR_INVALID_ARGUMENT, msg); \
    } while (0)

constexpr int kWinRows = 16;   // rows per window
constexpr int kTileCols = 8;   // condensed columns per tile
constexpr int kTileElems = 128;

// Swizzle<2,2,3> over a row-major 16x8 tile (SR-BCRS value layout).
__host__ __device__ inline int sw223(int i) { return i ^ (((i >> 5) & 3) << 2); }
// Swizzle<1,2,3> over the same tile (ME-TCF COO index).
__host__ __device__ inline int sw123(int i) { return i ^ (((i >> 5) & 1) << 2); }

inline int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
        return 148;
    return n;
}

}  // namespace mask
