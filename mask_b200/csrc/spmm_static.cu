// SpMM entry point for callers that must not allocate device memory.
//
// Who this is for.  Some hosts hand the whole device heap to an arena of their own when they
// start (inference servers, engines that embed this library as a plug-in) and treat any later
// cudaMalloc -- theirs or a library's -- as an error; others sit in a latency-critical loop where
// the device-wide synchronisation that cudaMalloc/cudaFree imply is not acceptable.  Such a
// caller can still provide B and C, and the packed matrix and plan it prepared at start-up, but it
// has nowhere to get the partial-tile buffer that mask_spmm_srbcrs wants when the plan splits
// windows across thread blocks.  Here that buffer is a fixed array that lives in the library's
// own device image, so the call needs no allocator at all.
#include <mutex>

#include "common.cuh"
#include "plan.h"

namespace {

// Partial 16xN tiles of split windows.  32 MiB: 1024 partial tiles at N = 512.  Every GPU on
// which this library's module gets loaded carries the array until the process exits.
constexpr size_t kStaticScratchBytes = (size_t)32 << 20;
static __device__ __align__(256) float g_partial_tiles[kStaticScratchBytes / sizeof(float)];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void* g_device_ptr[kMaxDevices] = {};  // device address of g_partial_tiles, per device ordinal

// In host code `g_partial_tiles` is only a handle for the runtime, not an address a kernel could
// use; the device address has to be asked for, once per device, with that device current.
int static_scratch_for_current_device(void** out) {
    int dev = -1;
    MASK_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return mask::fail(MASK_ERR_NO_DEVICE, "device ordinal outside the supported range");
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_device_ptr[dev] == nullptr) {
        void* p = nullptr;
        MASK_CUDA_TRY(cudaGetSymbolAddress(&p, g_partial_tiles));
        g_device_ptr[dev] = p;
    }
    *out = g_device_ptr[dev];
    return MASK_OK;
}

}  // namespace

extern "C" size_t mask_static_scratch_capacity(void) { return kStaticScratchBytes; }

extern "C" int mask_spmm_srbcrs_static_scratch(const mask_plan* plan, const int32_t* d_val_soff,
                                               const int32_t* d_val_sidx, const float* d_val_block_val, int32_t M,
                                               int32_t K, int32_t N, const float* d_B, int64_t ldb, float* d_C,
                                               int64_t ldc, int epilogue, void* stream) {
    using namespace mask;
    MASK_REQUIRE(plan != nullptr, "plan is NULL");
    const size_t need = mask_plan_scratch_bytes(plan, N);
    if (need > kStaticScratchBytes) {
        set_error("this plan needs %zu bytes of partial tiles for N=%d but the built-in buffer holds %zu; use a plan "
                  "that splits fewer windows (policy row, or a larger group_tiles) or call mask_spmm_srbcrs with a "
                  "buffer of your own",
                  need, (int)N, kStaticScratchBytes);
        return MASK_ERR_SCRATCH_TOO_SMALL;
    }
    void* scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != MASK_OK) return rc;
    // Same kernels as mask_spmm_srbcrs; only where the partial tiles live differs.  Nothing in the
    // buffer has to start at zero: every partial tile the fix-up pass reads is written in full by
    // the main kernel of the same call.
    return mask_spmm_srbcrs(plan, d_val_soff, d_val_sidx, d_val_block_val, M, K, N, d_B, ldb, d_C, ldc, scratch,
                            kStaticScratchBytes, epilogue, stream);
}
