// Buffers that other processes on the same machine can map: the plumbing under
// mask_plan_set_peer_outputs when each GPU is driven by its own process.  One cudaMalloc per
// buffer (so that the exported handle refers to offset 0 of the allocation), CUDA IPC handles for
// the exchange; the handles travel through whatever channel the host program has.
#include <cstring>

#include "common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == MASK_PEER_HANDLE_BYTES, "handle size");

extern "C" int mask_peer_alloc(size_t bytes, void** d_ptr, void* handle) {
    MASK_REQUIRE(d_ptr != nullptr && handle != nullptr && bytes > 0, "bad arguments");
    void* p = nullptr;
    MASK_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        mask::set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        return MASK_ERR_CUDA;
    }
    std::memcpy(handle, &h, sizeof h);
    *d_ptr = p;
    return MASK_OK;
}

extern "C" int mask_peer_open(const void* handle, void** d_ptr) {
    MASK_REQUIRE(d_ptr != nullptr && handle != nullptr, "bad arguments");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof h);
    // The flag turns on peer access between the current device and the exporter's device.
    MASK_CUDA_TRY(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return MASK_OK;
}

extern "C" int mask_peer_close(void* d_ptr) {
    if (d_ptr == nullptr) return MASK_OK;
    MASK_CUDA_TRY(cudaIpcCloseMemHandle(d_ptr));
    return MASK_OK;
}

extern "C" int mask_peer_free(void* d_ptr) {
    if (d_ptr == nullptr) return MASK_OK;
    MASK_CUDA_TRY(cudaFree(d_ptr));
    return MASK_OK;
}
