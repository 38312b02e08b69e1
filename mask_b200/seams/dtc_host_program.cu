// Drop-in replacement for the reference ME-TCF testbed's host program
// examples/src_fp32/dtc/testbed/host_program.cu: it defines the function the testbed's main.cu
// declares (main.cu:35-50) -- host pointers to the packed ME-TCF arrays and to B in, C (M x N,
// host) out, "mykernel_time: <ms> ms" on stdout -- on top of libmask_b200.so.  TILE_B only selects
// the instantiation main.cu asks for; the library picks its own column tiling.
// Build the testbed with this file in place of host_program.cu and link -lmask_b200.
#include <cstdio>
#include <cstdlib>

#include <cuda_runtime_api.h>

#include "mask_b200.h"

namespace {
void check(int rc, const char* what) {
    if (rc != MASK_OK) {
        fprintf(stderr, "mask_b200 %s: %s\n", what, mask_last_error());
        exit(-1);
    }
}
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(e));
        exit(-1);
    }
}
template <class T>
T* to_device(const T* h, size_t n) {
    T* d = nullptr;
    cuda_check(cudaMalloc(&d, sizeof(T) * (n ? n : 1)), "cudaMalloc");
    if (n) cuda_check(cudaMemcpy(d, h, sizeof(T) * n, cudaMemcpyHostToDevice), "cudaMemcpy");
    return d;
}
}  // namespace

template <int TILE_B>
void dtc_spmm_test_val_sidx_bind_reorder(int M, int N, int K, int TCBlock_num, int nnz, int* val_sidx, int* val_soff,
                                         float* B_val, int* val_coo_idx, float* val_coo_val, int* val_coo_off, float* C,
                                         bool is_ncu_test, int warmup_time, int execute_time) {
    const int W = (M + 15) / 16;
    const size_t T = (size_t)TCBlock_num;
    int* d_soff = to_device(val_soff, (size_t)W + 1);
    int* d_sidx = to_device(val_sidx, 8 * T);
    int* d_off = to_device(val_coo_off, 2 * T + 1);
    int* d_idx = to_device(val_coo_idx, (size_t)nnz);     // nnz = padded length of the COO arrays
    float* d_val = to_device(val_coo_val, (size_t)nnz);
    float* d_B = to_device(B_val, (size_t)K * N);
    float* d_C = nullptr;
    cuda_check(cudaMalloc(&d_C, sizeof(float) * (size_t)M * N), "cudaMalloc");
    mask_plan* plan = nullptr;
    check(mask_plan_create(d_soff, M, (int64_t)T, MASK_POLICY_AUTO, 0, nullptr, &plan), "mask_plan_create");
    const size_t sb = mask_plan_scratch_bytes(plan, N);
    void* d_scratch = nullptr;
    if (sb) cuda_check(cudaMalloc(&d_scratch, sb), "cudaMalloc");
    cudaEvent_t e0, e1;
    cuda_check(cudaEventCreate(&e0), "cudaEventCreate");
    cuda_check(cudaEventCreate(&e1), "cudaEventCreate");
    const int runs = is_ncu_test ? 1 : warmup_time + execute_time;
    for (int i = 0; i < runs; i++) {
        if (i == warmup_time) cuda_check(cudaEventRecord(e0, nullptr), "cudaEventRecord");
        check(mask_spmm_metcf(plan, d_soff, d_sidx, d_off, d_idx, d_val, M, K, N, d_B, N, d_C, N, d_scratch, sb,
                              MASK_EPILOGUE_NONE, nullptr), "mask_spmm_metcf");
    }
    cuda_check(cudaEventRecord(e1, nullptr), "cudaEventRecord");
    cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (!is_ncu_test && execute_time > 0) {
        float ms = 0.f;
        cuda_check(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
        printf("mykernel_time: %f ms\n", ms / execute_time);
    }
    cuda_check(cudaMemcpy(C, d_C, sizeof(float) * (size_t)M * N, cudaMemcpyDeviceToHost), "cudaMemcpy");
    mask_plan_destroy(plan);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(d_scratch); cudaFree(d_C); cudaFree(d_B); cudaFree(d_val); cudaFree(d_idx); cudaFree(d_off); cudaFree(d_sidx);
    cudaFree(d_soff);
}

#define MASK_DTC_INSTANTIATE(TB)                                                                                          \
    template void dtc_spmm_test_val_sidx_bind_reorder<TB>(int, int, int, int, int, int*, int*, float*, int*, float*, int*, \
                                                          float*, bool, int, int);
MASK_DTC_INSTANTIATE(64)
MASK_DTC_INSTANTIATE(32)
MASK_DTC_INSTANTIATE(16)
