// Test / baseline infrastructure, not product code.
//
// Builds the reference project's own SR-BCRS 16x8 GPU kernel (sr_bcrs_spmm_kernel_tf32, generated
// file examples/src_fp32/sr_bcrs/testbed/kernel.inc, launched as in host_program_16x8.cu:60-115)
// for sm_100a by including the reference translation unit unmodified, and exposes one entry that
// runs it on packed arrays with the reference's grid mapping (one 32-thread block per 16-row window
// and 64-column tile) and times it with CUDA events.  Used as a same-box GPU baseline and as a
// cross-check of results; it is the reference's SM80-style code (mma.sync, ldmatrix, cp.async)
// recompiled, not something this repository ships.
#include "sr_bcrs/testbed/host_program_16x8.cu"

extern "C" {

// Host arrays in; C (M x N) out; returns the mean kernel time in ms over `repeat` launches after
// `warmup` launches, or a negative CUDA error code.
float ref_gpu_srbcrs_run(int M, int N, int K, int T, const int* val_sidx, const int* val_soff, const float* B,
                         const float* val_block_val, float* C, int warmup, int repeat) {
    if (N % 64 != 0) return -1000.f;
    const int W = (M + 15) / 16;
    int *d_sidx = nullptr, *d_soff = nullptr;
    float *d_B = nullptr, *d_blk = nullptr, *d_C = nullptr;
    cudaError_t e;
#define REF_TRY(x) if ((e = (x)) != cudaSuccess) { return -(float)e; }
    REF_TRY(cudaMalloc(&d_sidx, sizeof(int) * (size_t)T * 8 + 16));
    REF_TRY(cudaMalloc(&d_soff, sizeof(int) * (size_t)(W + 1)));
    REF_TRY(cudaMalloc(&d_B, sizeof(float) * (size_t)K * N));
    REF_TRY(cudaMalloc(&d_blk, sizeof(float) * (size_t)T * 128 + 16));
    REF_TRY(cudaMalloc(&d_C, sizeof(float) * (size_t)W * 16 * N));   // the kernel stores whole windows
    REF_TRY(cudaMemcpy(d_sidx, val_sidx, sizeof(int) * (size_t)T * 8, cudaMemcpyHostToDevice));
    REF_TRY(cudaMemcpy(d_soff, val_soff, sizeof(int) * (size_t)(W + 1), cudaMemcpyHostToDevice));
    REF_TRY(cudaMemcpy(d_B, B, sizeof(float) * (size_t)K * N, cudaMemcpyHostToDevice));
    REF_TRY(cudaMemcpy(d_blk, val_block_val, sizeof(float) * (size_t)T * 128, cudaMemcpyHostToDevice));
    REF_TRY(cudaMemset(d_C, 0, sizeof(float) * (size_t)W * 16 * N));
    dim3 grid(W, N / 64), block(32);
    constexpr auto blk_mnk = make_shape(Int<16>{}, Int<64>{}, Int<8>{});
    using BLK_MNK = decltype(blk_mnk);
    constexpr auto mma_mnk = make_shape(_16{}, _8{}, _8{});
    using MMA_MNK = decltype(mma_mnk);
    constexpr auto blk_mma_mnk = make_shape(Int<1>{}, Int<8>{}, Int<1>{});
    using BLK_MMA_MNK = decltype(blk_mma_mnk);
    constexpr auto warp_mnk = make_shape(_1{}, _1{}, _1{});
    using WARP_MNK = decltype(warp_mnk);
    cudaEvent_t e0, e1;
    REF_TRY(cudaEventCreate(&e0));
    REF_TRY(cudaEventCreate(&e1));
    for (int i = 0; i < warmup; i++)
        sr_bcrs_spmm_kernel_tf32<BLK_MNK, MMA_MNK, BLK_MMA_MNK, WARP_MNK><<<grid, block>>>(d_B, d_C, d_blk, d_sidx, d_soff, K, M, W, N, T);
    REF_TRY(cudaDeviceSynchronize());
    REF_TRY(cudaEventRecord(e0));
    for (int i = 0; i < repeat; i++)
        sr_bcrs_spmm_kernel_tf32<BLK_MNK, MMA_MNK, BLK_MMA_MNK, WARP_MNK><<<grid, block>>>(d_B, d_C, d_blk, d_sidx, d_soff, K, M, W, N, T);
    REF_TRY(cudaEventRecord(e1));
    REF_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    REF_TRY(cudaEventElapsedTime(&ms, e0, e1));
    REF_TRY(cudaGetLastError());
    REF_TRY(cudaMemcpy(C, d_C, sizeof(float) * (size_t)M * N, cudaMemcpyDeviceToHost));
    cudaFree(d_sidx); cudaFree(d_soff); cudaFree(d_B); cudaFree(d_blk); cudaFree(d_C);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
#undef REF_TRY
    return ms / (repeat > 0 ? repeat : 1);
}

}  // extern "C"
