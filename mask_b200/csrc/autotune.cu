// Column features of a packed matrix, computed on the device, and the plan decisions keyed on them.
//
// The reference leaves these decisions to an LLM strategy agent working from the statistics of its
// featurizer (examples/src_fp32/dtc/testbed/featurize_mtx.cu:298-401: tiles per window, unique
// columns, density, top-5 window share) and a catalogue of knobs (python/sparsene/op_gen/
// strategy_agent.py:414-528: tile width, placement, stages); here they are a fixed rule over
// measured features.  The window statistics (mask_features) come from val_soff, which the planner
// has on the host anyway; what needs the device is the column side, from the 8 T entries of
// val_sidx:
//   * band: how far the gathered rows of B lie from the diagonal position of their window (a stencil
//     or banded matrix keeps them within a few thousand rows, so neighbouring windows share them and
//     they stay in L2 whatever their width);
//   * hub share: what fraction of all gathers goes to the most gathered columns whose rows of B fit
//     half the L2 -- at the full row width and at a half and a quarter of it.  On a power-law graph
//     that fraction is what L2 can serve; where a narrower row raises it markedly, sweeping the matrix
//     once per 256 columns instead of once per 512 saves more DRAM traffic (rows of B) than it costs
//     (tile values and ids read twice).
#include <cub/cub.cuh>

#include <algorithm>

#include "common.cuh"
#include "plan.h"

namespace mask {

namespace {

struct Scratch {
    void* p = nullptr;
    ~Scratch() { if (p) cudaFree(p); }
    int alloc(size_t bytes) {
        MASK_CUDA_TRY(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
        return MASK_OK;
    }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

constexpr int kBandBuckets = 33;   // bucket b: distances in [2^(b-1), 2^b), bucket 0: distance 0

// one thread per tile: window by binary search in val_soff, then its 8 ids
__global__ void column_stats_kernel(const int32_t* __restrict__ soff, const int32_t* __restrict__ sidx, int32_t W, int64_t T,
                                    int32_t M, int32_t K, int64_t local_rows, uint32_t* __restrict__ counts,
                                    unsigned long long* __restrict__ band_hist) {
    __shared__ unsigned int hist[kBandBuckets + 1];   // last entry: gathers within local_rows of the diagonal
    if (threadIdx.x <= kBandBuckets) hist[threadIdx.x] = 0;
    __syncthreads();
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) {
        int lo = 0, hi = W;   // last window whose first tile is <= t
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((int64_t)soff[mid] <= t) lo = mid; else hi = mid;
        }
        const int64_t diag = (int64_t)lo * kWinRows * K / M;
        for (int j = 0; j < kTileCols; j++) {
            const int id = sidx[t * kTileCols + j];
            if (id < 0 || id >= K) continue;
            atomicAdd(&counts[id], 1u);
            const int64_t d = id > diag ? id - diag : diag - id;
            atomicAdd(&hist[d == 0 ? 0 : 64 - __clzll((unsigned long long)d)], 1u);
            if (d <= local_rows) atomicAdd(&hist[kBandBuckets], 1u);
        }
    }
    __syncthreads();
    if (threadIdx.x <= kBandBuckets && hist[threadIdx.x]) atomicAdd(&band_hist[threadIdx.x], (unsigned long long)hist[threadIdx.x]);
}

__global__ void count_nonzero_kernel(const uint32_t* __restrict__ counts, int32_t K, int32_t* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool nz = i < K && counts[i] != 0;
    const unsigned b = __ballot_sync(0xffffffffu, nz);
    if ((threadIdx.x & 31) == 0 && b) atomicAdd(out, __popc(b));
}

struct ToU64 {
    __host__ __device__ unsigned long long operator()(uint32_t v) const { return v; }
};

}  // namespace

}  // namespace mask

extern "C" int mask_features_columns(const int32_t* d_val_soff, const int32_t* d_val_sidx, int32_t M, int32_t K, int64_t T, int32_t N,
                                     mask_column_features* out, void* stream) {
    using namespace mask;
    MASK_REQUIRE(out != nullptr && d_val_soff != nullptr && M >= 1 && K >= 1 && T >= 0 && N >= 1, "bad arguments");
    MASK_REQUIRE(T == 0 || d_val_sidx != nullptr, "val_sidx is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    *out = mask_column_features{};
    int dev = 0, l2 = 0;
    MASK_CUDA_TRY(cudaGetDevice(&dev));
    MASK_CUDA_TRY(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev));
    out->l2_bytes = l2;
    out->gathers = T * kTileCols;
    if (T == 0) return MASK_OK;
    const int32_t W = (M + kWinRows - 1) / kWinRows;
    Scratch counts, sorted, prefix, hist, nz, tmp;
    int rc = counts.alloc((size_t)K * 4);
    if (rc == MASK_OK) rc = sorted.alloc((size_t)K * 4);
    if (rc == MASK_OK) rc = prefix.alloc((size_t)K * 8);
    if (rc == MASK_OK) rc = hist.alloc((kBandBuckets + 1) * 8);
    if (rc == MASK_OK) rc = nz.alloc(16);
    if (rc != MASK_OK) return rc;
    MASK_CUDA_TRY(cudaMemsetAsync(counts.p, 0, (size_t)K * 4, st));
    MASK_CUDA_TRY(cudaMemsetAsync(hist.p, 0, (kBandBuckets + 1) * 8, st));
    MASK_CUDA_TRY(cudaMemsetAsync(nz.p, 0, 16, st));
    // "local": a band of windows keeps rows of B alive that take at most half the L2 at this row width
    const int width0 = std::min(N, 512);
    out->local_rows = (int32_t)std::min<int64_t>(K, std::max<int64_t>(0, ((int64_t)(l2 / 2) / ((int64_t)width0 * 4) - kWinRows) / 2));
    column_stats_kernel<<<(unsigned)((T + 255) / 256), 256, 0, st>>>(d_val_soff, d_val_sidx, W, T, M, K, (int64_t)out->local_rows,
                                                                    counts.as<uint32_t>(), hist.as<unsigned long long>());
    count_nonzero_kernel<<<(unsigned)((K + 255) / 256), 256, 0, st>>>(counts.as<uint32_t>(), K, nz.as<int32_t>());
    MASK_CUDA_TRY(cudaGetLastError());
    // gathers per column, most gathered first, and their running sum
    size_t b1 = 0, b2 = 0;
    cub::TransformInputIterator<unsigned long long, ToU64, const uint32_t*> as64(sorted.as<uint32_t>(), ToU64());
    MASK_CUDA_TRY(cub::DeviceRadixSort::SortKeysDescending(nullptr, b1, counts.as<uint32_t>(), sorted.as<uint32_t>(), K, 0, 32, st));
    MASK_CUDA_TRY(cub::DeviceScan::InclusiveSum(nullptr, b2, as64, prefix.as<unsigned long long>(), K, st));
    rc = tmp.alloc(std::max(b1, b2));
    if (rc != MASK_OK) return rc;
    MASK_CUDA_TRY(cub::DeviceRadixSort::SortKeysDescending(tmp.p, b1, counts.as<uint32_t>(), sorted.as<uint32_t>(), K, 0, 32, st));
    MASK_CUDA_TRY(cub::DeviceScan::InclusiveSum(tmp.p, b2, as64, prefix.as<unsigned long long>(), K, st));
    unsigned long long h[kBandBuckets + 1];
    MASK_CUDA_TRY(cudaMemcpyAsync(h, hist.p, sizeof(h), cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaMemcpyAsync(&out->distinct_columns, nz.p, 4, cudaMemcpyDeviceToHost, st));
    unsigned long long reach[3] = {0, 0, 0};
    for (int i = 0; i < 3; i++) {
        const int width = std::min(N, 512 >> i);                               // columns of one gathered row at 4, 2, 1 slabs
        const int64_t rows = std::max<int64_t>(1, (int64_t)(l2 / 2) / ((int64_t)width * 4));
        out->hub_columns[i] = (int32_t)std::min<int64_t>(rows, K);
        MASK_CUDA_TRY(cudaMemcpyAsync(&reach[i], prefix.as<unsigned long long>() + (out->hub_columns[i] - 1), 8, cudaMemcpyDeviceToHost, st));
    }
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    unsigned long long total = 0;
    for (int b = 0; b < kBandBuckets; b++) total += h[b];
    for (int i = 0; i < 3; i++) out->hub_share[i] = total ? (double)reach[i] / (double)total : 0.0;
    out->local_share = total ? (double)h[kBandBuckets] / (double)total : 1.0;
    auto percentile = [&](double q) -> int32_t {
        unsigned long long run = 0;
        for (int b = 0; b < kBandBuckets; b++) {
            run += h[b];
            if ((double)run >= q * (double)total) return b == 0 ? 0 : (int32_t)std::min<int64_t>((int64_t)1 << b, (int64_t)K);
        }
        return K;
    };
    out->band_p50 = percentile(0.50);
    out->band_p90 = percentile(0.90);
    return MASK_OK;
}

// The plan table.  Keyed on: does the matrix keep its gathers local (band), and if not, how much more
// of them L2 can serve when a gathered row is half as wide (hub shares).  Chooses the number of
// 128-column slabs per column block for wide (N > 256) and medium (128 < N <= 256) products; narrow
// products have one slab.  Thresholds fitted on the five benchmark configurations (27-point stencil
// and uniform-random: 4 slabs; power-law graphs with 2^21 and 2^22 nodes: 2 slabs, 3-5 % faster than
// 4; 2^20 nodes: a tie).
extern "C" int mask_plan_autotune(mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx, int32_t K, void* stream) {
    using namespace mask;
    MASK_REQUIRE(plan != nullptr, "plan is NULL");
    mask_column_features f;
    int rc = mask_features_columns(d_val_soff, d_val_sidx, plan->M, K, plan->T, 512, &f, stream);
    if (rc != MASK_OK) return rc;
    plan->col_features = f;
    plan->has_col_features = 1;
    const double half_l2 = 0.5 * (double)f.l2_bytes;
    const double b_bytes = (double)f.distinct_columns * 4.0 * 512.0;
    const bool local = f.local_share >= 0.9 || b_bytes <= half_l2;   // the gathers stay near the diagonal, or all of B fits
    // hub-heavy (a quarter of the gathers already fit at full width) and markedly more fits at half width
    const bool narrower_rows_pay = !local && b_bytes > 8.0 * half_l2 && f.hub_share[0] >= 0.25 && f.hub_share[1] - f.hub_share[0] >= 0.02;
    plan->nslab = narrower_rows_pay ? 2 : 4;
    return MASK_OK;
}

extern "C" int mask_plan_column_features(const mask_plan* plan, mask_column_features* out, int32_t* nslab_wide) {
    using namespace mask;
    MASK_REQUIRE(plan != nullptr && out != nullptr, "NULL argument");
    if (!plan->has_col_features) return fail(MASK_ERR_INVALID_ARGUMENT, "mask_plan_autotune has not run on this plan");
    *out = plan->col_features;
    if (nslab_wide) *nslab_wide = plan->nslab;
    return MASK_OK;
}
