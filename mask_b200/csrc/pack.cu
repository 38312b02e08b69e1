// Device format builder: CSR -> SR-BCRS 16x8 / ME-TCF, bit-identical to the reference host packers.
//
// The reference condenses the columns of every 16-row window with a per-thread byte mask over
// all K columns plus std::sort, then places every entry with a binary search
// (examples/src_fp32/sr_bcrs/testbed/main_16x8.cu:209-318).  Here the same result is obtained
// with flat, one-thread-per-entry kernels and two device-wide scans, so that hub windows with
// millions of entries cost no more per entry than small ones:
//
//   1. row_of[e]       row of entry e (binary search in rowptr).
//   2. rank            entry e = (row r, column c) gets its index p in the window's merged,
//                      column-sorted multiset: its offset in its own row plus, for every other
//                      row of the window, the number of entries < c (rows after r) or <= c (rows
//                      before r).  Rows are sorted, so each count is a binary search.  The column
//                      is scattered to merged[base + p]; rows that are not strictly ascending or
//                      columns outside [0,K) raise an error flag.
//   3. distinct scan   flag[q] = merged[q] starts a new column value inside its window;
//                      D = inclusive scan(flag).  The condensed position of a slot is
//                      D[q] - D[base]; a window holds D[last] - D[base] + 1 distinct columns.
//   4. tiles per window = ceil(distinct/8), exclusive scan -> val_soff, total T.
//   5. fill            column metadata from the flagged slots, values scattered by condensed
//                      position (Swizzle<2,2,3> for SR-BCRS); ME-TCF orders the entries of a tile
//                      by (row, CSR order) using a 16 x 4-bit per-tile row histogram.
#include <algorithm>

#include "common.cuh"

namespace mask {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 16;
constexpr int kScanChunk = kScanThreads * kScanItems;

struct PackScratch {
    int32_t* row_of;     // nnz
    int32_t* pos;        // nnz: merged index, later condensed position
    int32_t* merged;     // nnz
    int32_t* dscan;      // nnz: inclusive scan of distinct flags
    int64_t* spine;      // per scan chunk
    int32_t* status;     // [0] error flag, [1..2] int64 total
    size_t bytes;
};

static inline size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

static PackScratch carve(void* base, int32_t M, int64_t nnz) {
    (void)M;
    PackScratch s{};
    char* p = static_cast<char*>(base);
    size_t off = 0;
    const size_t n = (size_t)std::max<int64_t>(nnz, 1);
    auto take = [&](size_t bytes) { char* r = p ? p + off : nullptr; off += align_up(bytes); return r; };
    s.row_of = reinterpret_cast<int32_t*>(take(n * 4));
    s.pos = reinterpret_cast<int32_t*>(take(n * 4));
    s.merged = reinterpret_cast<int32_t*>(take(n * 4));
    s.dscan = reinterpret_cast<int32_t*>(take(n * 4));
    const size_t chunks = (std::max<size_t>(n, (size_t)M + 1) + kScanChunk - 1) / kScanChunk + 1;
    s.spine = reinterpret_cast<int64_t*>(take(chunks * 8));
    s.status = reinterpret_cast<int32_t*>(take(64));
    s.bytes = off;
    return s;
}

// ---- device-wide scan (reduce chunks, scan the spine in one block, apply) --------------------
// In: functor giving the int32 value at index i.  Out: functor receiving (i, exclusive, value).
template <typename In>
__global__ void __launch_bounds__(kScanThreads) scan_reduce_kernel(In in, int64_t n, int64_t* spine) {
    __shared__ int64_t warp_sum[kScanThreads / 32];
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    int64_t s = 0;
    for (int i = threadIdx.x; i < kScanChunk; i += kScanThreads) {
        const int64_t idx = base + i;
        if (idx < n) s += in(idx);
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        int64_t t = 0;
        for (int i = 0; i < kScanThreads / 32; i++) t += warp_sum[i];
        spine[blockIdx.x] = t;
    }
}

// One block: exclusive scan of spine[0..nchunks) in place; total -> spine[nchunks] and *total.
__global__ void __launch_bounds__(1024) scan_spine_kernel(int64_t* spine, int64_t nchunks, int64_t* total) {
    __shared__ int64_t warp_tot[32];
    __shared__ int64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int64_t base = 0; base < nchunks; base += 1024) {
        const int64_t idx = base + threadIdx.x;
        const int64_t v = idx < nchunks ? spine[idx] : 0;
        int64_t x = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int64_t y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        if (lane == 31) warp_tot[wid] = x;
        __syncthreads();
        if (wid == 0) {
            int64_t w = warp_tot[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const int64_t y = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += y;
            }
            warp_tot[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int64_t before = carry + (wid > 0 ? warp_tot[wid - 1] : 0);
        if (idx < nchunks) spine[idx] = before + x - v;
        __syncthreads();
        if (threadIdx.x == 0) carry += warp_tot[31];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        spine[nchunks] = carry;
        if (total) *total = carry;
    }
}

template <typename In, typename Out>
__global__ void __launch_bounds__(kScanThreads) scan_apply_kernel(In in, Out out, int64_t n, const int64_t* spine) {
    __shared__ int64_t warp_tot[kScanThreads / 32];
    const int64_t base = (int64_t)blockIdx.x * kScanChunk + (int64_t)threadIdx.x * kScanItems;
    int32_t v[kScanItems];
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        v[i] = (base + i < n) ? in(base + i) : 0;
        s += v[i];
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int64_t x = s;
    for (int o = 1; o < 32; o <<= 1) {
        const int64_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) warp_tot[wid] = x;
    __syncthreads();
    int64_t before = spine[blockIdx.x] + x - s;
    for (int i = 0; i < wid; i++) before += warp_tot[i];
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        if (base + i < n) out(base + i, before, v[i]);
        before += v[i];
    }
}

template <typename In, typename Out>
static int device_scan(In in, Out out, int64_t n, int64_t* spine, int64_t* d_total, cudaStream_t st) {
    const int64_t chunks = (n + kScanChunk - 1) / kScanChunk;
    if (chunks > 0) {
        scan_reduce_kernel<<<(unsigned)chunks, kScanThreads, 0, st>>>(in, n, spine);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    scan_spine_kernel<<<1, 1024, 0, st>>>(spine, chunks, d_total);
    MASK_CUDA_TRY(cudaGetLastError());
    if (chunks > 0) {
        scan_apply_kernel<<<(unsigned)chunks, kScanThreads, 0, st>>>(in, out, n, spine);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    return MASK_OK;
}

// ---- analysis kernels ----------------------------------------------------------------------
__global__ void row_of_kernel(const int32_t* __restrict__ rowptr, int32_t M, int64_t nnz, int32_t* __restrict__ row_of) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    int lo = 0, hi = M;  // last row with rowptr[row] <= e
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((int64_t)__ldg(rowptr + mid) <= e) lo = mid; else hi = mid;
    }
    row_of[e] = lo;
}

__device__ __forceinline__ int count_below(const int32_t* __restrict__ col, int lo, int hi, int key, bool inclusive) {
    // number of entries in col[lo,hi) that are < key (or <= key)
    const int start = lo;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        const int v = __ldg(col + mid);
        if (inclusive ? (v <= key) : (v < key)) lo = mid + 1; else hi = mid;
    }
    return lo - start;
}

__global__ void rank_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ colind, int32_t M, int32_t K,
                            int64_t nnz, const int32_t* __restrict__ row_of, int32_t* __restrict__ pos,
                            int32_t* __restrict__ merged, int32_t* __restrict__ status) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = row_of[e];
    const int c = __ldg(colind + e);
    const int rs = __ldg(rowptr + r);
    if (c < 0 || c >= K) { atomicOr(status, 2); }
    if (e > rs && __ldg(colind + e - 1) >= c) { atomicOr(status, 1); }
    const int r0 = (r / kWinRows) * kWinRows;
    const int r1 = min(r0 + kWinRows, M);
    int p = (int)(e - rs);
    int lo = __ldg(rowptr + r0);
    const int base = lo;
    for (int i = r0; i < r1; i++) {
        const int hi = __ldg(rowptr + i + 1);
        if (i != r) p += count_below(colind, lo, hi, c, i < r);
        lo = hi;
    }
    pos[e] = p;
    merged[base + p] = c;
}

struct FlagIn {
    const int32_t* rowptr;
    const int32_t* row_of;
    const int32_t* merged;
    __device__ int32_t operator()(int64_t q) const {
        const int w0 = (row_of[q] / kWinRows) * kWinRows;
        if (q == (int64_t)__ldg(rowptr + w0)) return 1;
        return merged[q] != merged[q - 1];
    }
};
struct InclusiveOut {
    int32_t* d;
    __device__ void operator()(int64_t i, int64_t before, int32_t v) const { d[i] = (int32_t)(before + v); }
};

// tiles per window from the distinct-column scan
struct WindowTilesIn {
    const int32_t* rowptr;
    const int32_t* dscan;
    int32_t M, W;
    __device__ int32_t operator()(int64_t w) const {
        if (w >= W) return 0;
        const int r0 = (int)w * kWinRows, r1 = min(r0 + kWinRows, M);
        const int b = __ldg(rowptr + r0), e = __ldg(rowptr + r1);
        if (e <= b) return 0;
        const int distinct = dscan[e - 1] - dscan[b] + 1;
        return (distinct + kTileCols - 1) / kTileCols;
    }
};
struct ExclusiveOut {
    int32_t* d;
    __device__ void operator()(int64_t i, int64_t before, int32_t) const { d[i] = (int32_t)before; }
};

__global__ void condensed_pos_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ row_of,
                                     const int32_t* __restrict__ dscan, int64_t nnz, int32_t* __restrict__ pos) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int base = __ldg(rowptr + (row_of[e] / kWinRows) * kWinRows);
    pos[e] = dscan[base + pos[e]] - dscan[base];
}

// ---- fill kernels --------------------------------------------------------------------------
// Column metadata: one thread per merged slot.  PAD_LAST: tail slots of a window's last tile
// repeat its last real column (SR-BCRS); otherwise they stay 0 (ME-TCF).
template <bool PAD_LAST>
__global__ void sidx_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ row_of,
                            const int32_t* __restrict__ merged, const int32_t* __restrict__ dscan,
                            const int32_t* __restrict__ val_soff, int32_t M, int64_t nnz, int32_t* __restrict__ val_sidx) {
    const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= nnz) return;
    const int w = row_of[q] / kWinRows;
    const int r0 = w * kWinRows, r1 = min(r0 + kWinRows, M);
    const int base = __ldg(rowptr + r0), end = __ldg(rowptr + r1);
    const int c = merged[q];
    const bool first = (q == base) || (merged[q - 1] != c);
    const int rank = dscan[q] - dscan[base];
    int32_t* out = val_sidx + (int64_t)__ldg(val_soff + w) * kTileCols;
    if (first) out[rank] = c;
    if (PAD_LAST && q == end - 1) {
        const int slots = (__ldg(val_soff + w + 1) - __ldg(val_soff + w)) * kTileCols;
        for (int j = rank + 1; j < slots; j++) out[j] = c;
    }
}

__global__ void srbcrs_values_kernel(const int32_t* __restrict__ row_of, const int32_t* __restrict__ pos,
                                     const float* __restrict__ values, const int32_t* __restrict__ val_soff, int64_t nnz,
                                     float* __restrict__ val_block_val, int32_t* __restrict__ edge_to_col,
                                     int32_t* __restrict__ edge_to_row) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = row_of[e], p = pos[e];
    const int w = r / kWinRows;
    const int64_t tile = (int64_t)__ldg(val_soff + w) + p / kTileCols;
    val_block_val[tile * kTileElems + sw223((r - w * kWinRows) * kTileCols + p % kTileCols)] = values[e];
    if (edge_to_col) edge_to_col[e] = p;
    if (edge_to_row) edge_to_row[e] = r;
}

__global__ void block_partition_kernel(const int32_t* __restrict__ val_soff, int32_t W, int32_t* __restrict__ bp) {
    const int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w < W) bp[w] = val_soff[w + 1] - val_soff[w];
}

// ME-TCF: per tile, a 64-bit word with one 4-bit counter per window row (a row holds at most 8
// entries of a tile, so the counters cannot carry).
__global__ void metcf_histogram_kernel(const int32_t* __restrict__ row_of, const int32_t* __restrict__ pos,
                                       const int32_t* __restrict__ val_soff, int64_t nnz,
                                       unsigned long long* __restrict__ tile_rows) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = row_of[e];
    const int w = r / kWinRows;
    const int64_t tile = (int64_t)__ldg(val_soff + w) + pos[e] / kTileCols;
    atomicAdd(tile_rows + tile, 1ull << (4 * (r - w * kWinRows)));
}

__device__ __forceinline__ int nibble_sum(unsigned long long x) {
    // sum of sixteen 4-bit fields (each <= 8)
    x = (x & 0x0f0f0f0f0f0f0f0full) + ((x >> 4) & 0x0f0f0f0f0f0f0f0full);
    return (int)((x * 0x0101010101010101ull) >> 56);
}

struct TilePadIn {
    const unsigned long long* tile_rows;
    __device__ int32_t operator()(int64_t t) const { return (nibble_sum(tile_rows[t]) + 7) & ~7; }
};
struct CooOffOut {
    const unsigned long long* tile_rows;
    int32_t* off;
    __device__ void operator()(int64_t t, int64_t before, int32_t) const {
        off[2 * t] = (int32_t)before;
        off[2 * t + 1] = (int32_t)before + nibble_sum(tile_rows[t]);
    }
};

__global__ void metcf_values_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ row_of,
                                    const int32_t* __restrict__ pos, const float* __restrict__ values,
                                    const int32_t* __restrict__ val_soff, const int32_t* __restrict__ coo_off,
                                    const unsigned long long* __restrict__ tile_rows, int64_t nnz,
                                    int32_t* __restrict__ coo_idx, float* __restrict__ coo_val) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = row_of[e], p = pos[e];
    const int w = r / kWinRows, rr = r - w * kWinRows, b = p / kTileCols;
    const int64_t tile = (int64_t)__ldg(val_soff + w) + b;
    // entries of earlier rows in this tile, then earlier entries of this row in this tile
    const unsigned long long below = rr == 0 ? 0ull : (tile_rows[tile] & ((1ull << (4 * rr)) - 1ull));
    int slot = __ldg(coo_off + 2 * tile) + nibble_sum(below);
    const int64_t rs = __ldg(rowptr + r);
    for (int64_t j = e - 1; j >= rs && pos[j] / kTileCols == b; j--) slot++;
    coo_idx[slot] = sw123(rr * kTileCols + p % kTileCols);
    coo_val[slot] = values ? values[e] : 1.0f;
}

// MCO (bitmap leaf): bit Swizzle<1,2,3>(8r+c) of the tile's two 64-bit words marks a stored entry.
__global__ void mco_mask_kernel(const int32_t* __restrict__ row_of, const int32_t* __restrict__ pos,
                                const float* __restrict__ values, const int32_t* __restrict__ val_soff, int64_t nnz,
                                int skip_zero_values, unsigned long long* __restrict__ masks) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    if (skip_zero_values && values && values[e] == 0.0f) return;
    const int r = row_of[e], p = pos[e];
    const int w = r / kWinRows;
    const int64_t tile = (int64_t)__ldg(val_soff + w) + p / kTileCols;
    const int phys = sw123((r - w * kWinRows) * kTileCols + p % kTileCols);
    atomicOr(masks + 2 * tile + (phys >> 6), 1ull << (phys & 63));
}

struct McoCountIn {
    const unsigned long long* masks;
    __device__ int32_t operator()(int64_t t) const { return (__popcll(masks[2 * t]) + __popcll(masks[2 * t + 1]) + 3) & ~3; }
};
struct McoOffOut {
    int32_t* off;
    __device__ void operator()(int64_t t, int64_t before, int32_t) const { off[t] = (int32_t)before; }
};

// Values in ascending bit order: an entry's slot is the number of mask bits below its own.
__global__ void mco_values_kernel(const int32_t* __restrict__ row_of, const int32_t* __restrict__ pos,
                                  const float* __restrict__ values, const int32_t* __restrict__ val_soff,
                                  const int32_t* __restrict__ mco_off, const unsigned long long* __restrict__ masks,
                                  int64_t nnz, int skip_zero_values, float* __restrict__ mco_val) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    if (skip_zero_values && values && values[e] == 0.0f) return;
    const int r = row_of[e], p = pos[e];
    const int w = r / kWinRows;
    const int64_t tile = (int64_t)__ldg(val_soff + w) + p / kTileCols;
    const int phys = sw123((r - w * kWinRows) * kTileCols + p % kTileCols);
    const unsigned long long m0 = masks[2 * tile], m1 = masks[2 * tile + 1];
    const int below = phys < 64 ? __popcll(m0 & ((1ull << phys) - 1ull)) : __popcll(m0) + __popcll(m1 & ((1ull << (phys - 64)) - 1ull));
    mco_val[__ldg(mco_off + tile) + below] = values ? values[e] : 1.0f;
}

static inline unsigned blocks_for(int64_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace mask

extern "C" size_t mask_pack_scratch_bytes(int32_t M, int64_t nnz) {
    if (M < 1 || nnz < 0) return 0;
    return mask::carve(nullptr, M, nnz).bytes;
}

extern "C" int mask_pack_analyze(const int32_t* d_rowptr, const int32_t* d_colind, int32_t M, int32_t K, int64_t nnz,
                                 void* d_scratch, size_t scratch_bytes, int32_t* d_val_soff, int64_t* h_T, void* stream) {
    using namespace mask;
    MASK_REQUIRE(d_rowptr && d_val_soff && h_T, "rowptr, val_soff or h_T is NULL");
    MASK_REQUIRE(M >= 1 && K >= 1 && nnz >= 0, "M and K must be positive, nnz non-negative");
    MASK_REQUIRE(nnz == 0 || d_colind, "colind is NULL");
    if (nnz >= ((int64_t)1 << 31) - kScanChunk) return fail(MASK_ERR_INDEX_OVERFLOW, "nnz does not fit int32");
    MASK_REQUIRE(d_scratch != nullptr, "scratch is NULL");
    MASK_REQUIRE((reinterpret_cast<uintptr_t>(d_scratch) & 255) == 0, "scratch must be 256-byte aligned");
    PackScratch s = carve(d_scratch, M, nnz);
    if (scratch_bytes < s.bytes) return fail(MASK_ERR_SCRATCH_TOO_SMALL, "scratch smaller than mask_pack_scratch_bytes");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int W = (M + kWinRows - 1) / kWinRows;
    MASK_CUDA_TRY(cudaMemsetAsync(s.status, 0, 64, st));
    if (nnz > 0) {
        row_of_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, M, nnz, s.row_of);
        MASK_CUDA_TRY(cudaGetLastError());
        rank_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, d_colind, M, K, nnz, s.row_of, s.pos, s.merged, s.status);
        MASK_CUDA_TRY(cudaGetLastError());
        int rc = device_scan(FlagIn{d_rowptr, s.row_of, s.merged}, InclusiveOut{s.dscan}, nnz, s.spine, nullptr, st);
        if (rc != MASK_OK) return rc;
    }
    int rc = device_scan(WindowTilesIn{d_rowptr, s.dscan, M, W}, ExclusiveOut{d_val_soff}, (int64_t)W + 1, s.spine,
                         reinterpret_cast<int64_t*>(s.status + 2), st);
    if (rc != MASK_OK) return rc;
    if (nnz > 0) {
        condensed_pos_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, s.row_of, s.dscan, nnz, s.pos);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    int32_t host_status[4] = {0, 0, 0, 0};
    MASK_CUDA_TRY(cudaMemcpyAsync(host_status, s.status, 16, cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    if (host_status[0] & 2) return fail(MASK_ERR_COLUMN_RANGE, "a column id is outside [0, K)");
    if (host_status[0] & 1) return fail(MASK_ERR_UNSORTED_ROWS, "CSR rows must hold strictly ascending column ids");
    int64_t T;
    memcpy(&T, host_status + 2, 8);
    if (T >= (int64_t)1 << 31 || T * kTileElems < 0) return fail(MASK_ERR_INDEX_OVERFLOW, "tile count does not fit int32");
    *h_T = T;
    return MASK_OK;
}

extern "C" int mask_srbcrs_fill(const int32_t* d_rowptr, const int32_t* d_colind, const float* d_values, int32_t M,
                                int64_t nnz, const void* d_scratch, const int32_t* d_val_soff, int64_t T,
                                int32_t* d_val_sidx, float* d_val_block_val, int32_t* d_block_partition,
                                int32_t* d_edge_to_col, int32_t* d_edge_to_row, void* stream) {
    using namespace mask;
    (void)d_colind;
    MASK_REQUIRE(d_rowptr && d_scratch && d_val_soff, "rowptr, scratch or val_soff is NULL");
    MASK_REQUIRE(M >= 1 && nnz >= 0 && T >= 0, "bad sizes");
    MASK_REQUIRE(nnz == 0 || (d_values && T > 0), "values is NULL or T is 0 for a non-empty matrix");
    MASK_REQUIRE(T == 0 || (d_val_sidx && d_val_block_val), "output arrays are NULL");
    PackScratch s = carve(const_cast<void*>(d_scratch), M, nnz);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int W = (M + kWinRows - 1) / kWinRows;
    if (T > 0) MASK_CUDA_TRY(cudaMemsetAsync(d_val_block_val, 0, (size_t)T * kTileElems * sizeof(float), st));
    if (nnz > 0) {
        sidx_kernel<true><<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, s.row_of, s.merged, s.dscan, d_val_soff, M, nnz, d_val_sidx);
        MASK_CUDA_TRY(cudaGetLastError());
        srbcrs_values_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(s.row_of, s.pos, d_values, d_val_soff, nnz,
                                                                   d_val_block_val, d_edge_to_col, d_edge_to_row);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    if (d_block_partition) {
        block_partition_kernel<<<blocks_for(W, 256), 256, 0, st>>>(d_val_soff, W, d_block_partition);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    return MASK_OK;
}

extern "C" int mask_metcf_offsets(const int32_t* d_rowptr, int32_t M, int64_t nnz, const void* d_scratch,
                                  const int32_t* d_val_soff, int64_t T, int32_t* d_val_coo_off, uint64_t* d_tile_rows,
                                  int64_t* h_nnz_pad, void* stream) {
    using namespace mask;
    (void)d_rowptr;
    MASK_REQUIRE(d_scratch && d_val_soff && d_val_coo_off && h_nnz_pad, "NULL argument");
    MASK_REQUIRE(M >= 1 && nnz >= 0 && T >= 0, "bad sizes");
    MASK_REQUIRE(T == 0 || d_tile_rows, "tile_rows is NULL");
    PackScratch s = carve(const_cast<void*>(d_scratch), M, nnz);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* rows = reinterpret_cast<unsigned long long*>(d_tile_rows);
    if (T > 0) MASK_CUDA_TRY(cudaMemsetAsync(rows, 0, (size_t)T * 8, st));
    if (nnz > 0) {
        metcf_histogram_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(s.row_of, s.pos, d_val_soff, nnz, rows);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    // the spine is sized for max(nnz, W+1) items and T <= nnz
    int rc = device_scan(TilePadIn{rows}, CooOffOut{rows, d_val_coo_off}, T, s.spine,
                         reinterpret_cast<int64_t*>(s.status + 2), st);
    if (rc != MASK_OK) return rc;
    int64_t total = 0;
    MASK_CUDA_TRY(cudaMemcpyAsync(&total, s.status + 2, 8, cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    if (total >= (int64_t)1 << 31) return fail(MASK_ERR_INDEX_OVERFLOW, "nnz_pad does not fit int32");
    const int32_t closing = (int32_t)total;
    MASK_CUDA_TRY(cudaMemcpyAsync(d_val_coo_off + 2 * T, &closing, 4, cudaMemcpyHostToDevice, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    *h_nnz_pad = total;
    return MASK_OK;
}

extern "C" int mask_metcf_fill(const int32_t* d_rowptr, const int32_t* d_colind, const float* d_values, int32_t M,
                               int64_t nnz, const void* d_scratch, const int32_t* d_val_soff, int64_t T,
                               const int32_t* d_val_coo_off, const uint64_t* d_tile_rows, int64_t nnz_pad,
                               int32_t* d_val_sidx, int32_t* d_val_coo_idx, float* d_val_coo_val, void* stream) {
    using namespace mask;
    (void)d_colind;
    MASK_REQUIRE(d_rowptr && d_scratch && d_val_soff && d_val_coo_off, "NULL argument");
    MASK_REQUIRE(M >= 1 && nnz >= 0 && T >= 0 && nnz_pad >= 0, "bad sizes");
    MASK_REQUIRE(T == 0 || (d_val_sidx && d_tile_rows), "output arrays are NULL");
    MASK_REQUIRE(nnz_pad == 0 || (d_val_coo_idx && d_val_coo_val), "output arrays are NULL");
    PackScratch s = carve(const_cast<void*>(d_scratch), M, nnz);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (T > 0) MASK_CUDA_TRY(cudaMemsetAsync(d_val_sidx, 0, (size_t)T * kTileCols * 4, st));
    if (nnz_pad > 0) {
        MASK_CUDA_TRY(cudaMemsetAsync(d_val_coo_idx, 0, (size_t)nnz_pad * 4, st));
        MASK_CUDA_TRY(cudaMemsetAsync(d_val_coo_val, 0, (size_t)nnz_pad * 4, st));
    }
    if (nnz > 0) {
        sidx_kernel<false><<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, s.row_of, s.merged, s.dscan, d_val_soff, M, nnz, d_val_sidx);
        MASK_CUDA_TRY(cudaGetLastError());
        metcf_values_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, s.row_of, s.pos, d_values, d_val_soff, d_val_coo_off,
                                                                  reinterpret_cast<const unsigned long long*>(d_tile_rows),
                                                                  nnz, d_val_coo_idx, d_val_coo_val);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    return MASK_OK;
}

extern "C" int mask_mco_offsets(const float* d_values, int32_t M, int64_t nnz, const void* d_scratch, const int32_t* d_val_soff,
                                int64_t T, int skip_zero_values, uint64_t* d_val_mco_mask, int32_t* d_val_mco_off,
                                int64_t* h_nval, void* stream) {
    using namespace mask;
    MASK_REQUIRE(d_scratch && d_val_soff && d_val_mco_off && h_nval, "NULL argument");
    MASK_REQUIRE(M >= 1 && nnz >= 0 && T >= 0, "bad sizes");
    MASK_REQUIRE(T == 0 || d_val_mco_mask, "val_mco_mask is NULL");
    PackScratch s = carve(const_cast<void*>(d_scratch), M, nnz);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto* masks = reinterpret_cast<unsigned long long*>(d_val_mco_mask);
    if (T > 0) MASK_CUDA_TRY(cudaMemsetAsync(masks, 0, (size_t)T * 16, st));
    if (nnz > 0) {
        mco_mask_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(s.row_of, s.pos, d_values, d_val_soff, nnz, skip_zero_values, masks);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    int rc = device_scan(McoCountIn{masks}, McoOffOut{d_val_mco_off}, T, s.spine, reinterpret_cast<int64_t*>(s.status + 2), st);
    if (rc != MASK_OK) return rc;
    int64_t total = 0;
    MASK_CUDA_TRY(cudaMemcpyAsync(&total, s.status + 2, 8, cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    if (total >= (int64_t)1 << 31) return fail(MASK_ERR_INDEX_OVERFLOW, "value count does not fit int32");
    const int32_t closing = (int32_t)total;
    MASK_CUDA_TRY(cudaMemcpyAsync(d_val_mco_off + T, &closing, 4, cudaMemcpyHostToDevice, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    *h_nval = total;
    return MASK_OK;
}

extern "C" int mask_mco_fill(const int32_t* d_rowptr, const float* d_values, int32_t M, int64_t nnz, const void* d_scratch,
                             const int32_t* d_val_soff, int64_t T, int skip_zero_values, const uint64_t* d_val_mco_mask,
                             const int32_t* d_val_mco_off, int64_t nval, int32_t* d_val_sidx, float* d_val_mco_val,
                             void* stream) {
    using namespace mask;
    MASK_REQUIRE(d_rowptr && d_scratch && d_val_soff && d_val_mco_off, "NULL argument");
    MASK_REQUIRE(M >= 1 && nnz >= 0 && T >= 0 && nval >= 0, "bad sizes");
    MASK_REQUIRE(T == 0 || (d_val_sidx && d_val_mco_mask), "output arrays are NULL");
    MASK_REQUIRE(nval == 0 || d_val_mco_val, "val_mco_val is NULL");
    PackScratch s = carve(const_cast<void*>(d_scratch), M, nnz);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (nval > 0) MASK_CUDA_TRY(cudaMemsetAsync(d_val_mco_val, 0, (size_t)nval * 4, st));
    if (nnz > 0) {
        sidx_kernel<true><<<blocks_for(nnz, 256), 256, 0, st>>>(d_rowptr, s.row_of, s.merged, s.dscan, d_val_soff, M, nnz, d_val_sidx);
        MASK_CUDA_TRY(cudaGetLastError());
        mco_values_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(s.row_of, s.pos, d_values, d_val_soff, d_val_mco_off,
                                                                reinterpret_cast<const unsigned long long*>(d_val_mco_mask), nnz,
                                                                skip_zero_values, d_val_mco_val);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    return MASK_OK;
}
