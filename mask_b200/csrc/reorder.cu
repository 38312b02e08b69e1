// Row reorders of the Format-DSL host bridge, computed on the device, and the device-side CSR row
// permutation.
//
// The bridge (examples/src_fp32/acc/testbed/custom_format_e2e.cu:163-347) defines three orders by
// sequential host algorithms whose tie-breaks are part of the result; here each is restated as the
// data-parallel computation that yields the same permutation:
//   first_col_sort  key(row) = smallest in-range column (K for none); stable radix sort by key.
//   jaccard_greedy  signature(row) = min over its columns of a 64-bit mix; rows ranked by
//                   (signature, first column, id) with two stable radix sorts; the ranking is cut into
//                   buckets of 64 and one thread block per bucket runs the greedy chain (next = the
//                   remaining row most similar to the last one, ties to the smaller id), every
//                   similarity a warp-wide intersection count by binary search.
//   row_rcm         reverse Cuthill-McKee.  The sequential queue order is reproduced level by level:
//                   a node's parent is the EARLIEST queue position among its visited neighbours
//                   (atomicMin), a level is its nodes sorted by (parent position, degree, id), and all
//                   connected components advance together; components are then laid out by the rank of
//                   their start node (the unvisited node of least (degree, id)) and each is reversed.
//                   One round of kernels per breadth-first level: the cost grows with the graph's
//                   diameter (tens of levels for graphs, hundreds for 3-D meshes).
// Applying an order -- gathering the rows of a device CSR matrix -- and undoing it are device work
// too: the SpMM kernels take the order as a row map and write output row order[new_row] directly,
// which replaces the bridge's host-side unpack_output (:1083-1100).
//
// Input contract (the packers'): column ids of a row strictly ascending.
#include <cub/cub.cuh>

#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace mask {

namespace {

// Device scratch that frees itself; sized once per call (these are format-conversion passes).
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
    int alloc(size_t bytes) {
        MASK_CUDA_TRY(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
        return MASK_OK;
    }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

__global__ void iota_kernel(int32_t* a, int32_t n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = i;
}

__device__ __forceinline__ uint64_t mix_column(uint64_t v) {   // the bridge's column hash (splitmix64 finaliser)
    v += 0x9e3779b97f4a7c15ULL;
    v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ULL;
    v = (v ^ (v >> 27)) * 0x94d049bb133111ebULL;
    return v ^ (v >> 31);
}

// one warp per row: first in-range column (K if none) and the min-hash signature over all its columns
__global__ void row_keys_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ colind, int32_t M, int32_t K,
                                uint32_t* __restrict__ first, uint64_t* __restrict__ sig) {
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= M) return;
    uint32_t f = (uint32_t)K;
    uint64_t s = ~0ULL;
    for (int q = rowptr[r] + lane; q < rowptr[r + 1]; q += 32) {
        const int c = colind[q];
        if (c >= 0 && c < K) f = min(f, (uint32_t)c);
        s = min(s, mix_column((uint64_t)(uint32_t)c));
    }
    for (int o = 16; o > 0; o >>= 1) {
        f = min(f, __shfl_xor_sync(0xffffffffu, f, o));
        s = min(s, __shfl_xor_sync(0xffffffffu, s, o));
    }
    if (lane == 0) {
        first[r] = f;
        if (sig) sig[r] = s;
    }
}

template <typename KeyT>
__global__ void gather_keys_kernel(const KeyT* __restrict__ key_of_row, const int32_t* __restrict__ rows, int32_t n, KeyT* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = key_of_row[rows[i]];
}

// Stable sort of `rows` (n row ids) by key_of_row[row]: keys gathered, CUB radix sort by key.
template <typename KeyT>
int sort_rows_by(const KeyT* key_of_row, int32_t* rows_in, int32_t* rows_out, int32_t n, int end_bit, cudaStream_t st) {
    if (n == 0) return MASK_OK;
    DevBuf kin, kout, tmp;
    int rc = kin.alloc((size_t)n * sizeof(KeyT));
    if (rc == MASK_OK) rc = kout.alloc((size_t)n * sizeof(KeyT));
    if (rc != MASK_OK) return rc;
    gather_keys_kernel<KeyT><<<(n + 255) / 256, 256, 0, st>>>(key_of_row, rows_in, n, kin.as<KeyT>());
    size_t bytes = 0;
    MASK_CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, bytes, kin.as<KeyT>(), kout.as<KeyT>(), rows_in, rows_out, n, 0, end_bit, st));
    rc = tmp.alloc(bytes);
    if (rc != MASK_OK) return rc;
    MASK_CUDA_TRY(cub::DeviceRadixSort::SortPairs(tmp.p, bytes, kin.as<KeyT>(), kout.as<KeyT>(), rows_in, rows_out, n, 0, end_bit, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));   // the scratch goes away with this frame
    return MASK_OK;
}

// |cols(a) & cols(b)| by one warp: lanes walk the shorter row and search the longer one
__device__ int warp_intersection(const int32_t* __restrict__ ci, int a0, int a1, int b0, int b1, int lane) {
    if (a1 - a0 > b1 - b0) { int t = a0; a0 = b0; b0 = t; t = a1; a1 = b1; b1 = t; }
    int hits = 0;
    for (int q = a0 + lane; q < a1; q += 32) {
        const int c = ci[q];
        int lo = b0, hi = b1;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (ci[mid] < c) lo = mid + 1; else hi = mid;
        }
        hits += (lo < b1 && ci[lo] == c);
    }
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
    return hits;
}

// One block per bucket of 64 ranked rows: greedy chain by exact Jaccard similarity to the row placed
// last; among equally similar rows the smaller id wins.
__global__ void __launch_bounds__(256) jaccard_chain_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ colind,
                                                            const int32_t* __restrict__ ranked, int32_t M, int32_t* __restrict__ order) {
    __shared__ int rows[64];
    __shared__ double score[64];
    __shared__ int alive[64];
    __shared__ int cur;
    const int base = blockIdx.x * 64;
    const int n = min(64, M - base);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < 64) {
        rows[tid] = tid < n ? ranked[base + tid] : -1;
        alive[tid] = tid < n && tid > 0;
    }
    if (tid == 0) { cur = ranked[base]; order[base] = ranked[base]; }
    __syncthreads();
    for (int placed = 1; placed < n; placed++) {
        const int c0 = rowptr[cur], c1 = rowptr[cur + 1];
        for (int c = warp; c < n; c += 8) {
            if (!alive[c]) continue;
            const int r = rows[c];
            const int r0 = rowptr[r], r1 = rowptr[r + 1];
            const int inter = warp_intersection(colind, c0, c1, r0, r1, lane);
            const int uni = (c1 - c0) + (r1 - r0) - inter;
            if (lane == 0) score[c] = uni ? (double)inter / (double)uni : 1.0;
        }
        __syncthreads();
        if (warp == 0) {   // argmax of (score, -row id) over the remaining candidates
            double bs = -1.0;
            int bi = -1, br = 0x7fffffff;
            for (int c = lane; c < n; c += 32) {
                if (!alive[c]) continue;
                const double sc = score[c];
                if (sc > bs || (sc == bs && rows[c] < br)) { bs = sc; bi = c; br = rows[c]; }
            }
            for (int o = 16; o > 0; o >>= 1) {
                const double os = __shfl_xor_sync(0xffffffffu, bs, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o), orow = __shfl_xor_sync(0xffffffffu, br, o);
                if (oi >= 0 && (bi < 0 || os > bs || (os == bs && orow < br))) { bs = os; bi = oi; br = orow; }
            }
            if (lane == 0) {
                alive[bi] = 0;
                cur = br;
                order[base + placed] = br;
            }
        }
        __syncthreads();
    }
}

// ---- reverse Cuthill-McKee ------------------------------------------------------------------------
__global__ void sym_edge_keys_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ colind, int32_t M,
                                     uint64_t* __restrict__ keys) {
    // one warp per row; every stored (r, c) with c != r in range gives (r, c) and (c, r); others give a sentinel
    const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (r >= M) return;
    for (int q = rowptr[r] + lane; q < rowptr[r + 1]; q += 32) {
        const int c = colind[q];
        const bool ok = c >= 0 && c < M && c != r;
        keys[2 * (int64_t)q] = ok ? ((uint64_t)(uint32_t)r << 32 | (uint32_t)c) : ~0ULL;
        keys[2 * (int64_t)q + 1] = ok ? ((uint64_t)(uint32_t)c << 32 | (uint32_t)r) : ~0ULL;
    }
}
__global__ void count_sources_kernel(const uint64_t* __restrict__ keys, int64_t n, int32_t* __restrict__ deg) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && keys[i] != ~0ULL) atomicAdd(&deg[(int32_t)(keys[i] >> 32)], 1);
}
__global__ void split_targets_kernel(const uint64_t* __restrict__ keys, int64_t n, int32_t* __restrict__ adj) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) adj[i] = (int32_t)(keys[i] & 0xffffffffu);
}
__global__ void scatter_rank_kernel(const int32_t* __restrict__ starts, int32_t M, int32_t* __restrict__ rank) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < M) rank[starts[i]] = i;
}
// label[v] = min(label[v], labels of its neighbours), then one shortcut through the node that label names
// (labels are ranks, starts[label] is a node of the same component), so chains collapse in a logarithmic
// number of rounds; flag set when anything moved
__global__ void propagate_labels_kernel(const int64_t* __restrict__ beg, const int32_t* __restrict__ adj,
                                        const int32_t* __restrict__ starts, int32_t M, int32_t* __restrict__ label,
                                        int32_t* __restrict__ changed) {
    const int v = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (v >= M) return;
    int best = label[v];
    for (int64_t q = beg[v] + lane; q < beg[v + 1]; q += 32) best = min(best, label[adj[q]]);
    for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0) {
        best = min(best, label[starts[best]]);
        if (best < label[v]) { label[v] = best; *changed = 1; }
    }
}
__global__ void seed_frontier_kernel(const int32_t* __restrict__ label, const int32_t* __restrict__ rank, int32_t M,
                                     int32_t* __restrict__ frontier, int32_t* __restrict__ count, int32_t* __restrict__ pos) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= M) return;
    pos[v] = -1;
    if (label[v] == rank[v]) frontier[atomicAdd(count, 1)] = v;   // the component's node of least (degree, id)
}
__global__ void assign_positions_kernel(const int32_t* __restrict__ frontier, int32_t n, int32_t base, int32_t* __restrict__ pos) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pos[frontier[i]] = base + i;
}
// every unvisited neighbour of a frontier node records the earliest queue position that reaches it and
// is appended to the next level once
__global__ void expand_frontier_kernel(const int64_t* __restrict__ beg, const int32_t* __restrict__ adj,
                                       const int32_t* __restrict__ frontier, int32_t n, int32_t base, const int32_t* __restrict__ pos,
                                       int32_t* __restrict__ parent, int32_t* __restrict__ claimed, int32_t* __restrict__ next,
                                       int32_t* __restrict__ next_count) {
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (i >= n) return;
    const int v = frontier[i];
    for (int64_t q = beg[v] + lane; q < beg[v + 1]; q += 32) {
        const int nb = adj[q];
        if (pos[nb] >= 0) continue;
        atomicMin(&parent[nb], base + i);
        if (atomicExch(&claimed[nb], 1) == 0) next[atomicAdd(next_count, 1)] = nb;
    }
}
__global__ void final_keys_kernel(const int32_t* __restrict__ label, const int32_t* __restrict__ pos, int32_t M,
                                  uint64_t* __restrict__ keys, int32_t* __restrict__ ids) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= M) return;
    keys[v] = ((uint64_t)(uint32_t)label[v] << 32) | (uint32_t)(0x7fffffff - pos[v]);   // component by start rank, queue order reversed
    ids[v] = v;
}

int order_rcm_device(const int32_t* rowptr, const int32_t* colind, int32_t M, int64_t nnz, int32_t* order, cudaStream_t st) {
    const unsigned row_blocks = (unsigned)(((int64_t)M * 32 + 255) / 256), node_blocks = (unsigned)((M + 255) / 256);
    // symmetrised, deduplicated adjacency
    DevBuf keys, keys_sorted, keys_unique, n_unique_d, tmp, deg_b, beg_b, adj_b;
    const int64_t n_keys = 2 * nnz;
    int rc = keys.alloc((size_t)n_keys * 8);
    if (rc == MASK_OK) rc = keys_sorted.alloc((size_t)n_keys * 8);
    if (rc == MASK_OK) rc = keys_unique.alloc((size_t)n_keys * 8);
    if (rc == MASK_OK) rc = n_unique_d.alloc(8);
    if (rc == MASK_OK) rc = deg_b.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = beg_b.alloc(((size_t)M + 1) * 8);
    if (rc != MASK_OK) return rc;
    int64_t n_edges = 0;
    if (n_keys > 0) {
        if (n_keys >= ((int64_t)1 << 31)) return fail(MASK_ERR_INDEX_OVERFLOW, "too many entries for the device reorder");
        sym_edge_keys_kernel<<<row_blocks, 256, 0, st>>>(rowptr, colind, M, keys.as<uint64_t>());
        size_t bytes = 0, bytes2 = 0;
        MASK_CUDA_TRY(cub::DeviceRadixSort::SortKeys(nullptr, bytes, keys.as<uint64_t>(), keys_sorted.as<uint64_t>(), (int)n_keys, 0, 64, st));
        MASK_CUDA_TRY(cub::DeviceSelect::Unique(nullptr, bytes2, keys_sorted.as<uint64_t>(), keys_unique.as<uint64_t>(), n_unique_d.as<int64_t>(), (int)n_keys, st));
        rc = tmp.alloc(std::max(bytes, bytes2));
        if (rc != MASK_OK) return rc;
        MASK_CUDA_TRY(cub::DeviceRadixSort::SortKeys(tmp.p, bytes, keys.as<uint64_t>(), keys_sorted.as<uint64_t>(), (int)n_keys, 0, 64, st));
        MASK_CUDA_TRY(cub::DeviceSelect::Unique(tmp.p, bytes2, keys_sorted.as<uint64_t>(), keys_unique.as<uint64_t>(), n_unique_d.as<int64_t>(), (int)n_keys, st));
        MASK_CUDA_TRY(cudaMemcpyAsync(&n_edges, n_unique_d.p, 8, cudaMemcpyDeviceToHost, st));
        MASK_CUDA_TRY(cudaStreamSynchronize(st));
        // the sentinel (all ones) sorts last and, if present, is one unique key: drop it
        if (n_edges > 0) {
            uint64_t last = 0;
            MASK_CUDA_TRY(cudaMemcpy(&last, keys_unique.as<uint64_t>() + (n_edges - 1), 8, cudaMemcpyDeviceToHost));
            if (last == ~0ULL) n_edges--;
        }
    }
    MASK_CUDA_TRY(cudaMemsetAsync(deg_b.p, 0, (size_t)M * 4, st));
    rc = adj_b.alloc((size_t)std::max<int64_t>(n_edges, 1) * 4);
    if (rc != MASK_OK) return rc;
    if (n_edges > 0) {
        const unsigned eb = (unsigned)((n_edges + 255) / 256);
        count_sources_kernel<<<eb, 256, 0, st>>>(keys_unique.as<uint64_t>(), n_edges, deg_b.as<int32_t>());
        split_targets_kernel<<<eb, 256, 0, st>>>(keys_unique.as<uint64_t>(), n_edges, adj_b.as<int32_t>());
    }
    {   // beg = exclusive scan of the degrees (64-bit), closing entry = n_edges
        size_t bytes = 0;
        DevBuf t2;
        auto deg64 = cub::TransformInputIterator<int64_t, cub::CastOp<int64_t>, const int32_t*>(deg_b.as<int32_t>(), cub::CastOp<int64_t>());
        MASK_CUDA_TRY(cub::DeviceScan::ExclusiveSum(nullptr, bytes, deg64, beg_b.as<int64_t>(), M, st));
        rc = t2.alloc(bytes);
        if (rc != MASK_OK) return rc;
        MASK_CUDA_TRY(cub::DeviceScan::ExclusiveSum(t2.p, bytes, deg64, beg_b.as<int64_t>(), M, st));
        MASK_CUDA_TRY(cudaMemcpyAsync(beg_b.as<int64_t>() + M, &n_edges, 8, cudaMemcpyHostToDevice, st));
        MASK_CUDA_TRY(cudaStreamSynchronize(st));
    }
    // rank of every node in (degree, id) order
    DevBuf ids, starts, rank, label, flag;
    rc = ids.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = starts.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = rank.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = label.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = flag.alloc(16);
    if (rc != MASK_OK) return rc;
    iota_kernel<<<node_blocks, 256, 0, st>>>(ids.as<int32_t>(), M);
    rc = sort_rows_by<uint32_t>(deg_b.as<uint32_t>(), ids.as<int32_t>(), starts.as<int32_t>(), M, 32, st);
    if (rc != MASK_OK) return rc;
    scatter_rank_kernel<<<node_blocks, 256, 0, st>>>(starts.as<int32_t>(), M, rank.as<int32_t>());
    // connected components: label = least rank in the component
    MASK_CUDA_TRY(cudaMemcpyAsync(label.p, rank.p, (size_t)M * 4, cudaMemcpyDeviceToDevice, st));
    for (int it = 0; it < M + 1; it++) {
        int32_t changed = 0;
        MASK_CUDA_TRY(cudaMemsetAsync(flag.p, 0, 4, st));
        propagate_labels_kernel<<<row_blocks, 256, 0, st>>>(beg_b.as<int64_t>(), adj_b.as<int32_t>(), starts.as<int32_t>(), M, label.as<int32_t>(), flag.as<int32_t>());
        MASK_CUDA_TRY(cudaMemcpyAsync(&changed, flag.p, 4, cudaMemcpyDeviceToHost, st));
        MASK_CUDA_TRY(cudaStreamSynchronize(st));
        if (!changed) break;
    }
    // breadth-first levels of all components at once, in queue order
    DevBuf pos, parent, claimed, fa, fb, fs, counter;
    rc = pos.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = parent.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = claimed.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = fa.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = fb.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = fs.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = counter.alloc(16);
    if (rc != MASK_OK) return rc;
    MASK_CUDA_TRY(cudaMemsetAsync(parent.p, 0x7f, (size_t)M * 4, st));
    MASK_CUDA_TRY(cudaMemsetAsync(claimed.p, 0, (size_t)M * 4, st));
    MASK_CUDA_TRY(cudaMemsetAsync(counter.p, 0, 16, st));
    seed_frontier_kernel<<<node_blocks, 256, 0, st>>>(label.as<int32_t>(), rank.as<int32_t>(), M, fa.as<int32_t>(), counter.as<int32_t>(), pos.as<int32_t>());
    int32_t n_front = 0;
    MASK_CUDA_TRY(cudaMemcpyAsync(&n_front, counter.p, 4, cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    // the start nodes in component order (by their rank)
    rc = sort_rows_by<uint32_t>(rank.as<uint32_t>(), fa.as<int32_t>(), fb.as<int32_t>(), n_front, 32, st);
    if (rc != MASK_OK) return rc;
    int32_t* cur = fb.as<int32_t>();
    int32_t* nxt = fa.as<int32_t>();
    int32_t base = 0;
    while (n_front > 0) {
        assign_positions_kernel<<<(n_front + 255) / 256, 256, 0, st>>>(cur, n_front, base, pos.as<int32_t>());
        MASK_CUDA_TRY(cudaMemsetAsync(counter.p, 0, 4, st));
        expand_frontier_kernel<<<(unsigned)(((int64_t)n_front * 32 + 255) / 256), 256, 0, st>>>(
            beg_b.as<int64_t>(), adj_b.as<int32_t>(), cur, n_front, base, pos.as<int32_t>(), parent.as<int32_t>(), claimed.as<int32_t>(), nxt,
            counter.as<int32_t>());
        int32_t n_next = 0;
        MASK_CUDA_TRY(cudaMemcpyAsync(&n_next, counter.p, 4, cudaMemcpyDeviceToHost, st));
        MASK_CUDA_TRY(cudaStreamSynchronize(st));
        base += n_front;
        if (n_next > 0) {   // next level in (parent position, degree, id) order: three stable passes, least significant key first
            rc = sort_rows_by<uint32_t>(ids.as<uint32_t>(), nxt, fs.as<int32_t>(), n_next, 32, st);          // key = the id itself
            if (rc == MASK_OK) rc = sort_rows_by<uint32_t>(deg_b.as<uint32_t>(), fs.as<int32_t>(), nxt, n_next, 32, st);
            if (rc == MASK_OK) rc = sort_rows_by<uint32_t>(parent.as<uint32_t>(), nxt, fs.as<int32_t>(), n_next, 32, st);
            if (rc != MASK_OK) return rc;
            MASK_CUDA_TRY(cudaMemcpyAsync(cur == fb.as<int32_t>() ? fa.p : fb.p, fs.p, (size_t)n_next * 4, cudaMemcpyDeviceToDevice, st));
        }
        std::swap(cur, nxt);
        n_front = n_next;
    }
    if (base != M) return fail(MASK_ERR_INVALID_ARGUMENT, "row_rcm: the traversal did not reach every row");
    // components by the rank of their start, each in reversed queue order
    DevBuf fk, fk2, tmp2;
    rc = fk.alloc((size_t)M * 8);
    if (rc == MASK_OK) rc = fk2.alloc((size_t)M * 8);
    if (rc != MASK_OK) return rc;
    final_keys_kernel<<<node_blocks, 256, 0, st>>>(label.as<int32_t>(), pos.as<int32_t>(), M, fk.as<uint64_t>(), ids.as<int32_t>());
    size_t bytes = 0;
    MASK_CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, bytes, fk.as<uint64_t>(), fk2.as<uint64_t>(), ids.as<int32_t>(), order, M, 0, 64, st));
    rc = tmp2.alloc(bytes);
    if (rc != MASK_OK) return rc;
    MASK_CUDA_TRY(cub::DeviceRadixSort::SortPairs(tmp2.p, bytes, fk.as<uint64_t>(), fk2.as<uint64_t>(), ids.as<int32_t>(), order, M, 0, 64, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    return MASK_OK;
}

}  // namespace

// ---- device: gather the rows of a CSR matrix in a given order ------------------------------------
__global__ void permuted_row_lengths_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ order, int32_t M,
                                            int32_t* __restrict__ len) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < M) { const int r = order[i]; len[i] = rowptr[r + 1] - rowptr[r]; }
}
// one warp per new row copies its entries
__global__ void gather_rows_kernel(const int32_t* __restrict__ rowptr, const int32_t* __restrict__ colind,
                                   const float* __restrict__ values, const int32_t* __restrict__ order,
                                   const int32_t* __restrict__ rowptr_out, int32_t M, int32_t* __restrict__ colind_out,
                                   float* __restrict__ values_out) {
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (i >= M) return;
    const int r = order[i];
    const int src = rowptr[r], n = rowptr[r + 1] - src, dst = rowptr_out[i];
    for (int j = lane; j < n; j += 32) {
        colind_out[dst + j] = colind[src + j];
        values_out[dst + j] = values[src + j];
    }
}
// single-block exclusive scan of M lengths (row counts are small next to the entry counts the
// format builder scans; 4 M rows take well under a millisecond)
__global__ void __launch_bounds__(1024) scan_lengths_kernel(const int32_t* __restrict__ len, int32_t M, int32_t* __restrict__ rowptr_out) {
    __shared__ int64_t warp_tot[32];
    __shared__ int64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int base = 0; base < M; base += 1024) {
        const int idx = base + threadIdx.x;
        const int64_t v = idx < M ? len[idx] : 0;
        int64_t x = v;
        for (int o = 1; o < 32; o <<= 1) { const int64_t y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        if (lane == 31) warp_tot[wid] = x;
        __syncthreads();
        if (wid == 0) {
            int64_t w = warp_tot[lane];
            for (int o = 1; o < 32; o <<= 1) { const int64_t y = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += y; }
            warp_tot[lane] = w;
        }
        __syncthreads();
        const int64_t before = carry + (wid > 0 ? warp_tot[wid - 1] : 0);
        if (idx < M) rowptr_out[idx] = (int32_t)(before + x - v);
        __syncthreads();
        if (threadIdx.x == 0) carry += warp_tot[31];
        __syncthreads();
    }
    if (threadIdx.x == 0) rowptr_out[M] = (int32_t)carry;
}

}  // namespace mask

extern "C" int mask_reorder_rows(int kind, const int32_t* d_rowptr, const int32_t* d_colind, int32_t M, int32_t K,
                                 int32_t* d_row_order, void* stream) {
    using namespace mask;
    MASK_REQUIRE(d_rowptr && d_row_order && M >= 1 && K >= 1, "bad arguments");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned node_blocks = (unsigned)((M + 255) / 256), row_blocks = (unsigned)(((int64_t)M * 32 + 255) / 256);
    if (kind == MASK_REORDER_NONE) {
        iota_kernel<<<node_blocks, 256, 0, st>>>(d_row_order, M);
        MASK_CUDA_TRY(cudaGetLastError());
        return MASK_OK;
    }
    MASK_REQUIRE(kind == MASK_REORDER_ROW_RCM || kind == MASK_REORDER_FIRST_COL_SORT || kind == MASK_REORDER_JACCARD_GREEDY,
                 "unknown reorder kind");
    int32_t nnz32 = 0;
    MASK_CUDA_TRY(cudaMemcpyAsync(&nnz32, d_rowptr + M, 4, cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    MASK_REQUIRE(nnz32 == 0 || d_colind, "colind is NULL");
    if (kind == MASK_REORDER_ROW_RCM) {
        if (M != K) return fail(MASK_ERR_INVALID_ARGUMENT, "row_rcm needs a square matrix");
        return order_rcm_device(d_rowptr, d_colind, M, nnz32, d_row_order, st);
    }
    DevBuf first, sig, ids, by_first;
    int rc = first.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = sig.alloc((size_t)M * 8);
    if (rc == MASK_OK) rc = ids.alloc((size_t)M * 4);
    if (rc == MASK_OK) rc = by_first.alloc((size_t)M * 4);
    if (rc != MASK_OK) return rc;
    row_keys_kernel<<<row_blocks, 256, 0, st>>>(d_rowptr, d_colind, M, K, first.as<uint32_t>(), sig.as<uint64_t>());
    iota_kernel<<<node_blocks, 256, 0, st>>>(ids.as<int32_t>(), M);
    MASK_CUDA_TRY(cudaGetLastError());
    if (kind == MASK_REORDER_FIRST_COL_SORT) return sort_rows_by<uint32_t>(first.as<uint32_t>(), ids.as<int32_t>(), d_row_order, M, 32, st);
    // (signature, first column, id): stable by first column, then stable by signature
    rc = sort_rows_by<uint32_t>(first.as<uint32_t>(), ids.as<int32_t>(), by_first.as<int32_t>(), M, 32, st);
    if (rc == MASK_OK) rc = sort_rows_by<uint64_t>(sig.as<uint64_t>(), by_first.as<int32_t>(), ids.as<int32_t>(), M, 64, st);
    if (rc != MASK_OK) return rc;
    jaccard_chain_kernel<<<(unsigned)((M + 63) / 64), 256, 0, st>>>(d_rowptr, d_colind, ids.as<int32_t>(), M, d_row_order);
    MASK_CUDA_TRY(cudaGetLastError());
    MASK_CUDA_TRY(cudaStreamSynchronize(st));   // the scratch goes away with this frame
    return MASK_OK;
}

extern "C" int mask_csr_permute_rows(const int32_t* d_rowptr, const int32_t* d_colind, const float* d_values, int32_t M,
                                     const int32_t* d_row_order, int32_t* d_rowptr_out, int32_t* d_colind_out,
                                     float* d_values_out, void* stream) {
    using namespace mask;
    MASK_REQUIRE(d_rowptr && d_row_order && d_rowptr_out && M >= 1, "bad arguments");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // row lengths in the new order go to rowptr_out[1..M] first, then are scanned in place
    permuted_row_lengths_kernel<<<(M + 255) / 256, 256, 0, st>>>(d_rowptr, d_row_order, M, d_rowptr_out + 1);
    MASK_CUDA_TRY(cudaGetLastError());
    // in place: the scan reads len[i] = rowptr_out[i+1] into registers before a block barrier and
    // writes rowptr_out[i] after it; later chunks only read positions no earlier chunk has written
    scan_lengths_kernel<<<1, 1024, 0, st>>>(d_rowptr_out + 1, M, d_rowptr_out);
    MASK_CUDA_TRY(cudaGetLastError());
    if (d_colind && d_values && d_colind_out && d_values_out) {
        gather_rows_kernel<<<(unsigned)(((int64_t)M * 32 + 255) / 256), 256, 0, st>>>(d_rowptr, d_colind, d_values, d_row_order,
                                                                                   d_rowptr_out, M, d_colind_out, d_values_out);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    return MASK_OK;
}
