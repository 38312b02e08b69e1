// SR-BCRS 16x8 SpMM with a TMA producer: the Blackwell pipeline with nothing in it but the tensor
// memory accelerator, the tensor core and the epilogue.
//
//   producer warp  --(full[s]: transaction bytes)-->  MMA thread  --(acc_full)-->  4 epilogue warps
//        ^------------------(empty[s]: tcgen05.commit)-----'  ^------(acc_empty)--------'
//
// Same transposed product, operand layouts, work decomposition (resident grid, column blocks of
// 128*NSLAB columns swept one after the other, groups dealt round-robin) and epilogue as
// spmm_sweep.cu; what differs is how the operands reach shared memory:
//   * The 8 gathered rows of B of a tile and 128-column slab are fetched by 8 instructions
//     cp.async.bulk.tensor.2d ... tile::gather4: each takes 4 row numbers and a column, copies
//     4 rows x 32 columns (4 x 128 bytes) and writes them in the 128-byte swizzle with 32-byte atoms
//     -- exactly one 512-byte atom of the MN-major operand layout the tensor core reads.  A step is
//     32 such copies, one per lane of the producer warp, so the gather costs the SM two warp
//     instructions per 16 KB instead of the 32 cp.async warp instructions (plus address arithmetic)
//     of the copy-based kernel.  Columns beyond N are filled with zeros by the unit.
//   * The unit writes through the asynchronous proxy, which is the one the tensor core reads
//     through: no proxy fence, hence no preparation stage between arrival and MMA.  The MMA thread
//     waits on full[s] itself.
//   * That leaves the rounding of the tile values to TF32 (ties away, like the reference's cvt.rna,
//     examples/src_fp32/sr_bcrs/testbed/kernel.inc:809-814): it is done once per matrix instead of once
//     per use.  The plan holds a rounded copy of val_block_val (mask_plan_prepare_values); tiles are
//     copied from it verbatim with one cp.async.bulk of 512 bytes each.
// Six warps, 192 threads: with that few threads the epilogue keeps a whole 16 x 512 accumulator
// in registers without spilling, and the role loops are short.
//
// The tensor map covers this GPU's own copy of B only; nothing here names a peer's memory, and no
// copy is multicast.  Every wait is bounded; an expired wait raises the block's abort flag and the
// plan's status word, every role leaves its loops, the block waits out its copies in flight and
// the tensor core's work, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "spmm_common.cuh"
#include "umma_ptx.cuh"

namespace mask {

constexpr int kTmaThreads = 192;

template <int NSLAB>
struct TmaLayout {
    static constexpr int KT = 4 / NSLAB;                            // tiles per step
    static constexpr int S = 6;                                     // ring stages
    static constexpr int kStageB = 4 * 4096;                        // gathered rows of one step
    static constexpr int kStageA = KT * 512;                        // tile operand(s) of one step
    static constexpr int kNacc = NSLAB == 4 ? 4 : 8;                // accumulator buffers
    static constexpr int kAccCols = 16 * NSLAB;
    static constexpr int kTmemCols = kNacc * kAccCols;              // 256, 256, 128: two blocks fit an SM's 512
    static constexpr int kB = 0;
    static constexpr int kA = S * kStageB;
    static constexpr int kBars = kA + S * kStageA;                  // full[S], empty[S], acc_full[NACC], acc_empty[NACC], drain
    static constexpr int kNumBars = 2 * S + 2 * kNacc + 1;
    static constexpr int kTmemSlot = kBars + kNumBars * 8;
    static constexpr int kAbort = kTmemSlot + 8;
    static constexpr int kBytes = kAbort + 8;
    static constexpr int kDynamicBytes = kBytes + 1024;             // room to align the base to 1024 B
};

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// 4 rows (y0..y3) x 32 columns starting at column x of the 2-D tensor behind `map`, to 512 bytes of
// shared memory in the map's swizzle; completes on `bar` with 512 transaction bytes.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y0, int y1, int y2, int y3) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
        : "memory");
}
__device__ __forceinline__ void bulk_copy_512(uint32_t dst, const void* src, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];" ::"r"(dst), "l"(src), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_wait_clock_only(uint32_t bar, uint32_t parity) {
    const long long start = clock64();
    while (!mbar_test(bar, parity)) {
        if (clock64() - start > kUmmaWaitCycles) return false;
    }
    return true;
}

template <int NSLAB>
__global__ void __launch_bounds__(kTmaThreads, 2) spmm_tma_kernel(const SpmmArgs p, const __grid_constant__ CUtensorMap bmap,
                                                                   const float* __restrict__ vals_tf32, int32_t* status) {
    using L = TmaLayout<NSLAB>;
    constexpr int KT = L::KT, S = L::S, NACC = L::kNacc, kAccCols = L::kAccCols;
    extern __shared__ unsigned char tma_smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(tma_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                   // swizzle patterns are functions of the address bits
    unsigned char* gbase = tma_smem_raw + (base - raw);
    const uint32_t bars = base + L::kBars;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * S + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * S + NACC + b); };
    const uint32_t drain_bar = bars + 8u * (2 * S + 2 * NACC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + L::kAbort);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::kTmemSlot);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.n_groups;
    const int n_items = p.n_col_blocks * G;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 1);     // the producer's arrive.expect_tx; the copies complete the bytes
            mbar_init(empty_bar(s), 1);    // tcgen05.commit
        }
        for (int b = 0; b < NACC; b++) {
            mbar_init(accf_bar(b), 1);     // tcgen05.commit
            mbar_init(acce_bar(b), 4);     // lane 0 of every epilogue warp
        }
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + L::kTmemSlot),
                     "r"(L::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // item -> (column block, group): column blocks slowest, odd ones walk the groups backwards
    auto item_cb = [&](int item) { return item / G; };
    auto item_group = [&](int item, int cb) {
        const int gi = item - cb * G;
        return (cb & 1) ? G - 1 - gi : gi;
    };

    if (warp == 5) {
        // ------------------------------ producer (one warp, every lane issues one gather per step) ----
        const int unit = lane >> 3;              // which of the step's 4 units: tile u = unit / NSLAB, slab sl = unit % NSLAB
        const int u = unit / NSLAB, sl = unit % NSLAB;
        const int atom = (lane >> 1) & 3;        // 32-column atom of the unit
        const int half = lane & 1;               // rows 0-3 or 4-7 of the tile
        const uint32_t dst_off = (uint32_t)(unit * 4096 + atom * 1024 + half * 512);
        const int idl = lane & (8 * KT - 1);     // which of the step's 8*KT ids this lane loads
        const int id_src = u * kTileCols + half * 4;
        int s = 0;
        uint32_t round = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int cb = item_cb(item);
            const int g = item_group(item, cb);
            const int t0 = p.group_tile[g], t1 = p.group_tile[g + 1];
            const int x = cb * (128 * NSLAB) + sl * 128 + atom * 32;
            const bool col_ok = x < p.N;
            auto load_ids = [&](int tb) -> int {
                const int64_t at = (int64_t)tb * kTileCols + idl;
                return at < (int64_t)t1 * kTileCols ? __ldg(p.val_sidx + at) : 0;
            };
            // One step; q holds its ids (loaded four steps ago) and is refilled in place for the step four
            // ahead, so a queue register is never moved while its load is in flight.
            auto produce = [&](int tb, int& q) -> bool {
                const int cnt = min(KT, t1 - tb);
                const int y0 = __shfl_sync(0xffffffffu, q, id_src), y1 = __shfl_sync(0xffffffffu, q, id_src + 1);
                const int y2 = __shfl_sync(0xffffffffu, q, id_src + 2), y3 = __shfl_sync(0xffffffffu, q, id_src + 3);
                q = load_ids(tb + 4 * KT);
                if (round > 0 && !__all_sync(0xffffffffu, mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag))) return false;
                const bool active = col_ok && u < cnt;
                const uint32_t n_active = __popc(__ballot_sync(0xffffffffu, active));
                const uint32_t bar = full_bar(s);
                if (lane == 0) mbar_arrive_expect_tx(bar, 512u * (n_active + (uint32_t)cnt));
                __syncwarp();   // the bytes are announced before any copy can complete them
                if (active) tma_gather4(base + L::kB + s * L::kStageB + dst_off, &bmap, bar, x, y0, y1, y2, y3);
                if (lane < cnt) bulk_copy_512(base + L::kA + s * L::kStageA + lane * 512, vals_tf32 + (int64_t)(tb + lane) * kTileElems, bar);
                if (++s == S) { s = 0; round++; }
                return true;
            };
            int q0 = load_ids(t0), q1 = load_ids(t0 + KT), q2 = load_ids(t0 + 2 * KT), q3 = load_ids(t0 + 3 * KT);
            for (int tb = t0; tb < t1; tb += 4 * KT) {
                if (!produce(tb, q0)) { ok = false; break; }
                if (tb + KT >= t1) break;
                if (!produce(tb + KT, q1)) { ok = false; break; }
                if (tb + 2 * KT >= t1) break;
                if (!produce(tb + 2 * KT, q2)) { ok = false; break; }
                if (tb + 3 * KT >= t1) break;
                if (!produce(tb + 3 * KT, q3)) { ok = false; break; }
            }
        }
    } else if (warp == 4) {
        // ------------------------------ MMA issuer (one lane) ------------------------------------------
        if (lane == 0) {
            const uint64_t a0 = umma_smem_desc(base + L::kB, 64, 32, kSwizzle128B32B);
            const uint64_t b0 = umma_smem_desc(base + L::kA, 1, 16, kSwizzle32B);
            const uint32_t a_hi = (uint32_t)(a0 >> 32), b_hi = (uint32_t)(b0 >> 32);
            uint32_t a_lo = (uint32_t)a0, b_lo = (uint32_t)b0;     // of stage s
            int s = 0;
            uint32_t round = 0, acc_it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const int g = item_group(item, item_cb(item));
                int f = p.group_off[g];
                const int t1 = p.group_tile[g + 1];
                int t = p.group_tile[g];
                int f_end_tile = p.frag_off[f + 1];                               // end of fragment f
                int f_next_end = p.frag_off[min((int64_t)f + 2, p.n_frag)];      // end of fragment f + 1, loaded ahead
                uint32_t open = 0;                                                // 1 while the fragment has MMAs in flight
                uint32_t acc = tmem_base;                                         // accumulator of the open fragment
                uint32_t buf = 0;
                while (t < t1) {
                    const int cnt = min(KT, t1 - t);
                    if (!mbar_wait_spin(full_bar(s), round & 1, abort_flag)) { ok = false; break; }   // spins: this thread paces the block
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int u = 0; u < KT; u++) {
                        if (u < cnt) {
                            if (t >= f_end_tile || !open) {
                                while (t >= f_end_tile) {   // on to the fragment that holds tile t (fragments without tiles are skipped)
                                    if (open) { umma_commit(accf_bar(buf)); acc_it++; open = 0; }
                                    f++;
                                    f_end_tile = f_next_end;
                                    f_next_end = p.frag_off[min((int64_t)f + 2, p.n_frag)];
                                }
                                buf = acc_it % NACC;
                                acc = tmem_base + buf * kAccCols;
                                if (acc_it >= (uint32_t)NACC && !mbar_wait(acce_bar(buf), (acc_it / NACC - 1) & 1, abort_flag)) { ok = false; break; }
                                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            }
#pragma unroll
                            for (int sl = 0; sl < NSLAB; sl++)
                                umma_tf32_split(acc + sl * 16, a_lo + (u * NSLAB + sl) * (4096 >> 4), a_hi, b_lo + u * (512 >> 4), b_hi, open);
                            open = 1;
                            t++;
                        }
                    }
                    if (!ok) break;
                    umma_commit(empty_bar(s));   // the slot is free once these MMAs have read it
                    a_lo += L::kStageB >> 4;
                    b_lo += L::kStageA >> 4;
                    if (++s == S) {
                        s = 0; round++;
                        a_lo = (uint32_t)a0; b_lo = (uint32_t)b0;
                    }
                }
                if (open) { umma_commit(accf_bar(buf)); acc_it++; }
            }
            // whatever was issued must have finished before shared and tensor memory go away
            umma_commit(drain_bar);
            if (!mbar_wait_clock_only(drain_bar, 0)) *abort_flag = 1;
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue -------------------------------------------------
        uint32_t acc_it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int cb = item_cb(item);
            const int g = item_group(item, cb);
            const int col = cb * (128 * NSLAB) + 32 * warp + lane;   // + 128 * slab
            const int f0 = p.group_off[g], f_end = p.group_off[g + 1];
            // fragment f's tile count, window and slot are loaded one fragment ahead
            int nxt_n = 0, nxt_w = 0, nxt_slot = -1;
            if (f0 < f_end) {
                nxt_n = p.frag_off[f0 + 1] - p.frag_off[f0];
                nxt_w = p.frag_win[f0];
                nxt_slot = p.frag_slot[f0];
            }
            bool colok[NSLAB];
#pragma unroll
            for (int sl = 0; sl < NSLAB; sl++) colok[sl] = col + 128 * sl < p.N;
            for (int f = f0; f < f_end; f++) {
                const int n = nxt_n, w = nxt_w, slot = nxt_slot;
                if (f + 1 < f_end) {
                    nxt_n = p.frag_off[f + 2] - p.frag_off[f + 1];
                    nxt_w = p.frag_win[f + 1];
                    nxt_slot = p.frag_slot[f + 1];
                }
                const int rows_ok = slot < 0 ? p.M - w * kWinRows : kWinRows;
                const bool relu = p.relu && slot < 0;
                uint32_t v[NSLAB][16];
                if (n == 0) {
#pragma unroll
                    for (int sl = 0; sl < NSLAB; sl++)
#pragma unroll
                        for (int i = 0; i < 16; i++) v[sl][i] = 0u;
                } else {
                    const uint32_t buf = acc_it % NACC;
                    if (!__all_sync(0xffffffffu, mbar_wait(accf_bar(buf), (acc_it / NACC) & 1, abort_flag))) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t taddr = tmem_base + ((uint32_t)(32 * warp) << 16) + buf * kAccCols;
#pragma unroll
                    for (int sl = 0; sl < NSLAB; sl++) tmem_ld16(taddr + sl * 16, v[sl]);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acce_bar(buf));   // the MMA warp may reuse this buffer
                    acc_it++;
                }
                if (relu) {
#pragma unroll
                    for (int sl = 0; sl < NSLAB; sl++)
#pragma unroll
                        for (int i = 0; i < 16; i++) v[sl][i] = __float_as_uint(fmaxf(__uint_as_float(v[sl][i]), 0.f));
                }
                // destination 0 is C (or the partial-tile scratch); 1.. are the peers' copies of C, which
                // get the finished rows with plain stores over NVLink
                const int n_dst = slot < 0 ? 1 + p.n_peer_out : 1;
                const int64_t ld = slot >= 0 ? (int64_t)p.N : p.ldc;
                const int32_t* rm = slot >= 0 ? nullptr : p.row_map;
                const int row00 = slot >= 0 ? 0 : w * kWinRows;
#pragma unroll 1
                for (int d = 0; d < n_dst; d++) {
                    int row0 = row00;
                    asm volatile("" : "+r"(row0));   // keeps the 16 row offsets from being hoisted out of this loop into registers
                    float* dst = (slot >= 0 ? p.scratch + (int64_t)slot * kWinRows * p.N : (d == 0 ? p.C : p.peer_out[d - 1])) + col;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int r = i ^ (i >> 3);   // MMA-N index -> window row (SR-BCRS stores rows 8..15 swapped pairwise)
                        if (r < rows_ok) {
                            float* rowp = dst + (int64_t)(rm ? rm[row0 + r] : row0 + r) * ld;
#pragma unroll
                            for (int sl = 0; sl < NSLAB; sl++) {
                                if (colok[sl]) {
                                    rowp[128 * sl] = __uint_as_float(v[sl][i]);
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    // ---- teardown: everybody gets here, aborting or not ---------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        // copies that were issued but never consumed may still be landing in this block's shared memory:
        // give them a millisecond (they take microseconds) before the block goes away
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {
        }
        __syncthreads();
    }
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::kTmemCols) : "memory");
    }
    if (tid == 0 && *abort_flag) atomicExch(status, 1);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (the library does not link libcuda).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// B as a 2-D tensor [K rows][N columns] with row pitch ldb; box = 32 columns x 1 row (gather4 takes
// four such rows), 128-byte swizzle with 32-byte atoms: the MN-major operand layout for 32-bit types.
static int make_b_map(CUtensorMap* map, const float* B, int64_t K, int32_t N, int64_t ldb) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(MASK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
    const cuuint64_t strides[1] = {(cuuint64_t)ldb * 4};
    const cuuint32_t box[2] = {32, 1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(B), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (K=%lld N=%d ldb=%lld)", (int)r, (long long)K, (int)N, (long long)ldb);
        return MASK_ERR_CUDA;
    }
    return MASK_OK;
}

template <int NSLAB>
static int launch_tma_variant(const mask_plan* plan, SpmmArgs a, const CUtensorMap& map, cudaStream_t st) {
    using L = TmaLayout<NSLAB>;
    static_assert(2 * (L::kDynamicBytes + 1024) <= 228 * 1024, "two blocks per SM");
    auto kern = spmm_tma_kernel<NSLAB>;
    MASK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));   // per device
    MASK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    // two blocks per SM by construction (shared memory asserted above; tensor memory at most 256 of 512 columns per block)
    a.n_col_blocks = (a.N + 128 * NSLAB - 1) / (128 * NSLAB);
    const int64_t items = (int64_t)a.n_col_blocks * plan->G;
    if (items >= ((int64_t)1 << 31)) return fail(MASK_ERR_INVALID_ARGUMENT, "too many work items");
    const int64_t resident = 2 * (int64_t)sm_count();
    const unsigned grid = (unsigned)(items < resident ? items : resident);
    kern<<<grid, kTmaThreads, L::kDynamicBytes, st>>>(a, map, plan->d_vals_tf32, plan->d_status);
    MASK_CUDA_TRY(cudaGetLastError());
    return MASK_OK;
}

// True when this plan and operand can take the TMA kernel: rounded tile values prepared from exactly
// these values, and a row pitch the tensor map can express.
bool spmm_tma_applies(const mask_plan* plan, const SpmmArgs& a) {
    return plan->d_vals_tf32 != nullptr && plan->vals_src == a.val_blk && a.coo_off == nullptr && a.mco_mask == nullptr &&
           a.N >= 32 && a.ldb % 4 == 0 && (reinterpret_cast<uintptr_t>(a.B) & 15) == 0 && encode_tiled_fn() != nullptr;
}

int launch_spmm_tma(const mask_plan* plan, const SpmmArgs& a, int64_t K, cudaStream_t st, int nslab) {
    const int fills = a.N > 256 ? 4 : (a.N > 128 ? 2 : 1);   // slabs N can fill
    if (nslab != 1 && nslab != 2 && nslab != 4) nslab = fills;
    nslab = nslab < fills ? nslab : fills;
    CUtensorMap map;
    int rc = make_b_map(&map, a.B, K, a.N, a.ldb);
    if (rc != MASK_OK) return rc;
    SpmmArgs b = a;
    b.group_tile = plan->d_group_tile;
    b.n_groups = (int32_t)plan->G;
    b.n_frag = plan->F;
    if (nslab == 1) return launch_tma_variant<1>(plan, b, map, st);
    if (nslab == 2) return launch_tma_variant<2>(plan, b, map, st);
    return launch_tma_variant<4>(plan, b, map, st);
}

// ---- the rounded copy of the tile values --------------------------------------------------------------
__global__ void round_values_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int64_t n_vec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        uint4 v = __ldg(in + i);
        v.x += 0x1000u; v.y += 0x1000u; v.z += 0x1000u; v.w += 0x1000u;   // nearest, ties away: the tensor core drops the low 13 bits
        out[i] = v;
    }
}

}  // namespace mask

extern "C" int mask_plan_prepare_values(mask_plan* plan, const float* d_val_block_val, void* stream) {
    using namespace mask;
    MASK_REQUIRE(plan != nullptr, "plan is NULL");
    if (plan->d_vals_tf32) {
        MASK_CUDA_TRY(cudaFree(plan->d_vals_tf32));
        plan->d_vals_tf32 = nullptr;
    }
    plan->vals_src = nullptr;
    if (d_val_block_val == nullptr || plan->T == 0) return MASK_OK;
    MASK_REQUIRE((reinterpret_cast<uintptr_t>(d_val_block_val) & 15) == 0, "val_block_val must be 16-byte aligned");
    const int64_t n_vec = plan->T * (kTileElems / 4);
    MASK_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&plan->d_vals_tf32), (size_t)n_vec * 16));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (unsigned)std::min<int64_t>((n_vec + 255) / 256, (int64_t)sm_count() * 16);
    round_values_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(d_val_block_val), reinterpret_cast<uint4*>(plan->d_vals_tf32), n_vec);
    MASK_CUDA_TRY(cudaGetLastError());
    plan->vals_src = d_val_block_val;
    return MASK_OK;
}
