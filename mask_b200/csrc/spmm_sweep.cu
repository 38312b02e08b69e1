// Persistent tcgen05 SpMM: one resident grid sweeps the matrix once per block of 128*NSLAB columns.
//
// The product is issued transposed: for every tile t and 128-column slab,
//     D^T[128 columns x 16 rows] += Bg^T[128 x 8] * Atile^T[8 x 16]      (tcgen05.mma kind::tf32)
// with the 8 gathered rows of B as the MN-major operand (128-byte swizzle, 32-byte base) and the
// stored 16x8 tile as the K-major SWIZZLE_32B operand, accumulators in tensor memory.
//
// What differs is who does what, when:
//   * The grid is resident (blocks per SM x SMs) and every block walks work items
//     item -> (column block cb = item / G, tile group g = item % G) in item order b, b + grid, ...
//     Column blocks are the slow index, so the whole GPU works on the same 128*NSLAB columns of B at
//     about the same time: a row of B then competes for L2 with 512*NSLAB bytes instead of 4N, which is
//     what cuts the re-fetching of rows on power-law matrices (NSLAB = 1 or 2), while matrices whose
//     gathers already hit in L2 take the whole width at once (NSLAB = 4 at N = 512: tile values and
//     column ids are read once).  Odd column blocks walk the groups backwards, so the tile values
//     that are still in L2 at the end of one sweep are the first ones the next sweep wants.
//   * A pipeline step is always 4 units of 8 rows x 128 columns (16 KB of gathered rows): the NSLAB
//     slabs of KT = 4 / NSLAB consecutive tiles.  Steps run through the tiles of a group without
//     regard to window boundaries; only the MMA issuer and the epilogue know about windows.
//   * The block lives for the whole launch: barriers, tensor memory and the pipeline are set up
//     once, not once per group, and groups can be as long as the planner likes.
//   * Column ids are not staged in shared memory: a copy warp loads the ids of a step with one
//     coalesced load and hands them out with shuffles.
//   * Any N % 4 == 0: units are filled only where the column exists and the epilogue stores only
//     such columns (tensor-memory lanes of missing columns hold garbage that is never read).
//
// Roles (352 threads): warps 0-3 epilogue (tensor-memory lanes 32w..32w+31 = columns of a slab),
// warp 4 issues the MMAs (one lane), warps 5-8 copy, warps 9-10 hand over.  A copy warp owns every
// fourth step WHOLE: it waits for the slot, gathers the step's 16 KB with cp.async (lane -> (row,
// 16-byte chunk), so every quarter-warp reads one contiguous 128-byte line of B and writes one
// bank-conflict-free row of the swizzled operand), copies the tile operand(s) or what they are rebuilt
// from, and lets the copies themselves arrive on full[s] (cp.async.mbarrier.arrive.noinc): it never waits
// for data.  The hand-over warp that owns ring stage s waits on full[s], brings the tile operand into its
// final form (SR-BCRS: round the values to TF32 in place; ME-TCF: scatter the COO run into a zeroed tile;
// MCO: expand mask + packed values), issues the fence.proxy.async that cp.async data needs before the
// tensor core may read it, and signals ready[s] -- as soon as the step has landed, not when its copy warp
// comes round again (which measured 3-6 % slower at N = 512, 13-17 % at N <= 128, and twice as slow for the
// encodings whose hand-over is a few hundred cycles of dependent shared-memory work).  Compared with
// splitting every step over all copy warps, one warp per step costs a third of the instructions (the
// per-step bookkeeping is paid once, not four times), and the look-ahead of the column ids comes for
// free: a warp loads the ids of its next step while it works on the current one.  Rings: full[s]
// (copies -> hand-over warps), ready[s] (hand-over -> MMA), empty[s] (tcgen05.commit -> copy warps),
// acc_full / acc_empty[NACC] (accumulator buffers of 16*NSLAB tensor-memory columns, so the epilogue of a
// window overlaps the MMAs of the next ones).
//
// Every wait is bounded (about a second of SM clock).  On expiry the block raises its abort flag and
// the plan's device status word; every role leaves its loops, the producers wait for their copies,
// the MMA lane commits to a drain barrier and waits (bounded) until the tensor core has finished
// with shared and tensor memory, and only then is tensor memory freed.
#include "spmm_common.cuh"
#include "umma_ptx.cuh"

namespace mask {

constexpr int kSweepThreads = 352;   // 4 epilogue warps, the MMA warp, 4 copy warps, 2 hand-over warps

template <int NSLAB, int FMT>
struct SweepLayout {
    static constexpr int KT = 4 / NSLAB;                            // tiles per step
    static constexpr int S = FMT == kFmtSrbcrs ? 6 : 5;             // ring stages
    static constexpr int kStageB = 4 * 4096;                        // gathered rows of one step
    static constexpr int kStageA = KT * 512;                        // tile operand(s) of one step
    // staging per tile: ME-TCF 32 idx + 32 val of the run, then [begin, end); MCO 16 B of mask, up to
    // 128 values, then [begin, end) of the values
    static constexpr int kCooStride = FMT == kFmtMco ? 544 : (FMT == kFmtMetcf ? 272 : 0);
    static constexpr int kRunAt = FMT == kFmtMco ? 528 : 256;       // where [begin, end) sits in a tile's staging
    static constexpr int kNacc = NSLAB == 4 ? 4 : 8;                // accumulator buffers
    static constexpr int kAccCols = 16 * NSLAB;
    static constexpr int kTmemCols = kNacc * kAccCols;              // 256, 256, 128: two blocks fit an SM's 512
    static constexpr int kB = 0;
    static constexpr int kA = S * kStageB;
    static constexpr int kCoo = kA + S * kStageA;
    static constexpr int kBars = kCoo + ((S * KT * kCooStride + 15) & ~15);   // empty[S], ready[S], acc_full[NACC], acc_empty[NACC], drain
    static constexpr int kNumBars = 3 * S + 2 * kNacc + 1;   // empty, ready, full, acc_full, acc_empty, drain
    static constexpr int kTmemSlot = kBars + kNumBars * 8;
    static constexpr int kAbort = kTmemSlot + 8;
    static constexpr int kBytes = kAbort + 8;
    static constexpr int kDynamicBytes = kBytes + 1024;             // room to align the base to 1024 B
    static_assert(kTmemCols == 128 || kTmemCols == 256, "tensor-memory allocations are powers of two");
};

// A wait that only the clock bounds: used once, at teardown, when the abort flag may already be up.
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity) {
    const long long start = clock64();
    while (!mbar_test(bar, parity)) {
        if (clock64() - start > kUmmaWaitCycles) return false;
    }
    return true;
}

template <int NSLAB, int FMT>
__global__ void __launch_bounds__(kSweepThreads, 2) spmm_sweep_kernel(const SpmmArgs p, int32_t* status) {
    constexpr bool METCF = FMT == kFmtMetcf, MCO = FMT == kFmtMco, SRB = !METCF && !MCO;
    using L = SweepLayout<NSLAB, FMT>;
    constexpr int KT = L::KT, S = L::S, NACC = L::kNacc, kAccCols = L::kAccCols;
    extern __shared__ unsigned char sweep_smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(sweep_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                   // swizzle patterns are functions of the address bits
    unsigned char* gbase = sweep_smem_raw + (base - raw);
    const uint32_t bars = base + L::kBars;
    auto empty_bar = [&](int s) { return bars + 8u * s; };
    auto ready_bar = [&](int s) { return bars + 8u * (S + s); };
    auto full_bar = [&](int s) { return bars + 8u * (2 * S + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (3 * S + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (3 * S + NACC + b); };
    const uint32_t drain_bar = bars + 8u * (3 * S + 2 * NACC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + L::kAbort);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::kTmemSlot);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.n_groups;
    const int n_items = p.n_col_blocks * G;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S; s++) {
            mbar_init(empty_bar(s), 1);    // tcgen05.commit
            mbar_init(ready_bar(s), 1);    // lane 0 of the hand-over warp
            mbar_init(full_bar(s), 32);    // one deferred arrive per lane of the copying warp
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

    if (warp >= 5 && warp < 9) {
        // ------------------------------ copy warps (each owns every fourth step) -----------------------
        const int pw = warp - 5;
        const int lr = lane >> 3, lc = lane & 7; // row (and row + 4), 16-byte chunk
        const uint32_t off0 = (uint32_t)(lr * 128 + ((lc ^ (2 * lr)) * 16));   // 32-byte chunks swizzled by row % 4
        const uint32_t ldb_bytes = (uint32_t)(p.ldb * 4);
        const int idl = lane & (8 * KT - 1);     // which of a step's 8*KT ids this lane loads
        uint32_t gstep = 0;                      // steps of the items before the current one
        bool ok = true;

        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int cb = item_cb(item);
            const int g = item_group(item, cb);
            const int t0 = p.group_tile[g], t1 = p.group_tile[g + 1];
            const int n_steps = (t1 - t0 + KT - 1) / KT;
            const int cols_left = p.N - cb * (128 * NSLAB) - 4 * lc;    // > 32 j: this thread's chunk of 32-column atom j exists
            const bool whole = p.N - cb * (128 * NSLAB) >= 128 * NSLAB; // every column of the block exists
            const char* Bcol = reinterpret_cast<const char*>(p.B + cb * (128 * NSLAB) + 4 * lc);
            auto load_ids = [&](int j) -> int {
                const int64_t at = ((int64_t)t0 + (int64_t)j * KT) * kTileCols + idl;
                return (j < n_steps && at < (int64_t)t1 * kTileCols) ? __ldg(p.val_sidx + at) : 0;
            };
            // ME-TCF / MCO: [begin, end) of the value run of tile (step j, lane), loaded ahead like the ids
            auto load_run = [&](int j) -> int2 {
                int2 r = make_int2(0, 0);
                if (!SRB) {
                    const int64_t tile = (int64_t)t0 + (int64_t)j * KT + lane;
                    if (j < n_steps && lane < KT && tile < t1) {
                        if (METCF) r = __ldg(reinterpret_cast<const int2*>(p.coo_off) + tile);
                        else r = make_int2(__ldg(p.coo_off + tile), __ldg(p.coo_off + tile + 1));
                    }
                }
                return r;
            };
            const int j0 = (int)((pw - gstep) & 3u);   // this warp's first step of the item
            int q = load_ids(j0);
            int2 rq = load_run(j0);
            for (int j = j0; j < n_steps; j += 4) {
                const int tb = t0 + j * KT;
                const int cnt = min(KT, t1 - tb);
                const uint32_t gi = gstep + (uint32_t)j;
                const int s = (int)(gi % S);
                const uint32_t round = gi / S;
                int id0[KT], id1[KT];
#pragma unroll
                for (int u = 0; u < KT; u++) {
                    id0[u] = __shfl_sync(0xffffffffu, q, u * kTileCols + lr);
                    id1[u] = __shfl_sync(0xffffffffu, q, u * kTileCols + lr + 4);
                }
                int2 run[KT];
                if (!SRB) {
#pragma unroll
                    for (int u = 0; u < KT; u++) run[u] = make_int2(__shfl_sync(0xffffffffu, rq.x, u), __shfl_sync(0xffffffffu, rq.y, u));
                }
                q = load_ids(j + 4);        // the ids of this warp's next step travel while it works on this one
                rq = load_run(j + 4);
                // the verdict of a wait is made warp-uniform: every lane takes part in the shuffles above
                if (round > 0 && !__all_sync(0xffffffffu, mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag))) { ok = false; break; }
                const uint32_t dst = base + L::kB + s * L::kStageB + off0;
#pragma unroll
                for (int u = 0; u < KT; u++) {
                    if (u < cnt) {
                        const char* r0 = Bcol + (uint64_t)(uint32_t)id0[u] * ldb_bytes;
                        const char* r1 = Bcol + (uint64_t)(uint32_t)id1[u] * ldb_bytes;
                        if (whole) {
#pragma unroll
                            for (int a4 = 0; a4 < 4 * NSLAB; a4++) {   // 32-column atom a4 of the block: unit a4 / 4, atom a4 % 4
                                cp16(dst + u * NSLAB * 4096 + a4 * 1024, r0 + a4 * 128);
                                cp16(dst + u * NSLAB * 4096 + a4 * 1024 + 512, r1 + a4 * 128);
                            }
                        } else {
#pragma unroll
                            for (int a4 = 0; a4 < 4 * NSLAB; a4++) {
                                if (cols_left > 32 * a4) {
                                    cp16(dst + u * NSLAB * 4096 + a4 * 1024, r0 + a4 * 128);
                                    cp16(dst + u * NSLAB * 4096 + a4 * 1024 + 512, r1 + a4 * 128);
                                }
                            }
                        }
                        // the tile operand, or what it is rebuilt from
                        const int64_t tile = (int64_t)tb + u;
                        if (METCF) {
                            // [begin, end) of the run, then its first 32 entries (runs start on multiples of 8
                            // entries and are padded to 8)
                            const uint32_t st = base + L::kCoo + (s * KT + u) * L::kCooStride;
                            if (lane == 16)
                                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(st + L::kRunAt), "l"(p.coo_off + 2 * tile) : "memory");
                            const int chunk = lane & 7;   // 4 entries
                            if (lane < 16 && run[u].x + 4 * chunk < ((run[u].y + 7) & ~7)) {
                                const void* src = lane < 8 ? static_cast<const void*>(p.coo_idx + run[u].x + 4 * chunk)
                                                           : static_cast<const void*>(p.coo_val + run[u].x + 4 * chunk);
                                cp16(st + lane * 16, src);
                            }
                        } else if (MCO) {
                            const uint32_t st = base + L::kCoo + (s * KT + u) * L::kCooStride;
                            if (lane == 0) cp16(st, p.mco_mask + 2 * tile);
                            if (lane < 2)
                                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(st + L::kRunAt + 4 * lane), "l"(p.coo_off + tile + lane) : "memory");
                            if (run[u].x + 4 * lane < run[u].y) cp16(st + 16 + lane * 16, p.coo_val + run[u].x + 4 * lane);   // runs are multiples of 4 values
                        } else {
                            cp16(base + L::kA + s * L::kStageA + u * 512 + lane * 16, p.val_blk + tile * kTileElems + lane * 4);
                        }
                    }
                }
                // arrives on full[s] once every copy this lane has issued so far has landed
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar(s)) : "memory");
            }
            gstep += (uint32_t)n_steps;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");   // nothing of this warp's is in flight when the block leaves
    } else if (warp >= 9) {
        // ------------------------------ hand-over warps (ring stages split between the two) ------------
        const int q = warp - 9;
        uint32_t gi = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int g = item_group(item, item_cb(item));
            const int t0 = p.group_tile[g], t1 = p.group_tile[g + 1];
            for (int tb = t0; tb < t1; tb += KT, gi++) {
                // by stage, not by step: a barrier must be waited on in every one of its phases by the same
                // waiter (with an odd ring a step-parity split would hand each warp every other phase of a
                // stage, and a parity wait cannot tell phase k from phase k + 2)
                const int s = (int)(gi % S);
                if ((s & 1) != q) continue;
                if (!__all_sync(0xffffffffu, mbar_wait(full_bar(s), (gi / S) & 1, abort_flag))) { ok = false; break; }
                const int cnt = min(KT, t1 - tb);
#pragma unroll
                for (int u = 0; u < KT; u++) {
                    if (u < cnt) {
                        unsigned char* aslot = gbase + L::kA + s * L::kStageA + u * 512;
                        const unsigned char* st = gbase + L::kCoo + (s * KT + u) * L::kCooStride;
                        if (METCF) {  // rebuild the 16x8 operand: zero, then tile[idx] = rna(value) over the run
                            uint32_t* tile = reinterpret_cast<uint32_t*>(aslot);
                            reinterpret_cast<uint4*>(tile)[lane] = make_uint4(0u, 0u, 0u, 0u);
                            __syncwarp();
                            const int2 run = *reinterpret_cast<const int2*>(st + L::kRunAt);
                            const int rcnt = run.y - run.x;
                            const int* sidx = reinterpret_cast<const int*>(st);
                            const uint32_t* sval = reinterpret_cast<const uint32_t*>(st + 128);
                            if (lane < rcnt) tile[sidx[lane]] = sval[lane] + 0x1000u;
                            for (int e = run.x + 32 + lane; e < run.y; e += 32)   // dense tiles: entries beyond the staged 32
                                tile[__ldg(p.coo_idx + e)] = __float_as_uint(__ldg(p.coo_val + e)) + 0x1000u;
                            __syncwarp();
                        } else if (MCO) {
                            const ulonglong2 m = *reinterpret_cast<const ulonglong2*>(st);
                            reinterpret_cast<uint4*>(aslot)[lane] = mco_expand(m.x, m.y, reinterpret_cast<const uint32_t*>(st + 16), lane);
                        } else {   // dense tile: round to TF32 (nearest, ties away) in place
                            uint4* at = reinterpret_cast<uint4*>(aslot) + lane;
                            uint4 v = *at;
                            v.x += 0x1000u; v.y += 0x1000u; v.z += 0x1000u; v.w += 0x1000u;
                            *at = v;
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(ready_bar(s));
            }
        }
    } else if (warp == 4) {
        // ------------------------------ MMA issuer (one lane) ------------------------------------------
        if (lane == 0) {
            // This one thread paces the block, so its path per tile is kept to a handful of instructions:
            // descriptors are stepped by adding to their low halves, fragment boundaries cost a compare.
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
                    if (!mbar_wait(ready_bar(s), round & 1, abort_flag)) { ok = false; break; }
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
            if (!mbar_wait_drain(drain_bar, 0)) *abort_flag = 1;
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
                bool colok[NSLAB];
#pragma unroll
                for (int sl = 0; sl < NSLAB; sl++) colok[sl] = col + 128 * sl < p.N;
                // destination 0 is C (or the partial-tile scratch); 1.. are the peers' copies of C, which
                // get the finished rows with plain stores over NVLink
                const int n_dst = slot < 0 ? 1 + p.n_peer_out : 1;
#pragma unroll 1
                for (int d = 0; d < n_dst; d++) {
                    float* cb_ptr = slot >= 0 ? p.scratch + (int64_t)slot * kWinRows * p.N : (d == 0 ? p.C : p.peer_out[d - 1]);
                    int row0 = w * kWinRows;
                    asm volatile("" : "+r"(row0));   // keeps the 16 row offsets from being hoisted out of this loop into registers
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int r = !SRB ? i : (i ^ (i >> 3));   // MMA-N index -> window row (SR-BCRS: rows 8..15 swapped pairwise)
                        if (r < rows_ok) {
                            const int64_t off = slot >= 0 ? (int64_t)r * p.N
                                                          : (int64_t)(p.row_map ? p.row_map[row0 + r] : row0 + r) * p.ldc;
#pragma unroll
                            for (int sl = 0; sl < NSLAB; sl++) {
                                if (colok[sl]) {
                                    cb_ptr[off + col + 128 * sl] = __uint_as_float(v[sl][i]);
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
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::kTmemCols) : "memory");
    }
    if (tid == 0 && *abort_flag) atomicExch(status, 1);
}

template <int NSLAB, int FMT>
static int launch_sweep_variant(const mask_plan* plan, SpmmArgs a, cudaStream_t st) {
    using L = SweepLayout<NSLAB, FMT>;
    static_assert(2 * (L::kDynamicBytes + 1024) <= 228 * 1024, "two blocks per SM");
    auto kern = spmm_sweep_kernel<NSLAB, FMT>;
    MASK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));   // per device
    MASK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    // Two blocks per SM by construction: shared memory (asserted above), registers (launch bounds) and
    // tensor memory (at most 256 of the SM's 512 columns per block) all fit twice.  The occupancy
    // calculator is not asked: it answered 1 here because it assumes the default carveout.
    constexpr int blocks_per_sm = 2;
    a.n_col_blocks = (a.N + 128 * NSLAB - 1) / (128 * NSLAB);
    const int64_t items = (int64_t)a.n_col_blocks * plan->G;
    if (items >= ((int64_t)1 << 31)) return fail(MASK_ERR_INVALID_ARGUMENT, "too many work items");
    const int64_t resident = (int64_t)blocks_per_sm * sm_count();
    const unsigned grid = (unsigned)(items < resident ? items : resident);
    kern<<<grid, kSweepThreads, L::kDynamicBytes, st>>>(a, plan->d_status);
    MASK_CUDA_TRY(cudaGetLastError());
    return MASK_OK;
}

template <int FMT>
static int launch_sweep_fmt(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st, int nslab) {
    if (nslab == 1) return launch_sweep_variant<1, FMT>(plan, a, st);
    if (nslab == 2) return launch_sweep_variant<2, FMT>(plan, a, st);
    return launch_sweep_variant<4, FMT>(plan, a, st);
}

// nslab: 128-column slabs per column block (1, 2 or 4); 0 = the widest that N fills.
int launch_spmm_sweep(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st, int nslab) {
    if (a.N % 4 != 0) return fail(MASK_ERR_INVALID_ARGUMENT, "N must be a multiple of 4");
    if (plan->d_group_tile == nullptr) return fail(MASK_ERR_INVALID_ARGUMENT, "plan has no group tile table");
    const int fills = a.N > 256 ? 4 : (a.N > 128 ? 2 : 1);   // slabs N can fill
    if (nslab != 1 && nslab != 2 && nslab != 4) nslab = fills;
    nslab = nslab < fills ? nslab : fills;
    SpmmArgs b = a;
    b.group_tile = plan->d_group_tile;
    b.n_groups = (int32_t)plan->G;
    b.n_frag = plan->F;
    if (a.mco_mask) return launch_sweep_fmt<kFmtMco>(plan, b, st, nslab);
    if (a.coo_off) return launch_sweep_fmt<kFmtMetcf>(plan, b, st, nslab);
    return launch_sweep_fmt<kFmtSrbcrs>(plan, b, st, nslab);
}

}  // namespace mask
