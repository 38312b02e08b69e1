// SR-BCRS 16x8 SpMM on the 5th-generation tensor cores: tcgen05.mma (TF32) with accumulators in
// tensor memory, operands staged in shared memory by warp-specialised producers.
//
// Mapping.  A 16-row window is far too short for the MMA's M (64/128), so the product is issued
// TRANSPOSED: for every tile t of window w and every 128-column slab of B,
//
//     D^T[128 columns x 16 rows] += Bg^T[128 x 8] * Atile^T[8 x 16]
//
// MMA-M = 128 output columns, MMA-N = 16 window rows, MMA-K = 8 condensed columns: no padding
// beyond the format's own 16x8 tile.  Operands:
//   * MMA "A" = the 8 gathered rows of B, which are contiguous along the MMA-M direction: an
//     MN-major operand.  For 32-bit element types the only MN-major shared-memory layout the
//     tensor core accepts is the 128-byte swizzle with a 32-byte base: atoms of 32 columns x 4
//     rows (4 x 128 bytes), the 32-byte chunk q of row r stored at chunk q ^ (r % 4); the two
//     4-row halves of a tile 512 bytes apart (stride byte offset), 32-column atoms 1024 bytes
//     apart (leading byte offset).  A descriptor with the plain 128-byte swizzle is accepted but
//     multiplies zeros (found with a one-instruction known-answer test).  Producer warps fill the
//     layout with cp.async using lane -> (row, 16-byte chunk), so every quarter-warp reads one
//     contiguous 128-byte line of B and writes one full, bank-conflict-free row.
//   * MMA "B" = the stored tile itself.  SR-BCRS stores element (r,c) at Swizzle<2,2,3>(8r+c) of
//     a row-major 16x8 float tile; in bytes that is the canonical K-major SWIZZLE_32B layout
//     (row pitch 32 B, 8-row groups 256 B apart) except that rows 8..15 are swapped pairwise.
//     So the 512-byte tile is copied verbatim and used as the operand; MMA-N index n then stands
//     for window row n ^ (n >> 3), which the epilogue undoes when it stores.
// Operand precision: the tensor core truncates FP32 to TF32.  The tile values are rounded to
// nearest (ties away) in place before use, like the reference kernel's cvt.rna; the gathered B
// values cannot be touched on their way from global to shared memory and are truncated.  Worst
// case per product 2^-10 + 2^-11 = 1.46e-3 relative, inside the 2e-3 contract.
//
// The same kernel serves the three tile encodings (template parameter FMT): SR-BCRS copies the
// stored tile verbatim; ME-TCF and MCO rebuild it in the preparation warps from the tile's COO run
// or from its bitmap and compact values (both use Swizzle<1,2,3>, which is the K-major SWIZZLE_32B
// operand layout itself, so their MMA-N index is the window row).
//
// Roles (352 threads): warps 0-3 epilogue (tensor-memory lanes 32w..32w+31 = columns of a slab),
// warp 4 issues the MMAs (one elected lane), warps 5-6 prepare (round the tile values of
// alternate tiles and make the copied data visible to the tensor core's asynchronous proxy),
// warps 7-10 produce.  cp.async writes through the generic proxy, so a fence.proxy.async has to
// sit between a stage's arrival and its MMAs; doing that (and the rounding) inside the issuing
// warp serialised ~15 % of the kernel's time into one warp, hence the separate, two-way
// interleaved preparation stage.  Rings: full[s] (producers -> prepare, completed by
// cp.async.mbarrier.arrive of 128 threads), ready[s] (prepare -> MMA), empty[s] (tcgen05.commit ->
// producers), acc_full/acc_empty[2] (double-buffered accumulators, 64 tensor-memory columns each,
// so the epilogue of one window overlaps the MMAs of the next).
//
// Every wait is bounded (about a second of SM clock): on expiry the block raises a shared abort
// flag and a device status word, drains its copies, frees its tensor memory and returns.
#include "spmm_common.cuh"
#include "umma_ptx.cuh"

namespace mask {

constexpr int kUmmaThreads = 352;
constexpr int kUmmaABytes = 512;
constexpr int kUmmaIdsBytes = kUmmaMaxGroupTiles * kTileCols * 4;

// A ring stage holds U "units" of 8 gathered rows x 128 columns (4 KB each):
//   KB == 1: the NSLAB column slabs of ONE tile (block = 128*NSLAB columns wide),
//   KB  > 1: the same 128-column slab of KB CONSECUTIVE tiles of one window (block = 128 columns
//            wide; blockIdx.y walks the slabs, and because blocks are dispatched x-fastest the whole
//            matrix is swept once per slab, so rows of B compete for L2 with 512 bytes each instead
//            of 4N bytes -- the lever against re-reading B on power-law matrices).
// Either way a stage is one pipeline step: one full/ready/empty round trip and U MMAs.
template <int NSLAB, int KB, int S, int FMT = kFmtSrbcrs>
struct UmmaLayout {
    // staging per stage and tile: ME-TCF 32 idx + 32 val of the run; MCO 16 B of mask + up to 128 values
    static constexpr int kCooStride = FMT == kFmtMco ? 528 : 256;
    static constexpr int kUnits = NSLAB * KB;
    static constexpr int kTilesPerStep = KB;
    static constexpr int kBBytes = kUnits * 4096;                 // gathered rows of one step
    static constexpr int kABytes = KB * kUmmaABytes;              // tile operand(s) of one step
    static constexpr int kTmemCols = 32 * NSLAB;                  // two accumulator buffers of 16*NSLAB columns
    static constexpr int kB = 0;
    static constexpr int kA = S * kBBytes;
    static constexpr int kIds = kA + S * kABytes;
    static constexpr int kRuns = kIds + kUmmaIdsBytes;            // ME-TCF: [begin, end) of every tile's COO run
    // ME-TCF: [begin, end) per tile; MCO: val_mco_off of the group's tiles plus the closing entry
    static constexpr int kRunsBytes = FMT == kFmtMco ? ((kUmmaMaxGroupTiles + 1) * 4 + 15) & ~15 : kUmmaMaxGroupTiles * 8;
    static constexpr int kCoo = kRuns + kRunsBytes;
    static constexpr int kBars = kCoo + ((S * KB * kCooStride + 15) & ~15);   // full[S], empty[S], ready[S], acc_full[2], acc_empty[2]
    static constexpr int kTmemSlot = kBars + (3 * S + 4) * 8;
    static constexpr int kAbort = kTmemSlot + 8;
    static constexpr int kBytes = kAbort + 8;
    static constexpr int kDynamicBytes = kBytes + 1024;           // room to align the base to 1024 B
};

// The same copy with compile-time offsets folded into the instruction's address immediates.
template <int DST_IMM, int SRC_IMM>
__device__ __forceinline__ void cp16_imm(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %3], 16;" ::"r"(dst), "l"(src), "n"(DST_IMM), "n"(SRC_IMM) : "memory");
}
// Rows r0 / r1 (= row + 4) of one unit group: the same 16-byte chunk of every 128-column slab.
template <int NSLAB, int U, int SL = 0>
struct CopySlabs {
    static __device__ __forceinline__ void run(uint32_t dst0, const char* r0, const char* r1) {
        cp16_imm<(U * NSLAB + SL) * 4096, SL * 512>(dst0, r0);
        cp16_imm<(U * NSLAB + SL) * 4096 + 512, SL * 512>(dst0, r1);
        if constexpr (SL + 1 < NSLAB) CopySlabs<NSLAB, U, SL + 1>::run(dst0, r0, r1);
    }
};
template <int NSLAB, int KB, int U = 0>
struct CopyUnits {
    static __device__ __forceinline__ void run(uint32_t dst0, const int* ids, int cnt, int lr, const char* Bcol, uint32_t ldb_bytes) {
        if (U < cnt) {
            const char* r0 = Bcol + (uint64_t)(uint32_t)ids[U * kTileCols + lr] * ldb_bytes;
            const char* r1 = Bcol + (uint64_t)(uint32_t)ids[U * kTileCols + lr + 4] * ldb_bytes;
            CopySlabs<NSLAB, U>::run(dst0, r0, r1);
        }
        if constexpr (U + 1 < KB) CopyUnits<NSLAB, KB, U + 1>::run(dst0, ids, cnt, lr, Bcol, ldb_bytes);
    }
};

// METCF: the tile operand is rebuilt per tile from its COO run (examples/src_fp32/dtc/testbed/
// kernel.inc:822-840 does the same in its shared-memory restore step).  ME-TCF's index
// Swizzle<1,2,3>(8r+c) is exactly the K-major SWIZZLE_32B operand layout, so tile[idx] = value
// yields the operand directly, rows unpermuted.
// MCO: the operand is expanded from the tile's 128-bit mask and its compact values (bit and operand
// position are both Swizzle<1,2,3>(8r+c)): no zero-fill, no scatter, one 16-byte store per lane.
template <int NSLAB, int KB, int S, int MIN_BLOCKS, int FMT>
__global__ void __launch_bounds__(kUmmaThreads, MIN_BLOCKS) spmm_umma_kernel(const SpmmArgs p, int32_t* status) {
    static_assert(KB == 1 || NSLAB == 1, "tiles are batched along K only in single-slab blocks");
    constexpr bool METCF = FMT == kFmtMetcf, MCO = FMT == kFmtMco;
    using L = UmmaLayout<NSLAB, KB, S, FMT>;
    constexpr int kAccCols = 16 * NSLAB;                          // accumulator columns per buffer
    extern __shared__ unsigned char umma_smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(umma_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;            // swizzle patterns are functions of the address bits
    unsigned char* gbase = umma_smem_raw + (base - raw);
    const uint32_t bars = base + L::kBars;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };
    auto ready_bar = [&](int s) { return bars + 8u * (2 * S + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (3 * S + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (3 * S + 2 + b); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + L::kAbort);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L::kTmemSlot);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int f0 = p.group_off[blockIdx.x], f_end = p.group_off[blockIdx.x + 1];
    const int t0 = p.frag_off[f0];
    const int n_tiles = p.frag_off[f_end] - t0;   // <= kUmmaMaxGroupTiles (checked by the launcher)
    const int col0 = blockIdx.y * (NSLAB * 128);

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 128);   // one deferred arrive per producer thread
            mbar_init(empty_bar(s), 1);    // tcgen05.commit
            mbar_init(ready_bar(s), 1);    // lane 0 of the preparing warp
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(accf_bar(b), 1);     // tcgen05.commit
            mbar_init(acce_bar(b), 4);     // lane 0 of every epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(base + L::kTmemSlot),
                     "r"(L::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp >= 7) {  // gathered-row ids of the whole group, once
        const int pt = tid - 224;
        const int chunks = n_tiles * 2;
        for (int c = pt; c < chunks; c += 128) cp16(base + L::kIds + c * 16, p.val_sidx + (int64_t)t0 * kTileCols + c * 4);
        if (METCF) {  // run offsets coo_off[2t], coo_off[2t+1]: 8-byte aligned pairs
            for (int c = pt; c < n_tiles; c += 128)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(base + L::kRuns + c * 8), "l"(p.coo_off + 2 * (int64_t)(t0 + c)) : "memory");
        }
        if (MCO) {    // value offsets val_mco_off[t0 .. t0 + n_tiles]
            for (int c = pt; c <= n_tiles; c += 128)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(base + L::kRuns + c * 4), "l"(p.coo_off + (int64_t)(t0 + c)) : "memory");
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // Every role walks the same sequence of steps: for each fragment with n > 0 tiles, ceil(n/KB)
    // steps of up to KB tiles (a step never spans two fragments: they accumulate separately).
    if (warp >= 7) {
        // ------------------------------ producers ------------------------------------------------
        const int pw = warp - 7;                 // this warp copies 32-column atom pw of every unit
        const int lr = lane >> 3, lc = lane & 7; // row (and row + 4), 16-byte chunk
        const uint32_t off0 = (uint32_t)(pw * 1024 + lr * 128 + ((lc ^ (2 * lr)) * 16));   // 32-byte chunks swizzled by row % 4
        const char* Bcol = reinterpret_cast<const char*>(p.B + col0 + 32 * pw + 4 * lc);
        const uint32_t ldb_bytes = (uint32_t)(p.ldb * 4);
        const int* ids = reinterpret_cast<const int*>(gbase + L::kIds);
        int s = 0, rel = 0;
        uint32_t round = 0;
        bool ok = true;
        for (int f = f0; f < f_end && ok; f++) {
            const int n = p.frag_off[f + 1] - p.frag_off[f];
            for (int i = 0; i < n; i += KB) {
                const int cnt = min(KB, n - i);
                if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, abort_flag)) { ok = false; break; }
                // off1 = off0 + 512: both rows of a thread go through one base register plus immediates
                CopyUnits<NSLAB, KB>::run(base + L::kB + s * L::kBBytes + off0, ids + rel * kTileCols, cnt, lr, Bcol, ldb_bytes);
                // tile operand(s): warp u copies the one of tile u of the step
                if (pw < cnt) {
                    const int tile = rel + pw;
                    if (METCF) {
                        // first 32 entries of the run (runs start on multiples of 8 entries and are padded to 8)
                        const int2 run = reinterpret_cast<const int2*>(gbase + L::kRuns)[tile];
                        const int chunk = lane & 7;   // 4 entries
                        if (lane < 16 && run.x + 4 * chunk < ((run.y + 7) & ~7)) {
                            const void* src = lane < 8 ? static_cast<const void*>(p.coo_idx + run.x + 4 * chunk)
                                                       : static_cast<const void*>(p.coo_val + run.x + 4 * chunk);
                            cp16(base + L::kCoo + (s * KB + pw) * 256 + lane * 16, src);
                        }
                    } else if (MCO) {
                        const int* offs = reinterpret_cast<const int*>(gbase + L::kRuns);
                        const int o0 = offs[tile], o1 = offs[tile + 1];
                        const uint32_t st = base + L::kCoo + (s * KB + pw) * L::kCooStride;
                        if (lane == 0) cp16(st, p.mco_mask + 2 * (int64_t)(t0 + tile));
                        if (o0 + 4 * lane < o1) cp16(st + 16 + lane * 16, p.coo_val + o0 + 4 * lane);   // runs are multiples of 4 values
                    } else {
                        cp16(base + L::kA + s * L::kABytes + pw * kUmmaABytes + lane * 16,
                             p.val_blk + (int64_t)(t0 + tile) * kTileElems + lane * 4);
                    }
                }
                // arrives on full[s] once every copy this thread has issued so far has landed
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar(s)) : "memory");
                rel += cnt;
                if (++s == S) { s = 0; round++; }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp >= 5) {
        // ------------------------------ prepare (two warps, alternate steps) -------------------------
        const int q = warp - 5;
        int s = 0, rel = 0, step = 0;
        uint32_t round = 0;
        bool ok = true;
        for (int f = f0; f < f_end && ok; f++) {
            const int n = p.frag_off[f + 1] - p.frag_off[f];
            for (int i = 0; i < n; i += KB, step++) {
                const int cnt = min(KB, n - i);
                if ((step & 1) == q) {
                    if (!mbar_wait(full_bar(s), round & 1, abort_flag)) { ok = false; break; }
                    for (int u = 0; u < cnt; u++) {
                        unsigned char* aslot = gbase + L::kA + s * L::kABytes + u * kUmmaABytes;
                        if (METCF) {  // rebuild the 16x8 operand: zero, then tile[idx] = rna(value) over the run
                            uint32_t* tile = reinterpret_cast<uint32_t*>(aslot);
                            reinterpret_cast<uint4*>(tile)[lane] = make_uint4(0u, 0u, 0u, 0u);
                            __syncwarp();
                            const int2 run = reinterpret_cast<const int2*>(gbase + L::kRuns)[rel + u];
                            const int rcnt = run.y - run.x;
                            const int* sidx = reinterpret_cast<const int*>(gbase + L::kCoo + (s * KB + u) * 256);
                            const uint32_t* sval = reinterpret_cast<const uint32_t*>(gbase + L::kCoo + (s * KB + u) * 256 + 128);
                            if (lane < rcnt) tile[sidx[lane]] = sval[lane] + 0x1000u;
                            for (int e = run.x + 32 + lane; e < run.y; e += 32)   // dense tiles: entries beyond the staged 32
                                tile[__ldg(p.coo_idx + e)] = __float_as_uint(__ldg(p.coo_val + e)) + 0x1000u;
                            __syncwarp();
                        } else if (MCO) {
                            const unsigned char* st = gbase + L::kCoo + (s * KB + u) * L::kCooStride;
                            const ulonglong2 m = *reinterpret_cast<const ulonglong2*>(st);
                            reinterpret_cast<uint4*>(aslot)[lane] = mco_expand(m.x, m.y, reinterpret_cast<const uint32_t*>(st + 16), lane);
                        } else if (!(p.hints & 4)) {  // round the tile values to TF32 (nearest, ties away) in place
                            uint4* at = reinterpret_cast<uint4*>(aslot) + lane;
                            uint4 v = *at;
                            v.x += 0x1000u; v.y += 0x1000u; v.z += 0x1000u; v.w += 0x1000u;
                            *at = v;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ready_bar(s));
                }
                rel += cnt;
                if (++s == S) { s = 0; round++; }
            }
        }
    } else if (warp == 4) {
        // ------------------------------ MMA issuer (one lane) ------------------------------------------
        if (lane == 0) {
            int s = 0;
            uint32_t round = 0, uses0 = 0, uses1 = 0;
            int buf = 0;
            bool ok = true;
            for (int f = f0; f < f_end && ok; f++) {
                const int n = p.frag_off[f + 1] - p.frag_off[f];
                if (n == 0) continue;
                const uint32_t uses = buf ? uses1 : uses0;
                if (uses > 0 && !mbar_wait(acce_bar(buf), (uses - 1) & 1, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int i = 0; i < n; i += KB) {
                    const int cnt = min(KB, n - i);
                    if (!mbar_wait(ready_bar(s), round & 1, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int u = 0; u < KB; u++) {
                        if (u < cnt) {
                            const uint64_t bdesc = umma_smem_desc(base + L::kA + s * L::kABytes + u * kUmmaABytes, 1, 16, kSwizzle32B);
#pragma unroll
                            for (int sl = 0; sl < NSLAB; sl++) {
                                const uint64_t adesc = umma_smem_desc(base + L::kB + s * L::kBBytes + (u * NSLAB + sl) * 4096, 64, 32, kSwizzle128B32B);
                                umma_tf32(tmem_base + buf * kAccCols + sl * 16, adesc, bdesc, (i + u) > 0 ? 1u : 0u);
                            }
                        }
                    }
                    umma_commit(empty_bar(s));   // the slot is free once these MMAs have read it
                    if (++s == S) { s = 0; round++; }
                }
                if (!ok) break;
                umma_commit(accf_bar(buf));      // accumulators of this fragment complete
                if (buf) uses1++; else uses0++;
                buf ^= 1;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue -------------------------------------------------
        uint32_t uses[2] = {0, 0};
        int buf = 0;
        const int col = col0 + 32 * warp + lane;   // + 128 * slab
        for (int f = f0; f < f_end; f++) {
            const int n = p.frag_off[f + 1] - p.frag_off[f];
            const int w = p.frag_win[f];
            const int slot = p.frag_slot[f];
            const int rows_ok = slot < 0 ? p.M - w * kWinRows : kWinRows;
            const bool relu = p.relu && slot < 0;
            uint32_t v[NSLAB][16];
            if (n == 0) {
#pragma unroll
                for (int sl = 0; sl < NSLAB; sl++)
#pragma unroll
                    for (int i = 0; i < 16; i++) v[sl][i] = 0u;
            } else {
                if (!mbar_wait(accf_bar(buf), uses[buf] & 1, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * warp) << 16) + buf * kAccCols;
#pragma unroll
                for (int sl = 0; sl < NSLAB; sl++) tmem_ld16(taddr + sl * 16, v[sl]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(acce_bar(buf));   // the MMA warp may reuse this buffer
                uses[buf]++;
                buf ^= 1;
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
#pragma unroll 1
            for (int d = 0; d < n_dst; d++) {
                float* cb = slot >= 0 ? p.scratch + (int64_t)slot * kWinRows * p.N : (d == 0 ? p.C : p.peer_out[d - 1]);
                int row0 = w * kWinRows;
                asm volatile("" : "+r"(row0));   // keeps the 16 row offsets from being hoisted out of this loop into registers
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int r = FMT != kFmtSrbcrs ? i : (i ^ (i >> 3));   // MMA-N index -> window row (SR-BCRS: rows 8..15 swapped pairwise)
                    if (r < rows_ok) {
                        const int64_t off = slot >= 0 ? (int64_t)r * p.N
                                                      : (int64_t)(p.row_map ? p.row_map[row0 + r] : row0 + r) * p.ldc;
#pragma unroll
                        for (int sl = 0; sl < NSLAB; sl++) cb[off + col + 128 * sl] = __uint_as_float(v[sl][i]);
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

template <int NSLAB, int KB, int S, int MIN_BLOCKS>
static int launch_umma_variant(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st) {
    const int fmt = a.mco_mask ? kFmtMco : (a.coo_off ? kFmtMetcf : kFmtSrbcrs);
    auto kern = fmt == kFmtMco ? spmm_umma_kernel<NSLAB, KB, S, MIN_BLOCKS, kFmtMco>
                               : (fmt == kFmtMetcf ? spmm_umma_kernel<NSLAB, KB, S, MIN_BLOCKS, kFmtMetcf>
                                                   : spmm_umma_kernel<NSLAB, KB, S, MIN_BLOCKS, kFmtSrbcrs>);
    const int smem = fmt == kFmtMco ? UmmaLayout<NSLAB, KB, S, kFmtMco>::kDynamicBytes : UmmaLayout<NSLAB, KB, S>::kDynamicBytes;
    static_assert(MIN_BLOCKS * (UmmaLayout<NSLAB, KB, S, kFmtMco>::kDynamicBytes + 1024) <= 228 * 1024, "shared memory per SM");
    MASK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid((unsigned)plan->G, (unsigned)(a.N / (NSLAB * 128)));
    if (grid.y > 65535) return fail(MASK_ERR_INVALID_ARGUMENT, "N too large");
    kern<<<grid, kUmmaThreads, smem, st>>>(a, plan->d_status);
    MASK_CUDA_TRY(cudaGetLastError());
    return MASK_OK;
}

// variant: 0 = by N (widest slab group that divides N: the tile values and ids are fetched once per
// block), 1 / 2 / 3 = 128-column slabs with 4 / 2 / 1 tiles per pipeline step (the matrix is swept
// once per slab), 4 = 256-column slabs
int launch_spmm_umma(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st, int variant) {
    if (a.N % 128 != 0) return fail(MASK_ERR_INVALID_ARGUMENT, "the tcgen05 kernel needs N % 128 == 0");
    if (plan->max_group_tiles > kUmmaMaxGroupTiles) return fail(MASK_ERR_INVALID_ARGUMENT, "plan groups too large for the tcgen05 kernel");
    if (variant == 1) return launch_umma_variant<1, 4, 5, 2>(plan, a, st);
    if (variant == 2) return launch_umma_variant<1, 2, 8, 2>(plan, a, st);
    if (variant == 3) return launch_umma_variant<1, 1, 8, 3>(plan, a, st);                     // 128-column slabs, one tile per step
    if (variant == 4 && a.N % 256 == 0) return launch_umma_variant<2, 1, 8, 2>(plan, a, st);   // 256-column slabs
    if (a.N % 512 == 0) return launch_umma_variant<4, 1, 6, 2>(plan, a, st);
    if (a.N % 256 == 0) return launch_umma_variant<2, 1, 8, 2>(plan, a, st);
    return launch_umma_variant<1, 1, 8, 3>(plan, a, st);
}

}  // namespace mask
