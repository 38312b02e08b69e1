// SR-BCRS 16x8 SpMM with a deep, warp-private shared-memory ring fed by cp.async.
//
// Why: the gather of B rows is bound by memory latency, not by bandwidth or math.  On B200 a
// DRAM miss costs well over a microsecond under load, so an SM needs on the order of 150-200 KB
// of loads in flight to keep HBM and L2 busy.  Registers cannot hold that (the register-pipelined
// kernel in spmm_mma.cu keeps about 1.5 tiles per warp in flight); shared memory can.
//
// Each warp owns S ring slots.  A slot holds one tile's worth of the warp's operands: for every
// 32-column group q the 8 gathered rows x 128 bytes, plus the 512-byte tile of A values.
//
// Copy mapping vs fragment mapping.  The load/store unit handles a 128-bit access one quarter-warp
// (8 lanes) at a time and spends one pass per distinct 128-byte line, so the copy is issued with
// lane l -> (row l/8, 16-byte chunk l%8): a quarter-warp reads one contiguous 128-byte line
// (4 passes per warp instruction; the fragment mapping of the register kernel needs 16).  The MMA
// side wants lane (g = l/4, k = l%4) to read chunk g of row k.  Chunk c of row r is therefore
// stored at position c ^ 2(r%4) of its row: both the asynchronous writes (fixed row, 8 chunks)
// and the fragment reads (rows 0..3, two chunks each) touch every bank exactly once.
//
// The gathered-row ids go through a second, twice as deep ring so that they have landed before
// the copies that need them as addresses are issued.  All synchronisation is
// cp.async.wait_group + __syncwarp: there is no block-wide barrier, and warps of a block drift
// freely.
//
// Per step t (one tile): wait for tile t's group, refill the slot freed by tile t-1 with tile
// t+S-1, fetch ids for tile t+2S-1, then run the 4*NQ MMAs of tile t from shared memory.
#include "spmm_common.cuh"

namespace mask {

// 16-byte asynchronous copy global -> shared, L2 only (.cg).  DST_IMM / SRC_IMM are folded into
// the instruction's address immediates, so per-group offsets cost no address arithmetic.
template <int DST_IMM, int SRC_IMM>
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %3], 16;\n" ::"r"(dst), "l"(src), "n"(DST_IMM), "n"(SRC_IMM)
                 : "memory");
}
// Same with zero fill: when !valid no source byte is read and the 16 destination bytes are zeroed.
template <int DST_IMM, int SRC_IMM>
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0 + %3], [%1 + %4], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes), "n"(DST_IMM),
                 "n"(SRC_IMM)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <int NQ, int S, int WPB = kWarpsPerBlock>
struct AsyncLayout {
    static constexpr int kBBytes = NQ * 1024;                   // per slot: NQ groups x 8 rows x 128 B
    static constexpr int kABytes = kTileElems * 4;              // per slot: the tile of A values
    static constexpr int kSlotBytes = kBBytes + kABytes;
    static constexpr int kIdxSlots = 2 * S;
    static constexpr int kIdxBytes = kIdxSlots * kTileCols * 4;  // per warp
    static constexpr int kWarpBytes = S * kSlotBytes + kIdxBytes;
    static constexpr int kBlockBytes = WPB * kWarpBytes;
};

// Copies of one tile's B rows, unrolled over the 32-column groups with immediate offsets.
template <int NQ, bool GUARD, int Q = 0>
struct CopyRows {
    static __device__ __forceinline__ void run(uint32_t dst, const float* r0, const float* r1, const bool (&qok)[NQ]) {
        if (GUARD) {
            cp_async16_zfill<Q * 1024, Q * 128>(dst, r0, qok[Q]);
            cp_async16_zfill<Q * 1024 + 512, Q * 128>(dst, r1, qok[Q]);
        } else {
            cp_async16<Q * 1024, Q * 128>(dst, r0);
            cp_async16<Q * 1024 + 512, Q * 128>(dst, r1);
        }
        if constexpr (Q + 1 < NQ) CopyRows<NQ, GUARD, Q + 1>::run(dst, r0, r1, qok);
    }
};

// WPB warps per block take adjacent column slabs of the same tiles.  blockIdx.y selects the
// group of WPB slabs; blocks are dispatched x-fastest, so with WPB = 1 the whole matrix is swept
// once per 32*NQ-column slab: the rows of B then compete for L2 with 32*NQ*4 bytes each instead of
// 4N bytes, which is what raises the hit rate on power-law matrices.
// GUARD = false requires N % (32*NQ*WPB) == 0 (every column group of every warp is full).
// COMP: three products per MMA (hi*hi and the two residual terms), see MASK_NUMERICS_TF32X3.
template <int NQ, int S, int MIN_BLOCKS, bool GUARD, int WPB = kWarpsPerBlock, bool COMP = false>
__global__ void __launch_bounds__(WPB * 32, MIN_BLOCKS) spmm_async_kernel(const SpmmArgs p) {
    using L = AsyncLayout<NQ, S, WPB>;
    extern __shared__ __align__(128) unsigned char smem[];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int k = lane & 3;
    const int col_base = (blockIdx.y * WPB + warp) * (32 * NQ);
    if (col_base >= p.N) return;

    int f = p.group_off[blockIdx.x];
    const int f_end = p.group_off[blockIdx.x + 1];
    if (f >= f_end) return;
    const int t0 = p.frag_off[f];
    const int n_tiles = p.frag_off[f_end] - t0;       // tiles of this block, indexed 0..n_tiles-1 below
    int f_tend = p.frag_off[f + 1] - t0;

    unsigned char* wbase = smem + warp * L::kWarpBytes;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(wbase);
    const uint32_t idx_s = ring_s + S * L::kSlotBytes;
    const unsigned char* idx_ring = wbase + S * L::kSlotBytes;

    const int ao0 = sw223(8 * g + k) * 4, ao1 = sw223(8 * (g + 8) + k) * 4;
    const int ao2 = sw223(8 * g + k + 4) * 4, ao3 = sw223(8 * (g + 8) + k + 4) * 4;

    // copy mapping: row lr (and lr+4), chunk lc of every 32-column group
    const int lr = lane >> 3, lc = lane & 7;
    bool qok[NQ];
#pragma unroll
    for (int q = 0; q < NQ; q++) qok[q] = (col_base + 32 * q + 4 * lc) < p.N;
    const char* Bcol = reinterpret_cast<const char*>(p.B + col_base + 4 * lc);
    const uint32_t ldb_bytes = (uint32_t)(p.ldb * 4);
    const uint32_t cp_off = (uint32_t)((lr * 8 + (lc ^ (2 * lr))) * 16);  // lr < 4, so lr % 4 == lr
    // fragment mapping: chunk g of rows k and k+4
    const int frag_off = (k * 8 + (g ^ (2 * k))) * 16;
    const float* a_src = p.val_blk + (int64_t)t0 * kTileElems + lane * 4;
    const int* i_src = p.val_sidx + (int64_t)t0 * kTileCols + (lane & 1) * 4;


    float acc[NQ][4][4];
#pragma unroll
    for (int q = 0; q < NQ; q++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[q][j][i] = 0.f;

    // gathered-row ids of tile tt -> id ring slot (byte offset islot); two 16-byte copies by lanes 0, 1
    auto issue_idx = [&](int tt, int islot) {
        if (tt < n_tiles && lane < 2) cp_async16<0, 0>(idx_s + islot + lane * 16, i_src + tt * kTileCols);
    };
    // operands of tile tt -> ring slot (byte offset slot); its ids (id ring byte offset islot) are visible
    auto issue_tile = [&](int tt, int slot, int islot) {
        if (tt < n_tiles) {
            const int* id = reinterpret_cast<const int*>(idx_ring + islot);
            const char* r0 = Bcol + (uint64_t)(uint32_t)id[lr] * ldb_bytes;
            const char* r1 = Bcol + (uint64_t)(uint32_t)id[lr + 4] * ldb_bytes;
            const uint32_t dst = ring_s + slot;
            CopyRows<NQ, GUARD>::run(dst + cp_off, reinterpret_cast<const float*>(r0), reinterpret_cast<const float*>(r1), qok);
            cp_async16<L::kBBytes, 0>(dst + lane * 16, a_src + tt * kTileElems);
        }
    };
    auto next = [](int x, int step, int wrap) { x += step; return x == wrap ? 0 : x; };

    // ---- prologue ----------------------------------------------------------------------------
    {
        int is = 0;
#pragma unroll 1
        for (int i = 0; i < 2 * S - 1; i++) { issue_idx(i, is); is += kTileCols * 4; }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    {
        int sl = 0, is = 0;
#pragma unroll 1
        for (int i = 0; i < S - 1; i++) {
            issue_tile(i, sl, is);
            cp_async_commit();
            sl += L::kSlotBytes;
            is += kTileCols * 4;
        }
    }

    // ---- main loop -----------------------------------------------------------------------------
    // byte offsets into the rings: slot of tile t (consume), of tile t+S-1 (refill), id slots of
    // tile t+S-1 (addresses for the refill) and of tile t+2S-1 (id prefetch)
    int t = 0;
    int c_slot = 0, r_slot = (S - 1) * L::kSlotBytes;
    int ri_slot = (S - 1) * kTileCols * 4, pi_slot = (2 * S - 1) * kTileCols * 4;
    while (true) {
        while (t == f_tend && f < f_end) {  // fragment finished (also: fragments without tiles)
            flush_fragment<NQ>(p, f, col_base, g, k, acc);
            f++;
            f_tend = (f < f_end) ? p.frag_off[f + 1] - t0 : -1;
        }
        if (f >= f_end) break;

        cp_async_wait<S - 2>();  // tile t has landed (this thread's copies) ...
        __syncwarp();            // ... and everybody's; also: all lanes are done with tile t-1's slot
        issue_tile(t + S - 1, r_slot, ri_slot);
        issue_idx(t + 2 * S - 1, pi_slot);
        cp_async_commit();

        const unsigned char* slot = wbase + c_slot;
        const unsigned char* at = slot + L::kBBytes;
        const float af[4] = {*reinterpret_cast<const float*>(at + ao0), *reinterpret_cast<const float*>(at + ao1),
                             *reinterpret_cast<const float*>(at + ao2), *reinterpret_cast<const float*>(at + ao3)};
        const unsigned char* bt = slot + frag_off;
        if constexpr (COMP) {
            uint32_t a[4], al[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = tf32_hi(af[i]); al[i] = tf32_lo(af[i], a[i]); }
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const float4 v0 = *reinterpret_cast<const float4*>(bt + q * 1024);
                const float4 v1 = *reinterpret_cast<const float4*>(bt + q * 1024 + 512);
                const float b0[4] = {v0.x, v0.y, v0.z, v0.w}, b1[4] = {v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t h0 = tf32_hi(b0[j]), h1 = tf32_hi(b1[j]);
                    mma_tf32(acc[q][j], al, h0, h1);                                       // small terms first
                    mma_tf32(acc[q][j], a, tf32_lo(b0[j], h0), tf32_lo(b1[j], h1));
                    mma_tf32(acc[q][j], a, h0, h1);
                }
            }
        } else {
            uint32_t a[4] = {rna_bits(af[0]), rna_bits(af[1]), rna_bits(af[2]), rna_bits(af[3])};
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const float4 v0 = *reinterpret_cast<const float4*>(bt + q * 1024);
                const float4 v1 = *reinterpret_cast<const float4*>(bt + q * 1024 + 512);
                mma_tf32(acc[q][0], a, rna_bits(v0.x), rna_bits(v1.x));
                mma_tf32(acc[q][1], a, rna_bits(v0.y), rna_bits(v1.y));
                mma_tf32(acc[q][2], a, rna_bits(v0.z), rna_bits(v1.z));
                mma_tf32(acc[q][3], a, rna_bits(v0.w), rna_bits(v1.w));
            }
        }
        t++;
        r_slot = c_slot;
        c_slot = next(c_slot, L::kSlotBytes, S * L::kSlotBytes);
        ri_slot = next(ri_slot, kTileCols * 4, L::kIdxBytes);
        pi_slot = next(pi_slot, kTileCols * 4, L::kIdxBytes);
    }
    cp_async_wait<0>();
}

template <int NQ, int S, int MIN_BLOCKS, int WPB = kWarpsPerBlock, bool COMP = false>
static int launch_variant(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st) {
    using L = AsyncLayout<NQ, S, WPB>;
    const int cols_per_block = 32 * NQ * WPB;
    const bool guard = (a.N % cols_per_block) != 0;
    auto kern = guard ? spmm_async_kernel<NQ, S, MIN_BLOCKS, true, WPB, COMP> : spmm_async_kernel<NQ, S, MIN_BLOCKS, false, WPB, COMP>;
    // opt in to more than 48 KB of dynamic shared memory (cheap; repeated per call so that it
    // holds for whichever device is current)
    MASK_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBlockBytes));
    dim3 grid((unsigned)plan->G, (unsigned)((a.N + cols_per_block - 1) / cols_per_block));
    if (grid.y > 65535) return fail(MASK_ERR_INVALID_ARGUMENT, "N too large");
    kern<<<grid, WPB * 32, L::kBlockBytes, st>>>(a);
    MASK_CUDA_TRY(cudaGetLastError());
    return MASK_OK;
}

int launch_spmm_async(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st, int nq, int stages) {
    if (nq != 1 && nq != 2 && nq != 4) nq = a.N > 256 ? 4 : (a.N > 128 ? 2 : 1);
    if (a.tf32x3) {   // compensated products: the default variant of each width
        if (nq == 4) return launch_variant<4, 4, 2, kWarpsPerBlock, true>(plan, a, st);
        if (nq == 2) return launch_variant<2, 4, 4, kWarpsPerBlock, true>(plan, a, st);
        return launch_variant<1, 8, 4, kWarpsPerBlock, true>(plan, a, st);
    }
    // `stages` = S (ring slots per warp) or 10*S + resident blocks per SM for the variants that
    // differ in occupancy.  Shared memory per block = 4 warps x S x (nq + 0.5) KB (+ ids).
    switch (nq) {
        case 4:
            switch (stages) {
                case 3: return launch_variant<4, 3, 3>(plan, a, st);
                case 43: return launch_variant<4, 4, 3>(plan, a, st);
                case 5: return launch_variant<4, 5, 2>(plan, a, st);
                case 6: return launch_variant<4, 6, 2>(plan, a, st);
                case 8: return launch_variant<4, 8, 1>(plan, a, st);
                case 104: return launch_variant<4, 4, 12, 1>(plan, a, st);   // one warp per block: 128-column slabs
                case 106: return launch_variant<4, 6, 8, 1>(plan, a, st);
                case 204: return launch_variant<4, 4, 6, 2>(plan, a, st);    // two warps per block: 256-column slabs
                default: return launch_variant<4, 4, 2>(plan, a, st);
            }
        case 2:
            switch (stages) {
                case 3: return launch_variant<2, 3, 5>(plan, a, st);
                case 45: return launch_variant<2, 4, 5>(plan, a, st);
                case 5: return launch_variant<2, 5, 4>(plan, a, st);
                case 6: return launch_variant<2, 6, 3>(plan, a, st);
                case 8: return launch_variant<2, 8, 2>(plan, a, st);
                case 104: return launch_variant<2, 4, 16, 1>(plan, a, st);   // one warp per block: 64-column slabs
                case 108: return launch_variant<2, 8, 12, 1>(plan, a, st);
                default: return launch_variant<2, 4, 4>(plan, a, st);
            }
        default:
            switch (stages) {
                case 4: return launch_variant<1, 4, 6>(plan, a, st);
                default: return launch_variant<1, 8, 4>(plan, a, st);
            }
    }
}

}  // namespace mask
