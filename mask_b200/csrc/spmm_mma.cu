// Warp-level TF32 SpMM kernels for SR-BCRS 16x8 and ME-TCF on sm_100a.
//
// One warp owns a 16 x CW slab of C (CW = 32*NQ columns) and walks a contiguous range of 16x8
// tiles that the plan assigned to its thread block.  For every tile it needs the 8 gathered rows
// of B restricted to its CW columns; those are loaded STRAIGHT INTO MMA FRAGMENT REGISTERS with
// 128-bit loads (each warp-wide load covers 4 rows x 128 contiguous bytes), double-buffered in
// registers two tiles ahead.  No shared-memory staging of B, no block-wide barrier: the kernel
// is a stream of coalesced loads feeding mma.sync.m16n8k8.tf32, which is what an HBM/L2-bound
// gather wants.  The four warps of a block take adjacent column slabs of the same tiles, so the
// tile values and column ids are fetched from L2 once per block and hit L1 for the other warps.
//
// Column permutation trick.  For a group of 32 columns starting at cb, lane (g = lane/4,
// k = lane%4) loads float4 B[row_k][cb+4g .. cb+4g+3] and B[row_{k+4}][same].  Component j of
// those vectors is the B fragment of MMA j, whose n index g therefore stands for column
// cb + 4g + j.  The accumulator fragment of MMA j holds n' = 2k, 2k+1, i.e. columns
// cb + 8k + j and cb + 8k + 4 + j, so over j = 0..3 a lane owns 8 consecutive columns of rows g
// and g+8 and stores them with 128-bit stores.
//
// Operand rounding.  The reference kernel rounds both operands with cvt.rna.tf32.f32
// (examples/src_fp32/sr_bcrs/testbed/kernel.inc:809-814).  The tensor core ignores the low 13
// mantissa bits of a TF32 operand, so adding 0x1000 to the FP32 bit pattern beforehand is
// exactly round-to-nearest, ties away from zero, for every finite value (values that round past
// FLT_MAX become infinity, as with cvt.rna; infinities are unchanged).  A NaN whose payload has
// all of bits 12..22 set would wrap; non-finite inputs are outside the contract of the format
// anyway, because a dense tile multiplies stored zeros by every gathered row.
//
// Windows split across blocks write their partial 16xN tiles to scratch; a second kernel sums
// them in fragment order, so no atomics and no zero-fill of C are needed.
#include <cstring>

#include "common.cuh"
#include "plan.h"
#include "spmm_common.cuh"

namespace mask {


// Development knobs (mask_tune): 0 = library default.
static int g_tune_nq = 0;
static int g_tune_min_blocks = 0;
static int g_tune_async = 1;   // 1 = shared-memory ring fed by cp.async (SR-BCRS), 0 = register pipeline
static int g_tune_stages = 0;
extern int g_session_chunk_cols;      // api.cu: column chunks of the host-buffer pipeline
constexpr int kNarrowN = 80;   // below: the warp-level ring kernel (see launch_spmm)
static int g_tune_sweep = 1;   // 1 = persistent tcgen05 kernel except where the warp-level one measures faster, 2 = always, 0 = warp-level kernels only
static int g_tune_nslab = 0;   // persistent kernel: 128-column slabs per column block (0 = the plan's choice)
static int g_tune_tma = 0;     // 1 = the TMA-fed kernel where the plan holds rounded tile values (spmm_tma.cu); measured slower, off by default

template <int NQ, int FMT, int MIN_BLOCKS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, MIN_BLOCKS) spmm_mma_kernel(const SpmmArgs p) {
    constexpr bool METCF = FMT == kFmtMetcf, MCO = FMT == kFmtMco;
    // ME-TCF / MCO: one private 16x8 tile per warp, rebuilt from the tile's COO run or bitmap
    // (MCO: a second 128-float area stages the tile's compact values).
    __shared__ __align__(16) float restore[FMT != kFmtSrbcrs ? kWarpsPerBlock * (MCO ? 2 : 1) : 1][kTileElems];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int k = lane & 3;
    const int col_base = (blockIdx.y * kWarpsPerBlock + warp) * (32 * NQ);
    if (col_base >= p.N) return;

    int f = p.group_off[blockIdx.x];
    const int f_end = p.group_off[blockIdx.x + 1];
    if (f >= f_end) return;
    int64_t t = p.frag_off[f];
    const int64_t t_end = p.frag_off[f_end];
    int64_t f_tend = p.frag_off[f + 1];

    // position of this lane's A fragment elements inside a stored tile
    int ao[4];
    if (FMT != kFmtSrbcrs) {
        ao[0] = sw123(8 * g + k);       ao[1] = sw123(8 * (g + 8) + k);
        ao[2] = sw123(8 * g + k + 4);   ao[3] = sw123(8 * (g + 8) + k + 4);
    } else {
        ao[0] = sw223(8 * g + k);       ao[1] = sw223(8 * (g + 8) + k);
        ao[2] = sw223(8 * g + k + 4);   ao[3] = sw223(8 * (g + 8) + k + 4);
    }

    bool qok[NQ];
#pragma unroll
    for (int q = 0; q < NQ; q++) qok[q] = (col_base + 32 * q + 4 * g) < p.N;

    float acc[NQ][4][4];
#pragma unroll
    for (int q = 0; q < NQ; q++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[q][j][i] = 0.f;

    // ---- register pipeline state -----------------------------------------------------------
    float4 breg[2][NQ][2];   // B fragments of the two tiles in flight
    float areg[2][4];        // SR-BCRS: A fragment values; ME-TCF: [0] = this lane's COO value
    int aidx[2];             // ME-TCF: this lane's COO index (or -1)
    int2 run[2];             // ME-TCF: [begin, end) of the tile's COO run
    int2 ix[2];              // gathered-row ids (k, k+4) of tiles t+2, t+3
    int2 nrun[2];            // ME-TCF: runs of tiles t+2, t+3
    ulonglong2 mk[2];        // MCO: mask words of the two tiles in flight
    float4 mv[2];            // MCO: this lane's chunk of the tile's compact values

    const float* Bcol = p.B + col_base + 4 * g;

    auto load_ix = [&](int slot, int64_t tt) {
        if (tt < t_end) {
            ix[slot].x = __ldg(p.val_sidx + tt * kTileCols + k);
            ix[slot].y = __ldg(p.val_sidx + tt * kTileCols + k + 4);
            if (METCF) {
                nrun[slot].x = __ldg(p.coo_off + 2 * tt);
                nrun[slot].y = __ldg(p.coo_off + 2 * tt + 1);
            }
            if (MCO) {
                nrun[slot].x = __ldg(p.coo_off + tt);
                nrun[slot].y = __ldg(p.coo_off + tt + 1);
            }
        }
    };
    auto load_tile = [&](int buf, int64_t tt, int2 id, int2 rn) {
        if (tt < t_end) {
            const float* r0 = Bcol + (int64_t)id.x * p.ldb;
            const float* r1 = Bcol + (int64_t)id.y * p.ldb;
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                if (qok[q]) {
                    breg[buf][q][0] = ldg_f4(r0 + 32 * q);
                    breg[buf][q][1] = ldg_f4(r1 + 32 * q);
                } else {
                    breg[buf][q][0] = make_float4(0.f, 0.f, 0.f, 0.f);
                    breg[buf][q][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            if (METCF) {
                run[buf] = rn;
                const int e = rn.x + lane;
                if (e < rn.y) {
                    aidx[buf] = __ldg(p.coo_idx + e);
                    areg[buf][0] = __ldg(p.coo_val + e);
                } else {
                    aidx[buf] = -1;
                }
            } else if (MCO) {
                run[buf] = rn;
                mk[buf] = __ldg(reinterpret_cast<const ulonglong2*>(p.mco_mask) + tt);
                if (rn.x + 4 * lane < rn.y) mv[buf] = ldg_f4(p.coo_val + rn.x + 4 * lane);   // runs are multiples of 4 values
            } else {
                const float* a = p.val_blk + tt * kTileElems;
#pragma unroll
                for (int i = 0; i < 4; i++) areg[buf][i] = __ldg(a + ao[i]);
            }
        }
    };

    auto flush = [&](int ff) {
        const int w = p.frag_win[ff];
        const int slot = p.frag_slot[ff];
        float* dst;
        int64_t ld;
        int rows_ok;
        if (slot < 0) {
            dst = p.C + (int64_t)w * kWinRows * p.ldc;
            ld = p.ldc;
            rows_ok = p.M - w * kWinRows;
        } else {
            dst = p.scratch + (int64_t)slot * kWinRows * p.N;
            ld = p.N;
            rows_ok = kWinRows;
        }
        const bool relu = p.relu && slot < 0;
#pragma unroll
        for (int q = 0; q < NQ; q++) {
            const int c0 = col_base + 32 * q + 8 * k;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int r = g + 8 * h;
                float4 v0 = make_float4(acc[q][0][2 * h], acc[q][1][2 * h], acc[q][2][2 * h], acc[q][3][2 * h]);
                float4 v1 = make_float4(acc[q][0][2 * h + 1], acc[q][1][2 * h + 1], acc[q][2][2 * h + 1],
                                        acc[q][3][2 * h + 1]);
                if (relu) {
                    v0.x = fmaxf(v0.x, 0.f); v0.y = fmaxf(v0.y, 0.f); v0.z = fmaxf(v0.z, 0.f); v0.w = fmaxf(v0.w, 0.f);
                    v1.x = fmaxf(v1.x, 0.f); v1.y = fmaxf(v1.y, 0.f); v1.z = fmaxf(v1.z, 0.f); v1.w = fmaxf(v1.w, 0.f);
                }
                if (r < rows_ok) {
                    float* row = (slot < 0 && p.row_map) ? p.C + (int64_t)p.row_map[w * kWinRows + r] * p.ldc
                                                         : dst + (int64_t)r * ld;
                    if (c0 < p.N) *reinterpret_cast<float4*>(row + c0) = v0;
                    if (c0 + 4 < p.N) *reinterpret_cast<float4*>(row + c0 + 4) = v1;
                    if (slot < 0) {  // the same row into every peer's copy of C
                        const int64_t off = row - p.C;
                        for (int j = 0; j < p.n_peer_out; j++) {
                            float* prow = p.peer_out[j] + off;
                            if (c0 < p.N) *reinterpret_cast<float4*>(prow + c0) = v0;
                            if (c0 + 4 < p.N) *reinterpret_cast<float4*>(prow + c0 + 4) = v1;
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[q][j][i] = 0.f;
        }
    };

    auto consume = [&](int buf) {
        uint32_t a[4];
        if (METCF) {
            float* tile = restore[warp];
            __syncwarp();
            reinterpret_cast<float4*>(tile)[lane] = make_float4(0.f, 0.f, 0.f, 0.f);
            __syncwarp();
            if (aidx[buf] >= 0) tile[aidx[buf]] = areg[buf][0];
            // runs longer than one entry per lane (more than 32 stored entries in the tile)
            for (int e = run[buf].x + 32 + lane; e < run[buf].y; e += 32) tile[__ldg(p.coo_idx + e)] = __ldg(p.coo_val + e);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = rna_bits(tile[ao[i]]);
        } else if (MCO) {
            float* tile = restore[2 * warp];
            float* vals = restore[2 * warp + 1];
            __syncwarp();
            if (run[buf].x + 4 * lane < run[buf].y) reinterpret_cast<float4*>(vals)[lane] = mv[buf];
            __syncwarp();
            reinterpret_cast<uint4*>(tile)[lane] = mco_expand(mk[buf].x, mk[buf].y, reinterpret_cast<const uint32_t*>(vals), lane);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = __float_as_uint(tile[ao[i]]);   // already rounded by mco_expand
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = rna_bits(areg[buf][i]);
        }
#pragma unroll
        for (int q = 0; q < NQ; q++) {
            const float4 v0 = breg[buf][q][0], v1 = breg[buf][q][1];
            mma_tf32(acc[q][0], a, rna_bits(v0.x), rna_bits(v1.x));
            mma_tf32(acc[q][1], a, rna_bits(v0.y), rna_bits(v1.y));
            mma_tf32(acc[q][2], a, rna_bits(v0.z), rna_bits(v1.z));
            mma_tf32(acc[q][3], a, rna_bits(v0.w), rna_bits(v1.w));
        }
    };

    // ---- prologue: ids of tiles t..t+3, fragments of tiles t, t+1 ---------------------------
    {
        int2 id0 = make_int2(0, 0), id1 = make_int2(0, 0), rn0 = make_int2(0, 0), rn1 = make_int2(0, 0);
        load_ix(0, t);
        load_ix(1, t + 1);
        id0 = ix[0]; id1 = ix[1]; rn0 = nrun[0]; rn1 = nrun[1];
        load_ix(0, t + 2);
        load_ix(1, t + 3);
        load_tile(0, t, id0, rn0);
        load_tile(1, t + 1, id1, rn1);
    }

    // ---- main loop, two tiles per trip so that buffer indices stay compile-time --------------
    while (true) {
#pragma unroll
        for (int s = 0; s < 2; s++) {
            while (t == f_tend && f < f_end) {  // fragment finished (also: fragments with no tile)
                flush(f);
                f++;
                f_tend = (f < f_end) ? p.frag_off[f + 1] : -1;
            }
            if (f >= f_end) return;
            consume(s);
            const int2 id = ix[s], rn = nrun[s];
            load_ix(s, t + 4);
            load_tile(s, t + 2, id, rn);
            t++;
        }
    }
}

// Sums the partial tiles of every split window in fragment (= tile) order and writes C.
__global__ void __launch_bounds__(256) spmm_fixup_kernel(const int32_t* head_frag, const int32_t* frag_win,
                                                        const int32_t* frag_slot, int64_t n_frag,
                                                        const float* scratch, float* C, int64_t ldc, int32_t M,
                                                        int32_t N, int32_t relu, const int32_t* row_map,
                                                        float* const* peer_out, int32_t n_peer_out) {
    const int64_t f0 = head_frag[blockIdx.x];
    const int w = frag_win[f0];
    int64_t f1 = f0;
    while (f1 < n_frag && frag_win[f1] == w && frag_slot[f1] >= 0) f1++;
    const int nvec = N >> 2;
    for (int v = blockIdx.y * blockDim.x + threadIdx.x; v < kWinRows * nvec; v += gridDim.y * blockDim.x) {
        const int r = v / nvec, c = (v - r * nvec) << 2;
        if (w * kWinRows + r >= M) continue;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int64_t ff = f0; ff < f1; ff++) {
            const float4 x = *reinterpret_cast<const float4*>(scratch + ((int64_t)frag_slot[ff] * kWinRows + r) * N + c);
            s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
        }
        if (relu) { s.x = fmaxf(s.x, 0.f); s.y = fmaxf(s.y, 0.f); s.z = fmaxf(s.z, 0.f); s.w = fmaxf(s.w, 0.f); }
        const int out_row = row_map ? row_map[w * kWinRows + r] : w * kWinRows + r;
        *reinterpret_cast<float4*>(C + (int64_t)out_row * ldc + c) = s;
        for (int j = 0; j < n_peer_out; j++) *reinterpret_cast<float4*>(peer_out[j] + (int64_t)out_row * ldc + c) = s;
    }
}

static int launch_fixup(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st) {
    if (plan->H > 0) {
        dim3 fgrid((unsigned)plan->H, (unsigned)((kWinRows * (a.N >> 2) + 255) / 256));
        spmm_fixup_kernel<<<fgrid, 256, 0, st>>>(plan->d_head_frag, plan->d_frag_win, plan->d_frag_slot, plan->F,
                                                 a.scratch, a.C, a.ldc, a.M, a.N, a.relu, a.row_map, a.peer_out, a.n_peer_out);
        MASK_CUDA_TRY(cudaGetLastError());
    }
    return MASK_OK;
}

template <int FMT>
static int launch_spmm(const mask_plan* plan, SpmmArgs a, cudaStream_t st) {
    if (plan->G == 0) return MASK_OK;
    a.frag_off = plan->d_frag_off;
    a.frag_win = plan->d_frag_win;
    a.frag_slot = plan->d_frag_slot;
    a.group_off = plan->d_group_off;
    a.row_map = plan->d_row_map;
    a.peer_out = plan->d_peer_out;
    a.n_peer_out = plan->n_peer_out;
    // columns per warp: wide slabs (fewer re-reads of the tile values per column) when N fills
    // four warps of them, else narrower slabs so that small N still spreads over a block
    const int N = a.N;
    constexpr bool METCF = FMT != kFmtSrbcrs;   // the COO and bitmap leaves take the same routes
    if (FMT == kFmtSrbcrs && a.tf32x3) {   // compensated products: mma.sync ring kernel
        int rc = launch_spmm_async(plan, a, st, 0, 0);
        if (rc != MASK_OK) return rc;
        return launch_fixup(plan, a, st);
    }
    // Narrow products: below about 80 columns a tile's one mostly empty 128-column MMA costs more than
    // the warp-level MMAs of the shared-memory ring kernel (measured on a 2^22-node power-law graph:
    // N = 64 5.33 against 6.33 ms, N = 80 6.57 against 6.48 ms, N = 128 6.8 ms for the tcgen05 kernel).
    if (FMT == kFmtSrbcrs && g_tune_sweep == 1 && N < kNarrowN && g_tune_async != 0) {
        int rc = launch_spmm_async(plan, a, st, g_tune_nq, g_tune_stages);
        if (rc != MASK_OK) return rc;
        return launch_fixup(plan, a, st);
    }
    if (g_tune_sweep != 0 && g_tune_tma != 0 && FMT == kFmtSrbcrs && spmm_tma_applies(plan, a)) {
        int rc = launch_spmm_tma(plan, a, a.K, st, g_tune_nslab != 0 ? g_tune_nslab : plan->nslab);
        if (rc != MASK_OK) return rc;
        return launch_fixup(plan, a, st);
    }
    if (g_tune_sweep != 0) {
        int rc = launch_spmm_sweep(plan, a, st, g_tune_nslab != 0 ? g_tune_nslab : plan->nslab);
        if (rc != MASK_OK) return rc;
        return launch_fixup(plan, a, st);
    }
    if (!METCF && g_tune_async != 0) {
        int rc = launch_spmm_async(plan, a, st, g_tune_nq, g_tune_stages);
        if (rc != MASK_OK) return rc;
        return launch_fixup(plan, a, st);
    }
    int nq = N > 256 ? 4 : (N > 128 ? 2 : 1);
    if (g_tune_nq == 1 || g_tune_nq == 2 || g_tune_nq == 4) nq = g_tune_nq;
    const int cols_per_block = 32 * nq * kWarpsPerBlock;
    dim3 grid((unsigned)plan->G, (unsigned)((N + cols_per_block - 1) / cols_per_block));
    dim3 block(kWarpsPerBlock * 32);
    if (grid.y > 65535) return fail(MASK_ERR_INVALID_ARGUMENT, "N too large");
    switch (nq) {
        case 4:
            if (g_tune_min_blocks == 3) spmm_mma_kernel<4, FMT, 3><<<grid, block, 0, st>>>(a);
            else spmm_mma_kernel<4, FMT, 2><<<grid, block, 0, st>>>(a);
            break;
        case 2:
            if (g_tune_min_blocks == 4) spmm_mma_kernel<2, FMT, 4><<<grid, block, 0, st>>>(a);
            else spmm_mma_kernel<2, FMT, 3><<<grid, block, 0, st>>>(a);
            break;
        default: spmm_mma_kernel<1, FMT, 4><<<grid, block, 0, st>>>(a); break;
    }
    MASK_CUDA_TRY(cudaGetLastError());
    return launch_fixup(plan, a, st);
}

static int check_common(const mask_plan* plan, int32_t M, int32_t K, int32_t N, const float* B, int64_t ldb,
                        float* C, int64_t ldc, void* scratch, size_t scratch_bytes) {
    MASK_REQUIRE(plan != nullptr, "plan is NULL");
    MASK_REQUIRE(M == plan->M, "M differs from the plan's");
    MASK_REQUIRE(M >= 1 && K >= 1 && N >= 0, "M, K must be positive and N non-negative");
    MASK_REQUIRE(N % 4 == 0, "N must be a multiple of 4");
    if (N == 0) return MASK_OK;
    MASK_REQUIRE(B != nullptr && C != nullptr, "B or C is NULL");
    MASK_REQUIRE(ldb >= N && ldc >= N && ldb % 4 == 0 && ldc % 4 == 0, "ldb/ldc must be >= N and multiples of 4");
    MASK_REQUIRE(ldb < ((int64_t)1 << 30), "ldb too large");
    MASK_REQUIRE((reinterpret_cast<uintptr_t>(B) & 15) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0,
                 "B and C must be 16-byte aligned");
    const size_t need = mask_plan_scratch_bytes(plan, N);
    if (need > 0) {
        if (scratch == nullptr || scratch_bytes < need) return fail(MASK_ERR_SCRATCH_TOO_SMALL, "scratch too small for the plan's split windows");
        MASK_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 15) == 0, "scratch must be 16-byte aligned");
    }
    return MASK_OK;
}

}  // namespace mask

extern "C" int mask_kernel_revision(void) { return 4; }

extern "C" int mask_spmm_kernel_name(const mask_plan* plan, int format, int32_t N, int epilogue, char* out, size_t capacity) {
    using namespace mask;
    MASK_REQUIRE(plan != nullptr && out != nullptr && capacity > 0, "NULL argument");
    MASK_REQUIRE(format >= kFmtSrbcrs && format <= kFmtMco && N > 0, "bad format or N");
    static const char* const fmt_name[] = {"srbcrs", "metcf", "mco"};
    if (format == kFmtSrbcrs && (epilogue & MASK_NUMERICS_TF32X3)) {
        snprintf(out, capacity, "spmm_async_kernel<tf32x3>");
    } else if (format == kFmtSrbcrs && g_tune_sweep == 1 && N < kNarrowN && g_tune_async != 0) {
        snprintf(out, capacity, "spmm_async_kernel<%s>", fmt_name[format]);
    } else if (g_tune_sweep != 0) {
        int nslab = g_tune_nslab != 0 ? g_tune_nslab : plan->nslab;
        const int fills = N > 256 ? 4 : (N > 128 ? 2 : 1);
        if (nslab != 1 && nslab != 2 && nslab != 4) nslab = fills;
        nslab = nslab < fills ? nslab : fills;
        const bool tma = g_tune_tma != 0 && format == kFmtSrbcrs && plan->d_vals_tf32 != nullptr;
        snprintf(out, capacity, "%s<nslab=%d,%s>", tma ? "spmm_tma_kernel" : "spmm_sweep_kernel", nslab, fmt_name[format]);
    } else {
        snprintf(out, capacity, "legacy routing (mask_tune sweep=0), %s", fmt_name[format]);
    }
    return MASK_OK;
}

extern "C" int mask_tune(const char* name, int value) {
    using namespace mask;
    MASK_REQUIRE(name != nullptr, "name is NULL");
    if (!strcmp(name, "nq")) g_tune_nq = value;
    else if (!strcmp(name, "min_blocks")) g_tune_min_blocks = value;
    else if (!strcmp(name, "async")) g_tune_async = value;
    else if (!strcmp(name, "stages")) g_tune_stages = value;
    else if (!strcmp(name, "sweep")) g_tune_sweep = value;
    else if (!strcmp(name, "nslab")) g_tune_nslab = value;
    else if (!strcmp(name, "tma")) g_tune_tma = value;
    else if (!strcmp(name, "session_chunk")) g_session_chunk_cols = value;
    else return fail(MASK_ERR_INVALID_ARGUMENT, "unknown tuning knob");
    return MASK_OK;
}

extern "C" int mask_spmm_srbcrs(const mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx,
                                const float* d_val_block_val, int32_t M, int32_t K, int32_t N, const float* d_B,
                                int64_t ldb, float* d_C, int64_t ldc, void* d_scratch, size_t scratch_bytes,
                                int epilogue, void* stream) {
    using namespace mask;
    (void)d_val_soff;
    int rc = check_common(plan, M, K, N, d_B, ldb, d_C, ldc, d_scratch, scratch_bytes);
    if (rc != MASK_OK || N == 0) return rc;
    MASK_REQUIRE(plan->T == 0 || (d_val_sidx != nullptr && d_val_block_val != nullptr), "packed arrays are NULL");
    SpmmArgs a{};
    a.val_sidx = d_val_sidx;
    a.val_blk = d_val_block_val;
    a.B = d_B; a.ldb = ldb; a.C = d_C; a.ldc = ldc;
    a.scratch = static_cast<float*>(d_scratch);
    a.M = M; a.K = K; a.N = N; a.relu = ((epilogue & 0xff) == MASK_EPILOGUE_RELU);
    a.tf32x3 = (epilogue & MASK_NUMERICS_TF32X3) ? 1 : 0;
    return launch_spmm<kFmtSrbcrs>(plan, a, static_cast<cudaStream_t>(stream));
}

extern "C" int mask_spmm_metcf(const mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx,
                               const int32_t* d_val_coo_off, const int32_t* d_val_coo_idx, const float* d_val_coo_val,
                               int32_t M, int32_t K, int32_t N, const float* d_B, int64_t ldb, float* d_C, int64_t ldc,
                               void* d_scratch, size_t scratch_bytes, int epilogue, void* stream) {
    using namespace mask;
    (void)d_val_soff;
    int rc = check_common(plan, M, K, N, d_B, ldb, d_C, ldc, d_scratch, scratch_bytes);
    if (rc != MASK_OK || N == 0) return rc;
    MASK_REQUIRE(plan->T == 0 || (d_val_sidx != nullptr && d_val_coo_off != nullptr && d_val_coo_idx != nullptr &&
                                  d_val_coo_val != nullptr), "packed arrays are NULL");
    SpmmArgs a{};
    a.val_sidx = d_val_sidx;
    a.coo_off = d_val_coo_off; a.coo_idx = d_val_coo_idx; a.coo_val = d_val_coo_val;
    a.B = d_B; a.ldb = ldb; a.C = d_C; a.ldc = ldc;
    a.scratch = static_cast<float*>(d_scratch);
    a.M = M; a.K = K; a.N = N; a.relu = ((epilogue & 0xff) == MASK_EPILOGUE_RELU);
    MASK_REQUIRE(!(epilogue & MASK_NUMERICS_TF32X3), "compensated products are implemented for SR-BCRS only");
    return launch_spmm<kFmtMetcf>(plan, a, static_cast<cudaStream_t>(stream));
}

extern "C" int mask_spmm_mco(const mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx,
                             const int32_t* d_val_mco_off, const uint64_t* d_val_mco_mask, const float* d_val_mco_val,
                             int32_t M, int32_t K, int32_t N, const float* d_B, int64_t ldb, float* d_C, int64_t ldc,
                             void* d_scratch, size_t scratch_bytes, int epilogue, void* stream) {
    using namespace mask;
    (void)d_val_soff;
    int rc = check_common(plan, M, K, N, d_B, ldb, d_C, ldc, d_scratch, scratch_bytes);
    if (rc != MASK_OK || N == 0) return rc;
    MASK_REQUIRE(plan->T == 0 || (d_val_sidx != nullptr && d_val_mco_off != nullptr && d_val_mco_mask != nullptr),
                 "packed arrays are NULL");
    MASK_REQUIRE((reinterpret_cast<uintptr_t>(d_val_mco_mask) & 15) == 0 && (reinterpret_cast<uintptr_t>(d_val_mco_val) & 15) == 0,
                 "val_mco_mask and val_mco_val must be 16-byte aligned");
    SpmmArgs a{};
    a.val_sidx = d_val_sidx;
    a.coo_off = d_val_mco_off;
    a.coo_val = d_val_mco_val;
    a.mco_mask = reinterpret_cast<const unsigned long long*>(d_val_mco_mask);
    a.B = d_B; a.ldb = ldb; a.C = d_C; a.ldc = ldc;
    a.scratch = static_cast<float*>(d_scratch);
    a.M = M; a.K = K; a.N = N; a.relu = ((epilogue & 0xff) == MASK_EPILOGUE_RELU);
    MASK_REQUIRE(!(epilogue & MASK_NUMERICS_TF32X3), "compensated products are implemented for SR-BCRS only");
    return launch_spmm<kFmtMco>(plan, a, static_cast<cudaStream_t>(stream));
}
