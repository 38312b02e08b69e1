// Pieces shared by the SpMM kernels: launch arguments, the TF32 MMA wrapper and operand rounding.
#pragma once

#include "common.cuh"
#include "plan.h"

namespace mask {

struct SpmmArgs {
    const int32_t* frag_off;
    const int32_t* frag_win;
    const int32_t* frag_slot;
    const int32_t* group_off;
    const int32_t* group_tile;  // first tile of every group (+ closing entry): persistent kernel only
    int64_t n_frag;             // fragments in the plan (frag_off has n_frag + 1 entries)
    int32_t n_groups;
    int32_t n_col_blocks;       // persistent kernel: column blocks of 128*NSLAB columns
    const int32_t* val_sidx;
    const float* val_blk;      // SR-BCRS
    const int32_t* coo_off;    // ME-TCF: [begin, end) pairs per tile (+ closing entry); MCO: val_mco_off[T+1]
    const int32_t* coo_idx;    // ME-TCF
    const float* coo_val;      // ME-TCF and MCO: the stored values
    const unsigned long long* mco_mask;   // MCO: two 64-bit words per tile, bit Swizzle<1,2,3>(8r+c)
    float* const* peer_out;    // optional: n_peer_out more output bases (peer GPUs' copies of C, same layout)
    int32_t n_peer_out;
    const int32_t* row_map;    // optional: packed row i is output row row_map[i] (row reorder undone on the fly)
    const float* B;
    int64_t ldb;
    float* C;
    int64_t ldc;
    float* scratch;
    int32_t M;
    int32_t K;
    int32_t N;
    int32_t relu;
    int32_t tf32x3;  // compensated products (MASK_NUMERICS_TF32X3)
};

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t rna_bits(float x) { return __float_as_uint(x) + 0x1000u; }
// Split for compensated products: the rounded value itself (low 13 bits cleared) and the TF32
// operand of what the rounding lost.
__device__ __forceinline__ uint32_t tf32_hi(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }
__device__ __forceinline__ uint32_t tf32_lo(float x, uint32_t hi) { return rna_bits(x - __uint_as_float(hi)); }

__device__ __forceinline__ float4 ldg_f4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

constexpr int kWarpsPerBlock = 4;

// Tile encodings the kernels read: dense SR-BCRS tiles, ME-TCF COO runs, MCO bitmaps.
constexpr int kFmtSrbcrs = 0, kFmtMetcf = 1, kFmtMco = 2;

// MCO: the 4 consecutive operand positions 4*lane .. 4*lane+3 of a tile as TF32 operand bits
// (rounded to nearest, ties away), from the tile's two mask words and its compact values
// (values in ascending position order): position p holds value number popcount(mask bits below p).
__device__ __forceinline__ uint4 mco_expand(unsigned long long m0, unsigned long long m1, const uint32_t* vals, int lane) {
    const unsigned long long m = (lane & 16) ? m1 : m0;
    const int sh = 4 * (lane & 15);
    const uint32_t bits = (uint32_t)(m >> sh) & 0xFu;
    int at = ((lane & 16) ? __popcll(m0) : 0) + __popcll(m & ((1ull << sh) - 1ull));
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (bits & 1u) o.x = vals[at++] + 0x1000u;
    if (bits & 2u) o.y = vals[at++] + 0x1000u;
    if (bits & 4u) o.z = vals[at++] + 0x1000u;
    if (bits & 8u) o.w = vals[at] + 0x1000u;
    return o;
}

// x + (-0.0f) == x bit for bit for every x (NaN payloads aside); as opaque assembly it yields a
// fresh register.
__device__ __forceinline__ float detach(float x) {
    float y;
    asm volatile("add.rn.f32 %0, %1, 0f80000000;" : "=f"(y) : "f"(x));
    return y;
}

// Writes (and clears) a warp's accumulators for fragment ff: straight to C when the fragment is
// its whole window, else to the fragment's partial tile in scratch.  acc[q][j][i]: 32-column
// group q, MMA j (column cb + 4n + j), accumulator register i.
template <int NQ>
__device__ __forceinline__ void flush_fragment(const SpmmArgs& p, int ff, int col_base, int g, int k,
                                               float (&acc)[NQ][4][4]) {
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
            // A 128-bit store needs its four values in consecutive registers, and so does every
            // MMA accumulator quad -- with a different grouping.  detach() gives the store its own
            // registers, so the unavoidable moves happen here, once per fragment, instead of around
            // every MMA of the main loop.
            float4 v0 = make_float4(detach(acc[q][0][2 * h]), detach(acc[q][1][2 * h]), detach(acc[q][2][2 * h]),
                                    detach(acc[q][3][2 * h]));
            float4 v1 = make_float4(detach(acc[q][0][2 * h + 1]), detach(acc[q][1][2 * h + 1]),
                                    detach(acc[q][2][2 * h + 1]), detach(acc[q][3][2 * h + 1]));
            if (relu) {
                v0.x = fmaxf(v0.x, 0.f); v0.y = fmaxf(v0.y, 0.f); v0.z = fmaxf(v0.z, 0.f); v0.w = fmaxf(v0.w, 0.f);
                v1.x = fmaxf(v1.x, 0.f); v1.y = fmaxf(v1.y, 0.f); v1.z = fmaxf(v1.z, 0.f); v1.w = fmaxf(v1.w, 0.f);
            }
            if (r < rows_ok) {
                float* row = (slot < 0 && p.row_map) ? p.C + (int64_t)p.row_map[w * kWinRows + r] * p.ldc : dst + (int64_t)r * ld;
                if (c0 < p.N) *reinterpret_cast<float4*>(row + c0) = v0;
                if (c0 + 4 < p.N) *reinterpret_cast<float4*>(row + c0 + 4) = v1;
                if (slot < 0) {  // the same row into every peer's copy of C (plain stores over NVLink)
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
}

// spmm_sweep.cu: persistent tcgen05 kernel, any N % 4 == 0, groups of any length.  nslab = 128-column
// slabs per column block (1, 2, 4; 0 = by N).
int launch_spmm_sweep(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st, int nslab);

// spmm_tma.cu: persistent tcgen05 kernel fed by the tensor memory accelerator (SR-BCRS with a prepared
// plan, see mask_plan_prepare_values).
bool spmm_tma_applies(const mask_plan* plan, const SpmmArgs& a);
int launch_spmm_tma(const mask_plan* plan, const SpmmArgs& a, int64_t K, cudaStream_t st, int nslab);

// spmm_async.cu: shared-memory ring variant (SR-BCRS).  nq / stages 0 = defaults.
int launch_spmm_async(const mask_plan* plan, const SpmmArgs& a, cudaStream_t st, int nq, int stages);

}  // namespace mask
