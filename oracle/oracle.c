/*
 * CPU oracle for the SR-BCRS 16x8 / ME-TCF SpMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, what the reference project (hd9568/MASK, "Sparsene")
 * computes on the host for this path.  It exists so that the CUDA kernels of this repository
 * can be checked against an independent implementation; it is never linked into, imported by
 * or called from the product library.  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load it.
 *
 * Parity status: PINNED.  Every packer / planner below is compared byte for byte against the
 * reference project's own host code (built from the reference sources into oracle/_ref by
 * oracle/Makefile) in tests/test_oracle.py, and against the committed fixtures
 * under tests/golden/ that were generated from those reference builds.
 *
 * Citations are paths inside the reference project.
 *
 * Preconditions shared by the packers (same as the reference testbed packers, which use a
 * monotone lower_bound hint that is only meaningful for such input,
 * examples/src_fp32/sr_bcrs/testbed/main_16x8.cu:304-310): CSR rows hold strictly ascending
 * column ids (sorted, no duplicates), int32 indices.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define WIN_ROWS 16
#define TILE_COLS 8
#define TILE_ELEMS 128

static int cmp_int(const void* a, const void* b) {
    int x = *(const int*)a, y = *(const int*)b;
    return (x > y) - (x < y);
}

/* Swizzle<2,2,3> over a row-major 16x8 tile, closed form
 * (cute::Swizzle<2,2,3> composed with (16,8):(8,1), main_16x8.cu:259-260). */
static inline int sw223(int i) { return i ^ (((i >> 5) & 3) << 2); }
/* Swizzle<1,2,3> over the same tile (examples/src_fp32/dtc/testbed/main.cu:436-438). */
static inline int sw123(int i) { return i ^ (((i >> 5) & 1) << 2); }

int oracle_sw223(int i) { return sw223(i); }
int oracle_sw123(int i) { return sw123(i); }

/* Ascending distinct columns of window w into `out` (capacity = window nnz); returns count.
 * Restates the col_mark + sort step (main_16x8.cu:214-236). */
static int window_unique_cols(int M, const int* rowptr, const int* colind, int w, int* out) {
    int r0 = w * WIN_ROWS, r1 = r0 + WIN_ROWS;
    if (r1 > M) r1 = M;
    int n = rowptr[r1] - rowptr[r0];
    if (n <= 0) return 0;
    memcpy(out, colind + rowptr[r0], sizeof(int) * (size_t)n);
    qsort(out, (size_t)n, sizeof(int), cmp_int);
    int u = 0;
    for (int i = 0; i < n; i++)
        if (i == 0 || out[i] != out[u - 1]) out[u++] = out[i];
    return u;
}

static int lower_bound_int(const int* a, int n, int key) {
    int lo = 0, hi = n;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (a[mid] < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

static int max_window_nnz(int M, const int* rowptr) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS, best = 0;
    for (int w = 0; w < W; w++) {
        int r0 = w * WIN_ROWS, r1 = r0 + WIN_ROWS;
        if (r1 > M) r1 = M;
        int n = rowptr[r1] - rowptr[r0];
        if (n > best) best = n;
    }
    return best;
}

/* ---- SR-BCRS 16x8 ----------------------------------------------------------------------
 * Pass 1: tiles per window and their exclusive scan (main_16x8.cu:209-251).
 * val_soff has W+1 entries.  Returns T. */
int64_t oracle_srbcrs_count(int M, const int* rowptr, const int* colind, int* val_soff) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int cap = max_window_nnz(M, rowptr);
    int* tiles = (int*)calloc((size_t)(W > 0 ? W : 1), sizeof(int));
#pragma omp parallel
    {
        int* buf = (int*)malloc(sizeof(int) * (size_t)(cap > 0 ? cap : 1));
#pragma omp for schedule(dynamic, 64)
        for (int w = 0; w < W; w++) {
            int u = window_unique_cols(M, rowptr, colind, w, buf);
            tiles[w] = (u + TILE_COLS - 1) / TILE_COLS;
        }
        free(buf);
    }
    int64_t T = 0;
    for (int w = 0; w < W; w++) { val_soff[w] = (int)T; T += tiles[w]; }
    val_soff[W] = (int)T;
    free(tiles);
    return T;
}

/* Pass 2: column metadata (padded with the window's last real column, main_16x8.cu:288-297)
 * and swizzled tile values (main_16x8.cu:299-318).  val_sidx: 8T ints, val_block_val: 128T. */
void oracle_srbcrs_fill(int M, const int* rowptr, const int* colind, const float* values,
                        const int* val_soff, int* val_sidx, float* val_block_val) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int cap = max_window_nnz(M, rowptr);
    int64_t T = val_soff[W];
    memset(val_block_val, 0, sizeof(float) * (size_t)T * TILE_ELEMS);
#pragma omp parallel
    {
        int* U = (int*)malloc(sizeof(int) * (size_t)(cap > 0 ? cap : 1));
#pragma omp for schedule(dynamic, 64)
        for (int w = 0; w < W; w++) {
            int u = window_unique_cols(M, rowptr, colind, w, U);
            int nt = (u + TILE_COLS - 1) / TILE_COLS;
            int* sidx = val_sidx + (int64_t)val_soff[w] * TILE_COLS;
            float* blk = val_block_val + (int64_t)val_soff[w] * TILE_ELEMS;
            for (int j = 0; j < nt * TILE_COLS; j++) sidx[j] = (j < u) ? U[j] : U[u - 1];
            for (int r = 0; r < WIN_ROWS; r++) {
                int row = w * WIN_ROWS + r;
                if (row >= M) break;
                for (int e = rowptr[row]; e < rowptr[row + 1]; e++) {
                    int pos = lower_bound_int(U, u, colind[e]);
                    blk[(int64_t)(pos / TILE_COLS) * TILE_ELEMS + sw223(r * TILE_COLS + pos % TILE_COLS)] =
                        values[e];
                }
            }
        }
        free(U);
    }
}

/* Side outputs of the extension packer (examples/src_fp32/sr_bcrs/testbed/SRBCRSSpMM_kernel.cu:
 * 241,250,268): block_partition[w] = tiles of window w, edge_to_row[e] = row of entry e,
 * edge_to_col[e] = condensed position of entry e in its window. */
void oracle_edge_maps(int M, const int* rowptr, const int* colind, int* block_partition,
                      int* edge_to_col, int* edge_to_row) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int cap = max_window_nnz(M, rowptr);
    int* U = (int*)malloc(sizeof(int) * (size_t)(cap > 0 ? cap : 1));
    for (int w = 0; w < W; w++) {
        int u = window_unique_cols(M, rowptr, colind, w, U);
        block_partition[w] = (u + TILE_COLS - 1) / TILE_COLS;
        for (int r = 0; r < WIN_ROWS; r++) {
            int row = w * WIN_ROWS + r;
            if (row >= M) break;
            for (int e = rowptr[row]; e < rowptr[row + 1]; e++) {
                edge_to_row[e] = row;
                edge_to_col[e] = lower_bound_int(U, u, colind[e]);
            }
        }
    }
    free(U);
}

/* ---- ME-TCF ------------------------------------------------------------------------------
 * Pass 1 (examples/src_fp32/dtc/testbed/main.cu:360-425): tiles per window, exclusive scan,
 * and the padded COO length.  Returns T; *nnz_pad_out = sum over tiles of ceil8(cnt). */
int64_t oracle_metcf_count(int M, const int* rowptr, const int* colind, int* val_soff,
                           int64_t* nnz_pad_out) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int cap = max_window_nnz(M, rowptr);
    int* U = (int*)malloc(sizeof(int) * (size_t)(cap > 0 ? cap : 1));
    int* cnt = (int*)malloc(sizeof(int) * (size_t)(cap / 1 + 1));
    int64_t T = 0, pad = 0;
    for (int w = 0; w < W; w++) {
        int u = window_unique_cols(M, rowptr, colind, w, U);
        int nt = (u + TILE_COLS - 1) / TILE_COLS;
        val_soff[w] = (int)T;
        T += nt;
        memset(cnt, 0, sizeof(int) * (size_t)(nt > 0 ? nt : 1));
        int r0 = w * WIN_ROWS, r1 = r0 + WIN_ROWS;
        if (r1 > M) r1 = M;
        for (int e = rowptr[r0]; e < rowptr[r1]; e++) cnt[lower_bound_int(U, u, colind[e]) / TILE_COLS]++;
        for (int b = 0; b < nt; b++) pad += (cnt[b] + 7) / 8 * 8;
    }
    val_soff[W] = (int)T;
    *nnz_pad_out = pad;
    free(U);
    free(cnt);
    return T;
}

/* Pass 2 (main.cu:427-517): val_sidx padded with 0, val_coo_off = [begin, begin+cnt] per tile
 * plus a closing nnz_pad, runs padded to 8 entries, entries in (row ascending, CSR order)
 * with idx = Swizzle<1,2,3>(8r+c).  Padding slots hold idx 0 / value 0. */
void oracle_metcf_fill(int M, const int* rowptr, const int* colind, const float* values,
                       const int* val_soff, int* val_sidx, int* val_coo_off, int* val_coo_idx,
                       float* val_coo_val, int64_t nnz_pad) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int cap = max_window_nnz(M, rowptr);
    int64_t T = val_soff[W];
    memset(val_sidx, 0, sizeof(int) * (size_t)T * TILE_COLS);
    memset(val_coo_idx, 0, sizeof(int) * (size_t)nnz_pad);
    memset(val_coo_val, 0, sizeof(float) * (size_t)nnz_pad);
    int* U = (int*)malloc(sizeof(int) * (size_t)(cap > 0 ? cap : 1));
    int* cur = (int*)malloc(sizeof(int) * (size_t)(cap + 1));
    int pos = 0;
    for (int w = 0; w < W; w++) {
        int u = window_unique_cols(M, rowptr, colind, w, U);
        int nt = val_soff[w + 1] - val_soff[w];
        memcpy(val_sidx + (int64_t)val_soff[w] * TILE_COLS, U, sizeof(int) * (size_t)u);
        memset(cur, 0, sizeof(int) * (size_t)(nt > 0 ? nt : 1));
        int r0 = w * WIN_ROWS, r1 = r0 + WIN_ROWS;
        if (r1 > M) r1 = M;
        for (int e = rowptr[r0]; e < rowptr[r1]; e++) cur[lower_bound_int(U, u, colind[e]) / TILE_COLS]++;
        for (int b = 0; b < nt; b++) {
            int t = val_soff[w] + b, c = cur[b];
            val_coo_off[2 * t] = pos;
            val_coo_off[2 * t + 1] = pos + c;
            cur[b] = pos;
            pos += (c + 7) / 8 * 8;
        }
        for (int row = r0; row < r1; row++) {
            for (int e = rowptr[row]; e < rowptr[row + 1]; e++) {
                int p = lower_bound_int(U, u, colind[e]);
                int slot = cur[p / TILE_COLS]++;
                val_coo_val[slot] = values[e];
                val_coo_idx[slot] = sw123((row - r0) * TILE_COLS + p % TILE_COLS);
            }
        }
    }
    val_coo_off[2 * T] = pos;
    free(U);
    free(cur);
}

/* ---- MCO / BIT-TCF (bitmap leaf) -----------------------------------------------------------
 * examples/src_fp32/acc/testbed/main.cu:300-383 (BIT-TCF testbed) and the Format-DSL bridge's
 * column_condensed mode (examples/src_fp32/acc/testbed/custom_format_e2e.cu:527-552): tiling and
 * val_sidx as SR-BCRS (tail = the window's last real column); per tile two 64-bit words with bit
 * Swizzle<1,2,3>(8r+c) set for every stored entry (LSB first, main.cu:96-118), the values in
 * ascending bit order padded with zeros to a multiple of 4, val_mco_off[t] = start of tile t's
 * values.  skip_zero_values = 1 is the bridge (entries equal to 0.0f are dropped, :543), 0 the
 * testbed.  val_soff comes from oracle_srbcrs_count; mco_val needs room for nnz + 3T floats.
 * Returns the number of stored values (val_mco_off[T]). */
int64_t oracle_mco_pack(int M, const int* rowptr, const int* colind, const float* values,
                        int skip_zero_values, const int* val_soff, int* val_sidx, int* val_mco_off,
                        uint64_t* val_mco_mask, float* val_mco_val) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int cap = max_window_nnz(M, rowptr);
    int* U = (int*)malloc(sizeof(int) * (size_t)(cap > 0 ? cap : 1));
    int max_nt = 1;
    for (int w = 0; w < W; w++)
        if (val_soff[w + 1] - val_soff[w] > max_nt) max_nt = val_soff[w + 1] - val_soff[w];
    float* tv = (float*)malloc(sizeof(float) * (size_t)max_nt * TILE_ELEMS);
    unsigned char* present = (unsigned char*)malloc((size_t)max_nt * TILE_ELEMS);
    int64_t pos = 0;
    for (int w = 0; w < W; w++) {
        int u = window_unique_cols(M, rowptr, colind, w, U);
        int nt = val_soff[w + 1] - val_soff[w];
        int* sidx = val_sidx + (int64_t)val_soff[w] * TILE_COLS;
        for (int i = 0; i < nt * TILE_COLS; i++) sidx[i] = U[i < u ? i : u - 1];
        memset(present, 0, (size_t)nt * TILE_ELEMS);
        int r0 = w * WIN_ROWS, r1 = r0 + WIN_ROWS;
        if (r1 > M) r1 = M;
        for (int row = r0; row < r1; row++) {
            for (int e = rowptr[row]; e < rowptr[row + 1]; e++) {
                if (skip_zero_values && values[e] == 0.0f) continue;
                int p = lower_bound_int(U, u, colind[e]);
                int at = (p / TILE_COLS) * TILE_ELEMS + sw123((row - r0) * TILE_COLS + p % TILE_COLS);
                present[at] = 1;
                tv[at] = values[e];
            }
        }
        for (int b = 0; b < nt; b++) {
            int t = val_soff[w] + b;
            uint64_t m0 = 0, m1 = 0;
            val_mco_off[t] = (int)pos;
            for (int i = 0; i < TILE_ELEMS; i++) {
                if (!present[b * TILE_ELEMS + i]) continue;
                if (i < 64) m0 |= (uint64_t)1 << i; else m1 |= (uint64_t)1 << (i - 64);
                val_mco_val[pos++] = tv[b * TILE_ELEMS + i];
            }
            while (pos % 4 != 0) val_mco_val[pos++] = 0.0f;
            val_mco_mask[2 * (int64_t)t] = m0;
            val_mco_mask[2 * (int64_t)t + 1] = m1;
        }
    }
    val_mco_off[val_soff[W]] = (int)pos;
    free(U);
    free(tv);
    free(present);
    return pos;
}

/* ---- task planners -----------------------------------------------------------------------
 * Strict load balance (examples/src_fp32/sr_bcrs/testbed/main_strict_lb_16x8.cu:208-256):
 * walk windows in order, cut their tile ranges into fragments so that every group of
 * fragments sums to exactly `workload` tiles (the last group may be short).
 * Two-call protocol: pass NULL arrays to get the counts. Returns the number of fragments. */
int64_t oracle_strict_lb_plan(int M, const int* val_soff, int workload, int* row_block_offset,
                              int* row_block_to_window, int* group_offset, int64_t* n_groups_out) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    int64_t nfrag = 0, ngrp = 0;
    int load = 0;
    if (group_offset) group_offset[0] = 0;
    for (int w = 0; w < W; w++) {
        int s = val_soff[w], e = val_soff[w + 1];
        while (s < e) {
            int take = workload - load;
            if (take > e - s) take = e - s;
            if (row_block_offset) { row_block_offset[nfrag] = s; row_block_to_window[nfrag] = w; }
            nfrag++;
            s += take;
            load += take;
            if (load == workload) {
                ngrp++;
                if (group_offset) group_offset[ngrp] = (int)nfrag;
                load = 0;
            }
        }
    }
    if (row_block_offset) row_block_offset[nfrag] = val_soff[W];
    if (load != 0 || ngrp == 0) {
        ngrp++;
        if (group_offset) group_offset[ngrp] = (int)nfrag;
    }
    *n_groups_out = ngrp;
    return nfrag;
}

/* Multi-binding (examples/src_fp32/sr_bcrs/testbed/main_multi_bind_16x8.cu:207-271): windows
 * with more than 2x the mean tile count (mean over all windows, empty included) are cut into
 * ceil(x/mean) near-equal tasks; empty windows get no task.  Returns the number of tasks.
 * NULL output arrays -> count only. window_split has W entries. */
int64_t oracle_multi_bind_plan(int M, const int* val_soff, int* task_window, int* window_split,
                               int* task_soff) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
    double sum = 0.0;
    for (int w = 0; w < W; w++) sum += (double)(val_soff[w + 1] - val_soff[w]);
    double avg = W > 0 ? sum / (double)W : 0.0;
    int64_t n = 0;
    int acc = 0;
    if (task_soff) task_soff[0] = 0;
    for (int w = 0; w < W; w++) {
        int x = val_soff[w + 1] - val_soff[w];
        if (window_split) window_split[w] = 0;
        if (x == 0) continue;
        int parts = 1;
        if (avg > 0.0 && (double)x > 2.0 * avg) {
            parts = (int)ceil((double)x / avg);
            if (parts > 9999) parts = 9999;
            if (parts < 1) parts = 1;
            if (parts > 1 && window_split) window_split[w] = 1;
        }
        int base = x / parts, rem = x % parts;
        for (int i = 0; i < parts; i++) {
            acc += base + (i < rem ? 1 : 0);
            if (task_window) { task_window[n] = w; task_soff[n + 1] = acc; }
            n++;
        }
    }
    return n;
}

/* ---- numerical oracle --------------------------------------------------------------------
 * Host FP32 SpMM, restating cpu_spmm
 * (examples/src_fp32/csr_tcf/testbed/test_checkpoint.cu:53-67): for every row, for every
 * stored entry in CSR order, C[i,:] += a * B[col,:], FP32 throughout.  `threads` <= 1 runs the
 * loops verbatim on one thread; larger values parallelise over rows (per-row arithmetic and
 * order unchanged, so the result is identical).  Row range [row_begin,row_end) lets callers
 * time a bounded sample. */
void oracle_spmm_f32(int row_begin, int row_end, int N, const int* rowptr, const int* colind,
                     const float* values, const float* B, int64_t ldb, float* C, int64_t ldc,
                     int threads) {
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 64) num_threads(threads)
#endif
    for (int i = row_begin; i < row_end; i++) {
        float* c = C + (int64_t)i * ldc;
        for (int n = 0; n < N; n++) c[n] = 0.0f;
        for (int e = rowptr[i]; e < rowptr[i + 1]; e++) {
            const float a = values[e];
            const float* b = B + (int64_t)colind[e] * ldb;
            for (int n = 0; n < N; n++) c[n] += a * b[n];
        }
    }
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Companion product for the tolerance |C - Cref|_ij <= rtol * (|A|.|B|)_ij + atol,
 * accumulated in FP64. */
void oracle_spmm_abs_f64(int row_begin, int row_end, int N, const int* rowptr, const int* colind,
                         const float* values, const float* B, int64_t ldb, double* Cabs,
                         int64_t ldc, int threads) {
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 64) num_threads(threads)
#endif
    for (int i = row_begin; i < row_end; i++) {
        double* c = Cabs + (int64_t)i * ldc;
        for (int n = 0; n < N; n++) c[n] = 0.0;
        for (int e = rowptr[i]; e < rowptr[i + 1]; e++) {
            const double a = fabs((double)values[e]);
            const float* b = B + (int64_t)colind[e] * ldb;
            for (int n = 0; n < N; n++) c[n] += a * fabs((double)b[n]);
        }
    }
}

/* Round-to-nearest, ties away from zero, to TF32 (10 explicit mantissa bits): what
 * cvt.rna.tf32.f32 does (used on both operands by the reference kernel,
 * examples/src_fp32/sr_bcrs/testbed/kernel.inc:809-814). */
static inline float rna_tf32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) u += 0x1000u;
    u &= 0xffffe000u;
    memcpy(&x, &u, 4);
    return x;
}
float oracle_rna_tf32(float x) { return rna_tf32(x); }

/* SpMM evaluated from the packed SR-BCRS arrays with the kernel's operand rounding:
 * C[16w+r, j] = sum over tiles t of window w (ascending), over c<8 (ascending) of
 * rna(tile_t[r,c]) * rna(B[val_sidx[8t+c], j]), FP32 accumulation.  The order inside one MMA
 * is hardware-defined, so this is a decode/semantics check, not a bit-exact model. */
void oracle_spmm_from_srbcrs(int M, int N, const int* val_soff, const int* val_sidx,
                             const float* val_block_val, const float* B, int64_t ldb, float* C,
                             int64_t ldc, int round_tf32) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
#pragma omp parallel for schedule(dynamic, 16)
    for (int w = 0; w < W; w++) {
        for (int r = 0; r < WIN_ROWS; r++) {
            int row = w * WIN_ROWS + r;
            if (row >= M) break;
            float* c = C + (int64_t)row * ldc;
            for (int n = 0; n < N; n++) c[n] = 0.0f;
            for (int t = val_soff[w]; t < val_soff[w + 1]; t++) {
                for (int k = 0; k < TILE_COLS; k++) {
                    float a = val_block_val[(int64_t)t * TILE_ELEMS + sw223(r * TILE_COLS + k)];
                    if (a == 0.0f) continue;
                    if (round_tf32) a = rna_tf32(a);
                    const float* b = B + (int64_t)val_sidx[(int64_t)t * TILE_COLS + k] * ldb;
                    if (round_tf32) for (int n = 0; n < N; n++) c[n] += a * rna_tf32(b[n]);
                    else for (int n = 0; n < N; n++) c[n] += a * b[n];
                }
            }
        }
    }
}

/* Same from ME-TCF arrays (tile restore semantics of
 * examples/src_fp32/dtc/testbed/kernel.inc:822-840: tile[idx_k] = val_k over the tile's run). */
void oracle_spmm_from_metcf(int M, int N, const int* val_soff, const int* val_sidx,
                            const int* val_coo_off, const int* val_coo_idx, const float* val_coo_val,
                            const float* B, int64_t ldb, float* C, int64_t ldc, int round_tf32) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
#pragma omp parallel for schedule(dynamic, 16)
    for (int w = 0; w < W; w++) {
        float tile[TILE_ELEMS];
        int rows = M - w * WIN_ROWS;
        if (rows > WIN_ROWS) rows = WIN_ROWS;
        for (int r = 0; r < rows; r++) {
            float* c = C + (int64_t)(w * WIN_ROWS + r) * ldc;
            for (int n = 0; n < N; n++) c[n] = 0.0f;
        }
        for (int t = val_soff[w]; t < val_soff[w + 1]; t++) {
            memset(tile, 0, sizeof(tile));
            for (int p = val_coo_off[2 * t]; p < val_coo_off[2 * t + 1]; p++)
                tile[val_coo_idx[p]] = val_coo_val[p];
            for (int r = 0; r < rows; r++) {
                float* c = C + (int64_t)(w * WIN_ROWS + r) * ldc;
                for (int k = 0; k < TILE_COLS; k++) {
                    float a = tile[sw123(r * TILE_COLS + k)];
                    if (a == 0.0f) continue;
                    if (round_tf32) a = rna_tf32(a);
                    const float* b = B + (int64_t)val_sidx[(int64_t)t * TILE_COLS + k] * ldb;
                    if (round_tf32) for (int n = 0; n < N; n++) c[n] += a * rna_tf32(b[n]);
                    else for (int n = 0; n < N; n++) c[n] += a * b[n];
                }
            }
        }
    }
}

/* The product from MCO arrays: tile element (r, k) is stored iff bit Swizzle<1,2,3>(8r+k) is set;
 * its value is number popcount(bits below) of the tile's run. */
void oracle_spmm_from_mco(int M, int N, const int* val_soff, const int* val_sidx, const int* val_mco_off,
                          const uint64_t* val_mco_mask, const float* val_mco_val, const float* B, int64_t ldb,
                          float* C, int64_t ldc, int round_tf32) {
    int W = (M + WIN_ROWS - 1) / WIN_ROWS;
#pragma omp parallel for schedule(dynamic, 16)
    for (int w = 0; w < W; w++) {
        float tile[TILE_ELEMS];
        int rows = M - w * WIN_ROWS;
        if (rows > WIN_ROWS) rows = WIN_ROWS;
        for (int r = 0; r < rows; r++) {
            float* c = C + (int64_t)(w * WIN_ROWS + r) * ldc;
            for (int n = 0; n < N; n++) c[n] = 0.0f;
        }
        for (int t = val_soff[w]; t < val_soff[w + 1]; t++) {
            int at = val_mco_off[t];
            for (int i = 0; i < TILE_ELEMS; i++) {
                uint64_t word = val_mco_mask[2 * (int64_t)t + (i >> 6)];
                tile[i] = ((word >> (i & 63)) & 1) ? val_mco_val[at++] : 0.0f;
            }
            for (int r = 0; r < rows; r++) {
                float* c = C + (int64_t)(w * WIN_ROWS + r) * ldc;
                for (int k = 0; k < TILE_COLS; k++) {
                    float a = tile[sw123(r * TILE_COLS + k)];
                    if (a == 0.0f) continue;
                    if (round_tf32) a = rna_tf32(a);
                    const float* b = B + (int64_t)val_sidx[(int64_t)t * TILE_COLS + k] * ldb;
                    if (round_tf32) for (int n = 0; n < N; n++) c[n] += a * rna_tf32(b[n]);
                    else for (int n = 0; n < N; n++) c[n] += a * b[n];
                }
            }
        }
    }
}

/* Counts elements violating |got - ref| <= rtol*absprod + atol (non-finite counts as a
 * violation); returns the count and writes the worst ratio |got-ref| / (rtol*absprod+atol). */
int64_t oracle_check_tolerance(int64_t rows, int N, const float* got, int64_t ldg, const float* ref,
                               int64_t ldr, const double* absprod, int64_t lda, double rtol,
                               double atol, double* worst_ratio) {
    int64_t bad = 0;
    double worst = 0.0;
#pragma omp parallel for reduction(+ : bad) reduction(max : worst) schedule(static)
    for (int64_t i = 0; i < rows; i++) {
        for (int n = 0; n < N; n++) {
            double g = got[i * ldg + n], r = ref[i * ldr + n];
            double lim = rtol * absprod[i * lda + n] + atol;
            double d = fabs(g - r);
            if (!isfinite(g) || !isfinite(r) || d > lim) bad++;
            if (isfinite(d) && d / lim > worst) worst = d / lim;
        }
    }
    *worst_ratio = worst;
    return bad;
}

/* ---- row reorders of the Format-DSL host bridge ------------------------------------------------
 * Restated from examples/src_fp32/acc/testbed/custom_format_e2e.cu:163-347.  Each returns
 * row_order[new_row] = original_row.  Deterministic tie-breaks are part of the contract. */

static const int* g_sort_key_a;

static const uint64_t* g_sort_key_u;
static int cmp_key_a_then_id(const void* x, const void* y) {
    int l = *(const int*)x, r = *(const int*)y;
    if (g_sort_key_a[l] != g_sort_key_a[r]) return g_sort_key_a[l] < g_sort_key_a[r] ? -1 : 1;
    return (l > r) - (l < r);
}
static int cmp_u_a_then_id(const void* x, const void* y) {
    int l = *(const int*)x, r = *(const int*)y;
    if (g_sort_key_u[l] != g_sort_key_u[r]) return g_sort_key_u[l] < g_sort_key_u[r] ? -1 : 1;
    if (g_sort_key_a[l] != g_sort_key_a[r]) return g_sort_key_a[l] < g_sort_key_a[r] ? -1 : 1;
    return (l > r) - (l < r);
}

static int first_col(int row, int K, const int* rowptr, const int* colind) {
    int first = K;
    for (int p = rowptr[row]; p < rowptr[row + 1]; p++)
        if (colind[p] >= 0 && colind[p] < K && colind[p] < first) first = colind[p];
    return first;
}

/* first_col_sort (custom_format_e2e.cu:233-255): stable order by (first structural column, row). */
void oracle_reorder_first_col(int M, int K, const int* rowptr, const int* colind, int* order) {
    int* first = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    for (int r = 0; r < M; r++) { first[r] = first_col(r, K, rowptr, colind); order[r] = r; }
    g_sort_key_a = first;
    qsort(order, (size_t)M, sizeof(int), cmp_key_a_then_id);  /* total order: ties broken by id */
    free(first);
}

/* row_rcm (custom_format_e2e.cu:163-231): reverse Cuthill-McKee on the symmetrised structure;
 * components started from the unvisited row of least (degree, id); neighbours enqueued in
 * (degree, id) order; every component reversed.  Square matrices only; returns 0 on success. */
int oracle_reorder_rcm(int M, int K, const int* rowptr, const int* colind, int* order) {
    if (M != K) return 1;
    int64_t* cnt = (int64_t*)calloc((size_t)M + 1, sizeof(int64_t));
    for (int r = 0; r < M; r++)
        for (int p = rowptr[r]; p < rowptr[r + 1]; p++) {
            int c = colind[p];
            if (c < 0 || c >= M || c == r) continue;
            cnt[r + 1]++; cnt[c + 1]++;
        }
    for (int r = 0; r < M; r++) cnt[r + 1] += cnt[r];
    int* adj = (int*)malloc(sizeof(int) * (size_t)(cnt[M] > 0 ? cnt[M] : 1));
    int64_t* fill = (int64_t*)malloc(sizeof(int64_t) * (size_t)(M > 0 ? M : 1));
    for (int r = 0; r < M; r++) fill[r] = cnt[r];
    for (int r = 0; r < M; r++)
        for (int p = rowptr[r]; p < rowptr[r + 1]; p++) {
            int c = colind[p];
            if (c < 0 || c >= M || c == r) continue;
            adj[fill[r]++] = c; adj[fill[c]++] = r;
        }
    int64_t* abeg = (int64_t*)malloc(sizeof(int64_t) * (size_t)(M + 1));
    int* degree = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    for (int r = 0; r < M; r++) {  /* sort + unique each neighbour list */
        int* a = adj + cnt[r];
        int n = (int)(cnt[r + 1] - cnt[r]);
        qsort(a, (size_t)n, sizeof(int), cmp_int);
        int u = 0;
        for (int i = 0; i < n; i++) if (i == 0 || a[i] != a[u - 1]) a[u++] = a[i];
        degree[r] = u;
        abeg[r] = cnt[r];
    }
    int* starts = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    for (int r = 0; r < M; r++) starts[r] = r;
    g_sort_key_a = degree;
    qsort(starts, (size_t)M, sizeof(int), cmp_key_a_then_id);
    unsigned char* visited = (unsigned char*)calloc((size_t)(M > 0 ? M : 1), 1);
    int* queue = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    int* next = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    int out = 0;
    for (int si = 0; si < M; si++) {
        int start = starts[si];
        if (visited[start]) continue;
        int qh = 0, qt = 0, comp_begin = out;
        visited[start] = 1;
        queue[qt++] = start;
        while (qh < qt) {
            int row = queue[qh++];
            order[out++] = row;
            int nn = 0;
            for (int i = 0; i < degree[row]; i++) {
                int nb = adj[abeg[row] + i];
                if (!visited[nb]) next[nn++] = nb;
            }
            qsort(next, (size_t)nn, sizeof(int), cmp_key_a_then_id);
            for (int i = 0; i < nn; i++)
                if (!visited[next[i]]) { visited[next[i]] = 1; queue[qt++] = next[i]; }
        }
        for (int i = comp_begin, j = out - 1; i < j; i++, j--) { int t = order[i]; order[i] = order[j]; order[j] = t; }
    }
    free(cnt); free(adj); free(fill); free(abeg); free(degree); free(starts); free(visited); free(queue); free(next);
    return out == M ? 0 : 2;
}

static uint64_t mix_column(uint64_t v) {
    v += 0x9e3779b97f4a7c15ULL;
    v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ULL;
    v = (v ^ (v >> 27)) * 0x94d049bb133111ebULL;
    return v ^ (v >> 31);
}

static double row_jaccard(int l, int r, const int* rowptr, const int* colind) {
    int a = rowptr[l], b = rowptr[r];
    const int ae = rowptr[l + 1], be = rowptr[r + 1];
    int inter = 0, lu = 0, ru = 0;
    while (a < ae || b < be) {
        const int lc = a < ae ? colind[a] : 2147483647, rc = b < be ? colind[b] : 2147483647;
        if (lc == rc) { inter++; lu++; ru++; while (a < ae && colind[a] == lc) a++; while (b < be && colind[b] == rc) b++; }
        else if (lc < rc) { lu++; while (a < ae && colind[a] == lc) a++; }
        else { ru++; while (b < be && colind[b] == rc) b++; }
    }
    const int uni = lu + ru - inter;
    return uni ? (double)inter / uni : 1.0;
}

/* jaccard_greedy (custom_format_e2e.cu:257-347): rows ranked by (min-hash of their columns, first
 * column, id), cut into buckets of 64 consecutive ranks; inside a bucket, starting from its first
 * row, repeatedly append the remaining row with the largest exact Jaccard similarity to the row
 * appended last (ties: smaller row id). */
void oracle_reorder_jaccard(int M, int K, const int* rowptr, const int* colind, int* order) {
    uint64_t* sig = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(M > 0 ? M : 1));
    int* first = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    int* ranked = (int*)malloc(sizeof(int) * (size_t)(M > 0 ? M : 1));
    for (int r = 0; r < M; r++) {
        uint64_t s = UINT64_MAX;
        for (int p = rowptr[r]; p < rowptr[r + 1]; p++) {
            uint64_t h = mix_column((uint64_t)(uint32_t)colind[p]);
            if (h < s) s = h;
        }
        sig[r] = s; first[r] = first_col(r, K, rowptr, colind); ranked[r] = r;
    }
    g_sort_key_u = sig; g_sort_key_a = first;
    qsort(ranked, (size_t)M, sizeof(int), cmp_u_a_then_id);
    int out = 0;
    int rem[64];
    for (int base = 0; base < M; base += 64) {
        int n = M - base < 64 ? M - base : 64;
        memcpy(rem, ranked + base, sizeof(int) * (size_t)n);
        int cur = rem[0];
        order[out++] = cur;
        memmove(rem, rem + 1, sizeof(int) * (size_t)(--n));
        while (n > 0) {
            int best = 0;
            double best_score = -1.0;
            for (int c = 0; c < n; c++) {
                double s = row_jaccard(cur, rem[c], rowptr, colind);
                if (s > best_score || (s == best_score && rem[c] < rem[best])) { best_score = s; best = c; }
            }
            cur = rem[best];
            order[out++] = cur;
            memmove(rem + best, rem + best + 1, sizeof(int) * (size_t)(n - best - 1));
            n--;
        }
    }
    free(sig); free(first); free(ranked);
}

/* Rows of a CSR matrix taken in `order` (new_row -> original_row): the input of the packers after
 * a reorder (custom_format_e2e.cu:554-568 walks rows through row_order the same way). */
void oracle_permute_csr(int M, const int* rowptr, const int* colind, const float* values, const int* order,
                        int* rowptr_out, int* colind_out, float* values_out) {
    rowptr_out[0] = 0;
    for (int i = 0; i < M; i++) {
        const int r = order[i], n = rowptr[r + 1] - rowptr[r];
        memcpy(colind_out + rowptr_out[i], colind + rowptr[r], sizeof(int) * (size_t)n);
        memcpy(values_out + rowptr_out[i], values + rowptr[r], sizeof(float) * (size_t)n);
        rowptr_out[i + 1] = rowptr_out[i] + n;
    }
}
