/*
 * mask_b200 -- C ABI of the B200 (sm_100a) SpMM engine for the SR-BCRS 16x8 and ME-TCF formats.
 *
 * C = A * B with A sparse FP32 packed into dense 16x8 tiles of window-condensed columns,
 * B dense FP32 row-major with N columns, TF32 tensor-core products (both operands rounded to
 * nearest, ties away, like cvt.rna.tf32.f32) and FP32 accumulation.
 *
 * Conventions
 *   - every function returns a mask_status (0 = success); nothing throws or aborts;
 *     mask_last_error() gives a per-thread message for the last failure.
 *   - pointers named d_* are device pointers on the current CUDA device, h_* are host pointers.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - sizes that can pass 2^31 (tile counts times 128, M*N) are 64-bit.
 *   - W = ceil(M/16) row windows, T = number of 16x8 tiles.
 *
 * Each entry point cites the interface of the reference project (hd9568/MASK) that it replaces,
 * as a path inside that project.
 */
#ifndef MASK_B200_H_
#define MASK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mask_status {
    MASK_OK = 0,
    MASK_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, N not a multiple of 4, ... */
    MASK_ERR_CUDA = 2,             /* a CUDA runtime call failed; see mask_last_error() */
    MASK_ERR_UNSORTED_ROWS = 3,    /* CSR rows must hold strictly ascending column ids */
    MASK_ERR_SCRATCH_TOO_SMALL = 4,
    MASK_ERR_INDEX_OVERFLOW = 5,   /* a count does not fit the int32 index arrays of the format */
    MASK_ERR_COLUMN_RANGE = 6,     /* a column id is outside [0, K) */
    MASK_ERR_NO_DEVICE = 7,
    MASK_ERR_KERNEL_TIMEOUT = 8    /* a kernel gave up on one of its bounded waits: the output is invalid */
} mask_status;

int mask_version(void);
const char* mask_status_string(int status);
const char* mask_last_error(void);

/* ------------------------------------------------------------------------------------------
 * Format builder (device).  Replaces the host packers convertToSRBCRS
 * (examples/src_fp32/sr_bcrs/testbed/main_16x8.cu:196-328), its extension twin
 * preprocess_gpu_srcfp32_srbcrs (examples/src_fp32/sr_bcrs/testbed/SRBCRSSpMM_kernel.cu:172-393)
 * and buildMETCFMetadata (examples/src_fp32/dtc/testbed/main.cu:352-520).  Output arrays are
 * bit-identical to those packers' for CSR input with strictly ascending rows.
 *
 * Protocol: analyze (window column condensation, gives T) -> caller allocates the packed arrays
 * -> fill.  The scratch buffer carries the analysis between the calls and must not be touched
 * in between.
 * ------------------------------------------------------------------------------------------ */

/* Bytes of scratch needed by mask_pack_analyze for a matrix with M rows and nnz entries. */
size_t mask_pack_scratch_bytes(int32_t M, int64_t nnz);

/* Window column condensation (main_16x8.cu:209-251): writes val_soff[W+1] (exclusive scan of
 * tiles per window) and returns T through *h_T.  Synchronises the stream. */
int mask_pack_analyze(const int32_t* d_rowptr, const int32_t* d_colind, int32_t M, int32_t K,
                      int64_t nnz, void* d_scratch, size_t scratch_bytes, int32_t* d_val_soff,
                      int64_t* h_T, void* stream);

/* SR-BCRS 16x8 arrays (main_16x8.cu:288-318): val_sidx[8T] (tail slots of a window repeat its
 * last real column), val_block_val[128T] (tile t, element (r,c) at 128t + Swizzle<2,2,3>(8r+c),
 * zeros elsewhere).  Optional side outputs of the extension packer
 * (SRBCRSSpMM_kernel.cu:241,250,268), each may be NULL: block_partition[W] = tiles per window,
 * edge_to_col[nnz] = condensed position of each entry, edge_to_row[nnz] = its row. */
int mask_srbcrs_fill(const int32_t* d_rowptr, const int32_t* d_colind, const float* d_values,
                     int32_t M, int64_t nnz, const void* d_scratch, const int32_t* d_val_soff,
                     int64_t T, int32_t* d_val_sidx, float* d_val_block_val,
                     int32_t* d_block_partition, int32_t* d_edge_to_col, int32_t* d_edge_to_row,
                     void* stream);

/* ME-TCF, step 1 (main.cu:393-453): val_coo_off[2T+1] ([begin, begin+count] per tile, runs
 * padded to 8, closing entry nnz_pad); returns nnz_pad through *h_nnz_pad.  d_tile_rows is
 * caller-provided scratch of T 64-bit words, consumed by mask_metcf_fill.  Synchronises. */
int mask_metcf_offsets(const int32_t* d_rowptr, int32_t M, int64_t nnz, const void* d_scratch,
                       const int32_t* d_val_soff, int64_t T, int32_t* d_val_coo_off,
                       uint64_t* d_tile_rows, int64_t* h_nnz_pad, void* stream);

/* ME-TCF, step 2 (main.cu:455-517): val_sidx[8T] (tail slots 0), val_coo_idx[nnz_pad]
 * (Swizzle<1,2,3>(8r+c)), val_coo_val[nnz_pad]; entries of a tile ordered by row, then CSR
 * order; padding slots idx 0 / value 0.  d_values may be NULL: every stored entry then gets
 * the value 1.0f, which is what the reference extension packer writes
 * (examples/src_fp32/dtc/testbed/DTCSpMM_kernel.cu:450). */
int mask_metcf_fill(const int32_t* d_rowptr, const int32_t* d_colind, const float* d_values,
                    int32_t M, int64_t nnz, const void* d_scratch, const int32_t* d_val_soff,
                    int64_t T, const int32_t* d_val_coo_off, const uint64_t* d_tile_rows,
                    int64_t nnz_pad, int32_t* d_val_sidx, int32_t* d_val_coo_idx,
                    float* d_val_coo_val, void* stream);

/* MCO / BIT-TCF (bitmap leaf): the tiling and val_sidx of SR-BCRS (window tail padded with the last
 * real column); per tile two 64-bit mask words, bit Swizzle<1,2,3>(8r+c) set for a stored entry,
 * and the entries' values in ascending bit order, each tile's run padded with zeros to a multiple
 * of 4; val_mco_off[T+1] = start of every tile's run.  Replaces the host packers
 * examples/src_fp32/acc/testbed/main.cu:300-383 (BIT-TCF testbed; skip_zero_values = 0: explicit
 * zeros are stored) and the Format-DSL bridge's "column_condensed" mode
 * (examples/src_fp32/acc/testbed/custom_format_e2e.cu:527-552; skip_zero_values = 1).  After
 * mask_pack_analyze with the same scratch.  Step 1 writes val_mco_mask[2T] and val_mco_off[T+1]
 * and returns the total value count through *h_nval (synchronises); step 2 writes val_sidx[8T]
 * and val_mco_val[nval].  d_values may be NULL (every entry 1.0f). */
int mask_mco_offsets(const float* d_values, int32_t M, int64_t nnz, const void* d_scratch,
                     const int32_t* d_val_soff, int64_t T, int skip_zero_values,
                     uint64_t* d_val_mco_mask, int32_t* d_val_mco_off, int64_t* h_nval, void* stream);
int mask_mco_fill(const int32_t* d_rowptr, const float* d_values, int32_t M, int64_t nnz,
                  const void* d_scratch, const int32_t* d_val_soff, int64_t T, int skip_zero_values,
                  const uint64_t* d_val_mco_mask, const int32_t* d_val_mco_off, int64_t nval,
                  int32_t* d_val_sidx, float* d_val_mco_val, void* stream);

/* ------------------------------------------------------------------------------------------
 * Row reorders of the Format-DSL host bridge (examples/src_fp32/acc/testbed/custom_format_e2e.cu:
 * 163-347): reverse_cuthill_mckee, first_column_order, jaccard_greedy_order, with the same
 * tie-breaks, so the orders are bit-identical.  d_row_order[new_row] = original_row.  Computed on
 * the device from a device CSR matrix (rows strictly ascending, the packers' contract); the call
 * allocates its scratch itself and synchronises the stream before it returns.
 * ------------------------------------------------------------------------------------------ */
typedef enum mask_reorder {
    MASK_REORDER_NONE = 0,
    MASK_REORDER_ROW_RCM = 1,        /* square matrices only */
    MASK_REORDER_FIRST_COL_SORT = 2,
    MASK_REORDER_JACCARD_GREEDY = 3
} mask_reorder;

int mask_reorder_rows(int kind, const int32_t* d_rowptr, const int32_t* d_colind, int32_t M,
                      int32_t K, int32_t* d_row_order, void* stream);

/* Applies an order on the device: row i of the output CSR is row d_row_order[i] of the input
 * (what the bridge's packer does while walking row_order, custom_format_e2e.cu:554-568).
 * d_rowptr_out has M+1 entries; the colind / values pairs may be NULL to get row pointers only. */
int mask_csr_permute_rows(const int32_t* d_rowptr, const int32_t* d_colind, const float* d_values,
                          int32_t M, const int32_t* d_row_order, int32_t* d_rowptr_out,
                          int32_t* d_colind_out, float* d_values_out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Task planners (host, pure functions).  Bit-identical to strict_load_balance
 * (examples/src_fp32/sr_bcrs/testbed/main_strict_lb_16x8.cu:208-256) and
 * multi_binding_load_balance (examples/src_fp32/sr_bcrs/testbed/main_multi_bind_16x8.cu:207-271).
 * Call with NULL output arrays to get the counts, then again with arrays of that size.
 * ------------------------------------------------------------------------------------------ */

/* Fragments of consecutive tiles such that every group sums to exactly `workload` tiles.
 * row_block_offset[F+1], row_block_to_window[F], group_offset[G+1]. Returns F via *n_frag. */
int mask_plan_strict_lb(const int32_t* h_val_soff, int32_t M, int32_t workload,
                        int32_t* row_block_offset, int32_t* row_block_to_window,
                        int32_t* group_offset, int64_t* n_frag, int64_t* n_groups);

/* Windows with more than twice the mean tile count are cut into ceil(x/mean) near-equal tasks.
 * task_window[P], window_split[W], task_soff[P+1]. */
int mask_plan_multi_bind(const int32_t* h_val_soff, int32_t M, int32_t* task_window,
                         int32_t* window_split, int32_t* task_soff, int64_t* n_tasks);

/* ------------------------------------------------------------------------------------------
 * Matrix features the execution plan is chosen from (the reference derives a larger set in
 * examples/src_fp32/dtc/testbed/featurize_mtx.cu:298-401; these are the ones that drive a
 * decision here).  Percentiles use the bridge's rank rule, heavy_tail is its test
 * tiles_max > max(64, 4 * p95) (examples/src_fp32/acc/testbed/custom_format_e2e.cu:652-663).
 * ------------------------------------------------------------------------------------------ */
typedef struct mask_features {
    int32_t row_windows;
    int32_t empty_windows;
    int64_t tiles;
    int64_t nnz;
    double tiles_mean;
    int32_t tiles_p50, tiles_p95, tiles_p99, tiles_max;
    double top5_window_share; /* share of all tiles held by the 5 largest windows */
    double tile_fill;         /* nnz / (128 * tiles) */
    int32_t heavy_tail;
} mask_features;

int mask_features_from_soff(const int32_t* h_val_soff, int32_t M, int64_t nnz, mask_features* out);

/* Column-side features, computed on the device from val_sidx (8 T gathered ids): what the rows of
 * B the product gathers look like to the L2.  Same role as the column statistics of the
 * reference's featurizer (unique columns per window, entries per unique column,
 * examples/src_fp32/dtc/testbed/featurize_mtx.cu:298-401), extended by what a B200 plan needs. */
typedef struct mask_column_features {
    int64_t gathers;          /* 8 T: rows of B fetched per sweep of the matrix */
    int32_t distinct_columns; /* columns that hold an entry = rows of B the product touches */
    int32_t band_p50, band_p90; /* distance of a gathered row from the diagonal position of its window
                                   (rows of B), percentiles over all gathers, rounded up to a power of 2 */
    int32_t hub_columns[3];   /* how many rows of B fit half the L2 at row widths of min(N,512), min(N,256), min(N,128) columns */
    double hub_share[3];      /* share of all gathers that go to that many most gathered columns */
    int32_t l2_bytes;
    int32_t local_rows;       /* half-width of the band whose rows of B (min(N,512) columns wide) fill half the L2 */
    double local_share;       /* share of all gathers within local_rows of their window's diagonal position */
} mask_column_features;
int mask_features_columns(const int32_t* d_val_soff, const int32_t* d_val_sidx, int32_t M, int32_t K, int64_t T,
                          int32_t N, mask_column_features* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * ME-TCF packed-format cache file, byte-compatible with the reference's storeCheckpoint /
 * loadCheckpoint (examples/src_fp32/dtc/testbed/main.cu:217-340): raw little-endian
 * [T][nnz_pad][val_soff][val_sidx][val_coo_off][val_coo_idx][val_coo_val]; host arrays.
 * ------------------------------------------------------------------------------------------ */
/* File name for a matrix known by name (the stem of its file). */
int mask_metcf_checkpoint_name(const char* matrix_name, int32_t M, int32_t K, char* out, size_t out_len);
/* File name exactly as the reference testbed derives it from the path it was given
 * (buildCheckpointStem, main.cu:205-230): stem of `file_path`, or for an empty path (matrix
 * generated in memory) "synthetic..._sp<sparsity token>". */
int mask_metcf_checkpoint_name_for(const char* file_path, int32_t M, int32_t K, float sparsity, char* out, size_t out_len);
int mask_metcf_checkpoint_write(const char* path, int32_t M, int64_t T, int64_t nnz_pad,
                                const int32_t* val_soff, const int32_t* val_sidx,
                                const int32_t* val_coo_off, const int32_t* val_coo_idx,
                                const float* val_coo_val);
int mask_metcf_checkpoint_header(const char* path, int64_t* T, int64_t* nnz_pad);
/* Arrays sized from the header; validates sizes, offsets and column range like the reference. */
int mask_metcf_checkpoint_read(const char* path, int32_t M, int32_t K, int64_t T, int64_t nnz_pad,
                               int32_t* val_soff, int32_t* val_sidx, int32_t* val_coo_off,
                               int32_t* val_coo_idx, float* val_coo_val);

/* ------------------------------------------------------------------------------------------
 * Execution plan: how tiles are dealt to thread blocks.  Replaces the grid mapping of the
 * reference kernels (one block per window, examples/src_fp32/sr_bcrs/testbed/host_program_16x8.cu:
 * 157-159; strict_lb / multi_bind tables, host_program_strict_lb.cu:163-289).
 * ------------------------------------------------------------------------------------------ */
typedef struct mask_plan mask_plan;

typedef enum mask_policy {
    MASK_POLICY_AUTO = 0,      /* window-aligned groups; windows larger than a group are split */
    MASK_POLICY_ROW = 1,       /* one task per window, never split */
    MASK_POLICY_STRICT_LB = 2, /* the reference's strict_lb tables (exact `group_tiles` per block) */
    MASK_POLICY_MULTI_BIND = 3, /* the reference's multi_bind tables */
    MASK_POLICY_REF_AUTO = 4    /* the bridge's rule: strict_lb if the tile distribution is heavy-tailed,
                                   else row (custom_format_e2e.cu:659-707) */
} mask_policy;

/* Builds a plan from val_soff (device).  group_tiles <= 0 picks a default from T and the SM
 * count.  Allocates small device arrays owned by the plan; synchronises the stream. */
int mask_plan_create(const int32_t* d_val_soff, int32_t M, int64_t T, int policy,
                     int32_t group_tiles, void* stream, mask_plan** out);
void mask_plan_destroy(mask_plan* plan);
/* Scratch bytes mask_spmm_* needs with this plan for an N-column product (0 if no window is
 * split). */
size_t mask_plan_scratch_bytes(const mask_plan* plan, int32_t N);
/* Introspection for tests: numbers of fragments, groups, split fragments, and the group size. */
int mask_plan_info(const mask_plan* plan, int64_t* n_frag, int64_t* n_groups, int64_t* n_partial,
                   int32_t* group_tiles);
/* Makes every SpMM launched with this plan write packed row i to output row d_row_order[i]
 * (NULL = identity): a matrix packed from reordered rows then produces C in the original row
 * order with no separate pass.  Replaces the bridge's host-side unpack_output
 * (custom_format_e2e.cu:1083-1100).  The array (M entries) is not owned by the plan. */
int mask_plan_set_row_map(mask_plan* plan, const int32_t* d_row_order);
/* Fused SpMM + all-gather for row-sharded multi-GPU use: every SpMM launched with this plan also
 * stores each finished output row into n_peers more buffers (d_peer_ptrs is a device array of
 * their bases, laid out like d_C; at most 15; NULL / 0 switches it off).  With peer-mapped
 * buffers of the other GPUs (plain P2P stores over NVLink) each rank's panel of C lands in every
 * rank's full copy while the product is still running, and no separate collective is needed:
 * only a barrier after the kernels.  The reference is single-GPU and has no counterpart.  The
 * pointer array is not owned by the plan. */
int mask_plan_set_peer_outputs(mask_plan* plan, float* const* d_peer_ptrs, int32_t n_peers);
/* Buffers for d_peer_ptrs when every GPU has its own process (no counterpart in the reference).
 * mask_peer_alloc: one cudaMalloc on the current device plus its CUDA IPC handle
 * (MASK_PEER_HANDLE_BYTES bytes, to be sent to the other processes by the host program's own
 * channel).  mask_peer_open, in another process of the same machine: maps that buffer for the
 * current device (peer access is switched on as needed) and returns its address there.  Close
 * every mapping (mask_peer_close) before the owner frees the buffer (mask_peer_free). */
#define MASK_PEER_HANDLE_BYTES 64
int mask_peer_alloc(size_t bytes, void** d_ptr, void* handle);
int mask_peer_open(const void* handle, void** d_ptr);
int mask_peer_close(void* d_ptr);
int mask_peer_free(void* d_ptr);
/* The plan table: computes the column features of the packed matrix (device) and sets the plan's
 * kernel parameters from them -- today the number of 128-column slabs a resident block sweeps at
 * a time (4: tile values and ids read once, for matrices whose gathers are local; 2: narrower rows
 * of B, for large power-law matrices where that lets the L2 serve more of the gathers).  Replaces
 * the knobs the reference hands to its strategy agent (python/sparsene/op_gen/strategy_agent.py:
 * 414-528).  Without this call a plan uses the widest block N fills.  Synchronises the stream.
 * mask_plan_column_features returns what was measured and chosen. */
int mask_plan_autotune(mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx, int32_t K, void* stream);
int mask_plan_column_features(const mask_plan* plan, mask_column_features* out, int32_t* nslab_wide);
/* Prepares the plan for the TMA-fed SpMM kernel: keeps a copy of val_block_val (128 T floats, owned
 * by the plan) with every value rounded to TF32 -- nearest, ties away, the reference kernels'
 * cvt.rna (examples/src_fp32/sr_bcrs/testbed/kernel.inc:809-814) done once per matrix instead of
 * once per use.  mask_spmm_srbcrs then takes its fastest path whenever it is called with the same
 * val_block_val pointer; with another pointer, or a plan that was not prepared, it runs the
 * copy-based kernel, which rounds on the fly.  Call it again after changing the values in place;
 * NULL drops the copy.  Allocates (cudaMalloc) and enqueues one kernel on `stream`. */
int mask_plan_prepare_values(mask_plan* plan, const float* d_val_block_val, void* stream);
/* Reads AND CLEARS the plan's device status word (synchronises the stream): 0, or non-zero if a
 * kernel launched with this plan since the last call gave up on one of its bounded waits (its
 * output is then invalid; the kernel has drained its copies and tensor-core work and freed its
 * tensor memory, so the context stays usable).  The device-pointer SpMM entry points are
 * asynchronous and cannot report this themselves: call this wherever the host synchronises anyway.
 * mask_session_spmm_host does so itself and returns MASK_ERR_KERNEL_TIMEOUT.  No counterpart in the
 * reference, whose kernels have no waits. */
int mask_plan_status(const mask_plan* plan, int32_t* h_status, void* stream);
/* Copies the plan tables to host arrays (frag_offset[F+1], frag_window[F], group_offset[G+1]). */
int mask_plan_export(const mask_plan* plan, int32_t* frag_offset, int32_t* frag_window,
                     int32_t* group_offset);

/* ------------------------------------------------------------------------------------------
 * SpMM.  Replaces sr_bcrs_spmm_kernel_tf32 and its load-balanced variants
 * (examples/src_fp32/sr_bcrs/testbed/kernel.inc:1590-1700, kernel_lb.inc:62-381) and
 * dtc_spmm_kernel_fp32_val_idx_bind_stage2 (examples/src_fp32/dtc/testbed/kernel.inc:1982-2134).
 *
 * C[M,N] (leading dimension ldc) is fully overwritten -- no zero-fill by the caller and no
 * atomics: windows split across blocks are summed in tile order from per-fragment partial
 * tiles in d_scratch, so results are run-to-run deterministic.  B is [K,N] with leading
 * dimension ldb.  Requirements: N % 4 == 0, ldb % 4 == 0, ldc % 4 == 0, 16-byte aligned B and C.
 * ------------------------------------------------------------------------------------------ */
#define MASK_EPILOGUE_NONE 0
#define MASK_EPILOGUE_RELU 1 /* C = max(A*B, 0), used between GCN layers */
/* OR-able into `epilogue` (SR-BCRS only): three TF32 products per MMA -- hi(A)*hi(B) plus the
 * residual terms lo(A)*hi(B) and hi(A)*lo(B) -- which brings the result to FP32-level accuracy
 * (the reference compiler's compensated MMA, python/sparsene/op_gen/nvir/templates.py:53-76, on
 * by default in its Format-DSL bridge).  Runs on the mma.sync ring kernel; 5.2 ms against 3.1 ms on
 * the 2^20-node power-law graph at N = 512. */
#define MASK_NUMERICS_TF32X3 0x100

int mask_spmm_srbcrs(const mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx,
                     const float* d_val_block_val, int32_t M, int32_t K, int32_t N,
                     const float* d_B, int64_t ldb, float* d_C, int64_t ldc, void* d_scratch,
                     size_t scratch_bytes, int epilogue, void* stream);

int mask_spmm_metcf(const mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx,
                    const int32_t* d_val_coo_off, const int32_t* d_val_coo_idx,
                    const float* d_val_coo_val, int32_t M, int32_t K, int32_t N, const float* d_B,
                    int64_t ldb, float* d_C, int64_t ldc, void* d_scratch, size_t scratch_bytes,
                    int epilogue, void* stream);

/* MCO / BIT-TCF SpMM: same contract; replaces acc_spmm_kernel_tf32tf32fp32
 * (examples/src_fp32/acc/testbed/kernel.inc:1947) and the bridge's bitmap operators.  The tile operand is expanded from its mask and
 * compact values in shared memory.  val_mco_mask and val_mco_val must be 16-byte aligned. */
int mask_spmm_mco(const mask_plan* plan, const int32_t* d_val_soff, const int32_t* d_val_sidx,
                  const int32_t* d_val_mco_off, const uint64_t* d_val_mco_mask,
                  const float* d_val_mco_val, int32_t M, int32_t K, int32_t N, const float* d_B,
                  int64_t ldb, float* d_C, int64_t ldc, void* d_scratch, size_t scratch_bytes,
                  int epilogue, void* stream);

/* SR-BCRS SpMM for callers that are not allowed to allocate device memory -- a process whose
 * whole device heap belongs to an arena of its own (an inference server, an engine that loads this
 * library as a plug-in) or a loop that cannot afford the device-wide synchronisation of
 * cudaMalloc/cudaFree.  It has NO COUNTERPART IN THE REFERENCE PROJECT.  Same arguments and result
 * as mask_spmm_srbcrs minus the scratch buffer: the partial tiles of split windows go to a fixed
 * 32 MiB array inside the library's device image (mask_static_scratch_capacity() bytes; every GPU
 * that loads the library keeps it until the process exits).  The call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 *   - A plan whose partial tiles for this N exceed the capacity (mask_plan_scratch_bytes(plan, N)
 *     > capacity; 1024 partial tiles at N = 512) is refused with MASK_ERR_SCRATCH_TOO_SMALL and
 *     nothing is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call during start-up,
 *     before any stream capture begins.  The address is remembered per device ordinal for the
 *     device's primary context; it is not valid after cudaDeviceReset or under another context on
 *     the same ordinal.
 *   - All calls on a device share the one array and it keeps whatever the last call left in it.
 *     Nothing in it needs clearing between calls (each call writes every partial tile before
 *     reading it), but two calls that overlap on the GPU -- different streams, or different
 *     threads -- race on it: serialise them, or give the others mask_spmm_srbcrs with their own
 *     buffer. */
size_t mask_static_scratch_capacity(void);
int mask_spmm_srbcrs_static_scratch(const mask_plan* plan, const int32_t* d_val_soff,
                                    const int32_t* d_val_sidx, const float* d_val_block_val,
                                    int32_t M, int32_t K, int32_t N, const float* d_B, int64_t ldb,
                                    float* d_C, int64_t ldc, int epilogue, void* stream);

/* Development knobs for kernel variants, process-wide: "sweep" (1 = persistent tcgen05 kernel except
 * where the warp-level one measures faster (N < 80), 2 = always, 0 = warp-level kernels only),
 * "nslab" (tcgen05 kernel: 128-column slabs per sweep, 1 / 2 / 4; 0 = the plan table's choice),
 * "tma" (1 = the TMA-fed kernel for plans prepared with mask_plan_prepare_values), and for the
 * warp-level kernels "nq" (32-column groups per warp: 1, 2, 4; 0 = chosen from N), "min_blocks"
 * (occupancy target; 0 = default), "async" (0 = register-pipelined kernel instead of the cp.async
 * ring), "stages" (ring depth); "session_chunk" (columns per chunk of mask_session_spmm_host).
 * Replaces the reference's tile_b environment switches SRBCRS_TILE_B / DTC_TILE_B
 * (examples/src_fp32/sr_bcrs/testbed/SRBCRSSpMM_kernel.cu:435-475). */
int mask_tune(const char* name, int value);

/* Which kernel the SpMM entry points launch for a plan, an encoding (0 SR-BCRS, 1 ME-TCF, 2 MCO), N
 * and an epilogue argument, as text ("spmm_sweep_kernel<nslab=4,srbcrs>"), and a number that
 * changes whenever the library's main kernel changes in a way that affects its memory traffic
 * (measurement harnesses pair captured profiler figures with it).  No counterpart in the
 * reference. */
int mask_spmm_kernel_name(const mask_plan* plan, int format, int32_t N, int epilogue, char* out, size_t capacity);
int mask_kernel_revision(void);

/* cudaMemcpy2DAsync behind the C ABI, for hosts that drive their own upload / product / download
 * pipeline over column chunks of row-major host matrices (kind: 1 = host to device, 2 = device to
 * host, 3 = device to device).  Pitches and width in bytes.  No counterpart in the reference. */
int mask_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                       size_t rows, int kind, void* stream);

/* ------------------------------------------------------------------------------------------
 * Host-buffer seam.  Replaces the testbed entry sr_bcrs_test_tf32<16,64,8>
 * (examples/src_fp32/sr_bcrs/testbed/main_16x8.cu:32-44, host_program_16x8.cu:118-191): packed
 * arrays, B and C are HOST pointers; the call uploads, runs once and downloads C.  A session
 * keeps the packed matrix and the plan on the device between calls, like the extension's module
 * cache (SRBCRSSpMM_kernel.cu:27-45), so a repeated product moves only B and C.
 * ------------------------------------------------------------------------------------------ */
typedef struct mask_session mask_session;

int mask_session_create_srbcrs(int32_t M, int32_t K, int64_t T, const int32_t* h_val_soff,
                               const int32_t* h_val_sidx, const float* h_val_block_val, int policy,
                               mask_session** out);
/* From CSR on the host: uploads, packs on the device, plans. */
int mask_session_create_csr(int32_t M, int32_t K, int64_t nnz, const int32_t* h_rowptr,
                            const int32_t* h_colind, const float* h_values, int policy,
                            mask_session** out);
/* C_host[M,N] = A * B_host[K,N]; pinned host buffers make the copies asynchronous.  kernel_ms,
 * if not NULL, receives the device time of the SpMM kernels alone.  When N is a multiple of 128
 * and at least 256 the product is cut into column chunks (independent products) whose upload,
 * multiplication and download overlap on three streams, so both directions of the host link are
 * busy at once; mask_tune("session_chunk", columns | 0 = off | -1 = automatic) overrides. */
int mask_session_spmm_host(mask_session* s, const float* h_B, float* h_C, int32_t N,
                           float* kernel_ms);
int64_t mask_session_tiles(const mask_session* s);
void mask_session_destroy(mask_session* s);

#ifdef __cplusplus
}
#endif
#endif /* MASK_B200_H_ */
