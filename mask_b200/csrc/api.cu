// Status reporting and the host-buffer session seam of the C ABI.
#include <cstdarg>
#include <cstring>

#include "common.cuh"
#include "plan.h"

namespace mask {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

}  // namespace mask

extern "C" int mask_version(void) { return 100; }

extern "C" const char* mask_last_error(void) { return mask::g_error; }

extern "C" int mask_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                                  size_t rows, int kind, void* stream) {
    using namespace mask;
    MASK_REQUIRE(dst != nullptr && src != nullptr, "NULL pointer");
    MASK_REQUIRE(kind >= 1 && kind <= 3, "kind must be 1 (host to device), 2 (device to host) or 3 (device to device)");
    MASK_REQUIRE(width_bytes <= dst_pitch && width_bytes <= src_pitch, "width exceeds a pitch");
    if (width_bytes == 0 || rows == 0) return MASK_OK;
    const cudaMemcpyKind k = kind == 1 ? cudaMemcpyHostToDevice : (kind == 2 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice);
    MASK_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, k, static_cast<cudaStream_t>(stream)));
    return MASK_OK;
}

extern "C" const char* mask_status_string(int status) {
    switch (status) {
        case MASK_OK: return "ok";
        case MASK_ERR_INVALID_ARGUMENT: return "invalid argument";
        case MASK_ERR_CUDA: return "CUDA error";
        case MASK_ERR_UNSORTED_ROWS: return "CSR rows are not strictly ascending";
        case MASK_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small";
        case MASK_ERR_INDEX_OVERFLOW: return "count does not fit the format's int32 indices";
        case MASK_ERR_COLUMN_RANGE: return "column id out of range";
        case MASK_ERR_NO_DEVICE: return "no CUDA device";
        case MASK_ERR_KERNEL_TIMEOUT: return "a kernel gave up on a bounded wait";
        default: return "unknown status";
    }
}

// A packed matrix resident on the device plus everything a repeated host-buffer product needs.
struct mask_session {
    int32_t M = 0, K = 0;
    int64_t T = 0;
    int32_t* d_soff = nullptr;
    int32_t* d_sidx = nullptr;
    float* d_blk = nullptr;
    mask_plan* plan = nullptr;
    void* d_scratch = nullptr;
    size_t scratch_bytes = 0;
    float* d_B = nullptr;
    float* d_C = nullptr;
    size_t b_bytes = 0, c_bytes = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // column-chunk pipeline of mask_session_spmm_host: upload, multiply and download on three streams
    static constexpr int kMaxChunks = 16;
    cudaStream_t up = nullptr, down = nullptr;
    cudaEvent_t uploaded[kMaxChunks] = {}, k0[kMaxChunks] = {}, k1[kMaxChunks] = {}, downloaded = nullptr;
};

namespace mask {

// -1 = automatic (128-column chunks), 0 = no chunking, else columns per chunk (mask_tune "session_chunk")
int g_session_chunk_cols = -1;

static int session_common_init(mask_session* s) {
    MASK_CUDA_TRY(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    MASK_CUDA_TRY(cudaEventCreate(&s->ev0));
    MASK_CUDA_TRY(cudaEventCreate(&s->ev1));
    MASK_CUDA_TRY(cudaStreamCreateWithFlags(&s->up, cudaStreamNonBlocking));
    MASK_CUDA_TRY(cudaStreamCreateWithFlags(&s->down, cudaStreamNonBlocking));
    for (int i = 0; i < mask_session::kMaxChunks; i++) {
        MASK_CUDA_TRY(cudaEventCreateWithFlags(&s->uploaded[i], cudaEventDisableTiming));
        MASK_CUDA_TRY(cudaEventCreate(&s->k0[i]));
        MASK_CUDA_TRY(cudaEventCreate(&s->k1[i]));
    }
    MASK_CUDA_TRY(cudaEventCreateWithFlags(&s->downloaded, cudaEventDisableTiming));
    return MASK_OK;
}

// Columns per chunk of the host-buffer pipeline: a multiple of 128 that gives 2..kMaxChunks chunks,
// or 0 when N is too narrow or ragged to be worth cutting.
static int session_chunk_cols(int32_t N) {
    if (g_session_chunk_cols == 0 || N % 128 != 0 || N < 256) return 0;
    int w = g_session_chunk_cols > 0 ? g_session_chunk_cols : 128;
    if (w % 32 != 0 || N % w != 0) w = 128;
    while (N / w > mask_session::kMaxChunks) w *= 2;
    return (N % w == 0 && N / w >= 2) ? w : 0;
}

// After the session's streams are idle: has a kernel of this call given up on a bounded wait?
static int session_kernel_status(mask_session* s) {
    int32_t st = 0;
    int rc = mask_plan_status(s->plan, &st, s->stream);
    if (rc != MASK_OK) return rc;
    if (st != 0) return fail(MASK_ERR_KERNEL_TIMEOUT, "a kernel gave up on a bounded wait; the product is invalid");
    return MASK_OK;
}

static int grow(void** p, size_t* have, size_t need) {
    if (need <= *have) return MASK_OK;
    if (*p) MASK_CUDA_TRY(cudaFree(*p));
    *p = nullptr;
    *have = 0;
    MASK_CUDA_TRY(cudaMalloc(p, need));
    *have = need;
    return MASK_OK;
}

}  // namespace mask

extern "C" void mask_session_destroy(mask_session* s) {
    if (!s) return;
    if (s->stream) cudaStreamSynchronize(s->stream);
    cudaFree(s->d_soff);
    cudaFree(s->d_sidx);
    cudaFree(s->d_blk);
    cudaFree(s->d_scratch);
    cudaFree(s->d_B);
    cudaFree(s->d_C);
    mask_plan_destroy(s->plan);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    if (s->up) { cudaStreamSynchronize(s->up); cudaStreamDestroy(s->up); }
    if (s->down) { cudaStreamSynchronize(s->down); cudaStreamDestroy(s->down); }
    for (int i = 0; i < mask_session::kMaxChunks; i++) {
        if (s->uploaded[i]) cudaEventDestroy(s->uploaded[i]);
        if (s->k0[i]) cudaEventDestroy(s->k0[i]);
        if (s->k1[i]) cudaEventDestroy(s->k1[i]);
    }
    if (s->downloaded) cudaEventDestroy(s->downloaded);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

extern "C" int mask_session_create_srbcrs(int32_t M, int32_t K, int64_t T, const int32_t* h_val_soff,
                                          const int32_t* h_val_sidx, const float* h_val_block_val, int policy,
                                          mask_session** out) {
    using namespace mask;
    MASK_REQUIRE(out != nullptr, "out is NULL");
    *out = nullptr;
    MASK_REQUIRE(M >= 1 && K >= 1 && T >= 0 && h_val_soff, "bad arguments");
    MASK_REQUIRE(T == 0 || (h_val_sidx && h_val_block_val), "packed arrays are NULL");
    mask_session* s = new mask_session();
    s->M = M; s->K = K; s->T = T;
    const size_t W = (size_t)(M + kWinRows - 1) / kWinRows;
    auto body = [&]() -> int {
        int rc = session_common_init(s);
        if (rc != MASK_OK) return rc;
        MASK_CUDA_TRY(cudaMalloc((void**)&s->d_soff, (W + 1) * 4));
        MASK_CUDA_TRY(cudaMalloc((void**)&s->d_sidx, std::max<size_t>((size_t)T * 8 * 4, 4)));
        MASK_CUDA_TRY(cudaMalloc((void**)&s->d_blk, std::max<size_t>((size_t)T * 128 * 4, 4)));
        MASK_CUDA_TRY(cudaMemcpyAsync(s->d_soff, h_val_soff, (W + 1) * 4, cudaMemcpyHostToDevice, s->stream));
        if (T > 0) {
            MASK_CUDA_TRY(cudaMemcpyAsync(s->d_sidx, h_val_sidx, (size_t)T * 8 * 4, cudaMemcpyHostToDevice, s->stream));
            MASK_CUDA_TRY(cudaMemcpyAsync(s->d_blk, h_val_block_val, (size_t)T * 128 * 4, cudaMemcpyHostToDevice, s->stream));
        }
        rc = mask_plan_create(s->d_soff, M, T, policy, 0, s->stream, &s->plan);
        if (rc != MASK_OK) return rc;
        return T > 0 ? mask_plan_autotune(s->plan, s->d_soff, s->d_sidx, K, s->stream) : MASK_OK;
    };
    int rc = body();
    if (rc != MASK_OK) { mask_session_destroy(s); return rc; }
    *out = s;
    return MASK_OK;
}

extern "C" int mask_session_create_csr(int32_t M, int32_t K, int64_t nnz, const int32_t* h_rowptr,
                                       const int32_t* h_colind, const float* h_values, int policy,
                                       mask_session** out) {
    using namespace mask;
    MASK_REQUIRE(out != nullptr, "out is NULL");
    *out = nullptr;
    MASK_REQUIRE(M >= 1 && K >= 1 && nnz >= 0 && h_rowptr, "bad arguments");
    MASK_REQUIRE(nnz == 0 || (h_colind && h_values), "colind or values is NULL");
    mask_session* s = new mask_session();
    s->M = M; s->K = K;
    const size_t W = (size_t)(M + kWinRows - 1) / kWinRows;
    int32_t *d_rowptr = nullptr, *d_colind = nullptr;
    float* d_values = nullptr;
    void* d_ws = nullptr;
    auto body = [&]() -> int {
        int rc = session_common_init(s);
        if (rc != MASK_OK) return rc;
        const size_t n = (size_t)std::max<int64_t>(nnz, 1);
        MASK_CUDA_TRY(cudaMalloc((void**)&d_rowptr, ((size_t)M + 1) * 4));
        MASK_CUDA_TRY(cudaMalloc((void**)&d_colind, n * 4));
        MASK_CUDA_TRY(cudaMalloc((void**)&d_values, n * 4));
        MASK_CUDA_TRY(cudaMemcpyAsync(d_rowptr, h_rowptr, ((size_t)M + 1) * 4, cudaMemcpyHostToDevice, s->stream));
        if (nnz > 0) {
            MASK_CUDA_TRY(cudaMemcpyAsync(d_colind, h_colind, (size_t)nnz * 4, cudaMemcpyHostToDevice, s->stream));
            MASK_CUDA_TRY(cudaMemcpyAsync(d_values, h_values, (size_t)nnz * 4, cudaMemcpyHostToDevice, s->stream));
        }
        const size_t ws = mask_pack_scratch_bytes(M, nnz);
        MASK_CUDA_TRY(cudaMalloc(&d_ws, ws));
        MASK_CUDA_TRY(cudaMalloc((void**)&s->d_soff, (W + 1) * 4));
        rc = mask_pack_analyze(d_rowptr, d_colind, M, K, nnz, d_ws, ws, s->d_soff, &s->T, s->stream);
        if (rc != MASK_OK) return rc;
        MASK_CUDA_TRY(cudaMalloc((void**)&s->d_sidx, std::max<size_t>((size_t)s->T * 8 * 4, 4)));
        MASK_CUDA_TRY(cudaMalloc((void**)&s->d_blk, std::max<size_t>((size_t)s->T * 128 * 4, 4)));
        rc = mask_srbcrs_fill(d_rowptr, d_colind, d_values, M, nnz, d_ws, s->d_soff, s->T, s->d_sidx, s->d_blk, nullptr,
                              nullptr, nullptr, s->stream);
        if (rc != MASK_OK) return rc;
        rc = mask_plan_create(s->d_soff, M, s->T, policy, 0, s->stream, &s->plan);
        if (rc != MASK_OK) return rc;
        return s->T > 0 ? mask_plan_autotune(s->plan, s->d_soff, s->d_sidx, K, s->stream) : MASK_OK;
    };
    int rc = body();
    if (s->stream) cudaStreamSynchronize(s->stream);
    cudaFree(d_rowptr);
    cudaFree(d_colind);
    cudaFree(d_values);
    cudaFree(d_ws);
    if (rc != MASK_OK) { mask_session_destroy(s); return rc; }
    *out = s;
    return MASK_OK;
}

extern "C" int64_t mask_session_tiles(const mask_session* s) { return s ? s->T : -1; }

extern "C" int mask_session_spmm_host(mask_session* s, const float* h_B, float* h_C, int32_t N, float* kernel_ms) {
    using namespace mask;
    MASK_REQUIRE(s != nullptr, "session is NULL");
    MASK_REQUIRE(N >= 0 && N % 4 == 0, "N must be a non-negative multiple of 4");
    if (kernel_ms) *kernel_ms = 0.f;
    if (N == 0) return MASK_OK;
    MASK_REQUIRE(h_B && h_C, "B or C is NULL");
    const size_t bb = (size_t)s->K * N * 4, cb = (size_t)s->M * N * 4;
    int rc = grow((void**)&s->d_B, &s->b_bytes, bb);
    if (rc == MASK_OK) rc = grow((void**)&s->d_C, &s->c_bytes, cb);
    if (rc == MASK_OK) rc = grow(&s->d_scratch, &s->scratch_bytes, mask_plan_scratch_bytes(s->plan, N));
    if (rc != MASK_OK) return rc;
    // Column chunks are independent products, so the upload of chunk i+1, the SpMM of chunk i and the
    // download of chunk i-1 overlap: the link carries both directions at once and the call costs
    // about (1 + 1/chunks) of one direction instead of both in sequence.
    const int w = session_chunk_cols(N);
    if (w > 0) {
        const int chunks = N / w;
        const size_t pitch = (size_t)N * 4, width = (size_t)w * 4;
        auto enqueue = [&]() -> int {
            for (int i = 0; i < chunks; i++) {
                const size_t c0 = (size_t)i * w;
                MASK_CUDA_TRY(cudaMemcpy2DAsync(s->d_B + c0, pitch, h_B + c0, pitch, width, (size_t)s->K, cudaMemcpyHostToDevice, s->up));
                MASK_CUDA_TRY(cudaEventRecord(s->uploaded[i], s->up));
                MASK_CUDA_TRY(cudaStreamWaitEvent(s->stream, s->uploaded[i], 0));
                MASK_CUDA_TRY(cudaEventRecord(s->k0[i], s->stream));
                int r = mask_spmm_srbcrs(s->plan, s->d_soff, s->d_sidx, s->d_blk, s->M, s->K, w, s->d_B + c0, N, s->d_C + c0, N,
                                         s->d_scratch, s->scratch_bytes, MASK_EPILOGUE_NONE, s->stream);
                if (r != MASK_OK) return r;
                MASK_CUDA_TRY(cudaEventRecord(s->k1[i], s->stream));
                MASK_CUDA_TRY(cudaStreamWaitEvent(s->down, s->k1[i], 0));
                MASK_CUDA_TRY(cudaMemcpy2DAsync(h_C + c0, pitch, s->d_C + c0, pitch, width, (size_t)s->M, cudaMemcpyDeviceToHost, s->down));
            }
            return MASK_OK;
        };
        rc = enqueue();
        // whatever was enqueued -- also when enqueueing failed half way -- must finish before the caller's
        // buffers are touched again
        cudaError_t e1 = cudaStreamSynchronize(s->up), e2 = cudaStreamSynchronize(s->stream), e3 = cudaStreamSynchronize(s->down);
        if (rc != MASK_OK) return rc;
        MASK_CUDA_TRY(e1);
        MASK_CUDA_TRY(e2);
        MASK_CUDA_TRY(e3);
        rc = session_kernel_status(s);
        if (rc != MASK_OK) return rc;
        if (kernel_ms) {
            for (int i = 0; i < chunks; i++) {
                float ms = 0.f;
                MASK_CUDA_TRY(cudaEventElapsedTime(&ms, s->k0[i], s->k1[i]));
                *kernel_ms += ms;
            }
        }
        return MASK_OK;
    }
    auto enqueue = [&]() -> int {
        MASK_CUDA_TRY(cudaMemcpyAsync(s->d_B, h_B, bb, cudaMemcpyHostToDevice, s->stream));
        MASK_CUDA_TRY(cudaEventRecord(s->ev0, s->stream));
        int r = mask_spmm_srbcrs(s->plan, s->d_soff, s->d_sidx, s->d_blk, s->M, s->K, N, s->d_B, N, s->d_C, N, s->d_scratch,
                                 s->scratch_bytes, MASK_EPILOGUE_NONE, s->stream);
        if (r != MASK_OK) return r;
        MASK_CUDA_TRY(cudaEventRecord(s->ev1, s->stream));
        MASK_CUDA_TRY(cudaMemcpyAsync(h_C, s->d_C, cb, cudaMemcpyDeviceToHost, s->stream));
        return MASK_OK;
    };
    rc = enqueue();
    cudaError_t es = cudaStreamSynchronize(s->stream);   // also after a failed enqueue: the upload may be in flight
    if (rc != MASK_OK) return rc;
    MASK_CUDA_TRY(es);
    rc = session_kernel_status(s);
    if (rc != MASK_OK) return rc;
    if (kernel_ms) MASK_CUDA_TRY(cudaEventElapsedTime(kernel_ms, s->ev0, s->ev1));
    return MASK_OK;
}
