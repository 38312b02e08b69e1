// ME-TCF packed-format cache file and matrix features (host code).
//
// File layout, little endian, no header beyond the two counts -- identical to the reference's
// storeCheckpoint / loadCheckpoint (examples/src_fp32/dtc/testbed/main.cu:232-340):
//   int32 T, int32 nnz_pad, val_soff[W+1], val_sidx[8T], val_coo_off[2T+1], val_coo_idx[nnz_pad],
//   val_coo_val[nnz_pad]
// and file name "<matrix>_M<M>_K<K>_TBK8_RWM16_METCF.checkpoint" (main.cu:217-228).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "plan.h"

extern "C" int mask_metcf_checkpoint_name(const char* matrix_name, int32_t M, int32_t K, char* out, size_t out_len) {
    using namespace mask;
    MASK_REQUIRE(out != nullptr && out_len > 0, "bad arguments");
    std::string base = (matrix_name && matrix_name[0]) ? matrix_name : "synthetic";
    const std::string name = base + "_M" + std::to_string(M) + "_K" + std::to_string(K) + "_TBK8_RWM16_METCF.checkpoint";
    if (name.size() + 1 > out_len) return fail(MASK_ERR_INVALID_ARGUMENT, "name buffer too small");
    std::memcpy(out, name.c_str(), name.size() + 1);
    return MASK_OK;
}

// The name the reference's testbed gives the file for a matrix read from `file_path` -- the file
// name without directories and without its last extension -- or, when the path is empty (a matrix
// generated in memory), "synthetic" plus a sparsity token: the sparsity printed with four decimals,
// trailing zeros and a trailing point dropped, the point written as 'p'
// (examples/src_fp32/dtc/testbed/main.cu:171-176, 205-230).
extern "C" int mask_metcf_checkpoint_name_for(const char* file_path, int32_t M, int32_t K, float sparsity, char* out,
                                              size_t out_len) {
    using namespace mask;
    MASK_REQUIRE(out != nullptr && out_len > 0, "bad arguments");
    std::string path = file_path ? file_path : "";
    std::string base = path;
    const size_t slash = base.find_last_of('/');
    if (slash != std::string::npos) base = base.substr(slash + 1);
    const size_t dot = base.find_last_of('.');
    if (dot != std::string::npos && dot > 0 && base != "..") base = base.substr(0, dot);
    if (base.empty()) base = "synthetic";
    std::string name = base + "_M" + std::to_string(M) + "_K" + std::to_string(K) + "_TBK8_RWM16";
    if (path.empty()) {
        char buf[64];
        std::snprintf(buf, sizeof(buf), "%.4f", (double)sparsity);
        std::string tok = buf;
        while (!tok.empty() && tok.back() == '0') tok.pop_back();
        if (!tok.empty() && tok.back() == '.') tok.pop_back();
        for (char& c : tok)
            if (c == '.') c = 'p';
        name += "_sp" + (tok.empty() ? std::string("unknown") : tok);
    }
    name += "_METCF.checkpoint";
    if (name.size() + 1 > out_len) return fail(MASK_ERR_INVALID_ARGUMENT, "name buffer too small");
    std::memcpy(out, name.c_str(), name.size() + 1);
    return MASK_OK;
}

extern "C" int mask_metcf_checkpoint_write(const char* path, int32_t M, int64_t T, int64_t nnz_pad, const int32_t* val_soff,
                                           const int32_t* val_sidx, const int32_t* val_coo_off, const int32_t* val_coo_idx,
                                           const float* val_coo_val) {
    using namespace mask;
    MASK_REQUIRE(path && val_soff && M >= 1 && T >= 0 && nnz_pad >= 0, "bad arguments");
    MASK_REQUIRE(T < ((int64_t)1 << 31) && nnz_pad < ((int64_t)1 << 31), "counts do not fit the file's int32 fields");
    FILE* f = std::fopen(path, "wb");
    if (!f) return fail(MASK_ERR_INVALID_ARGUMENT, "cannot open checkpoint file for writing");
    const int32_t t32 = (int32_t)T, p32 = (int32_t)nnz_pad;
    const size_t W = (size_t)(M + kWinRows - 1) / kWinRows;
    bool ok = std::fwrite(&t32, 4, 1, f) == 1 && std::fwrite(&p32, 4, 1, f) == 1;
    ok = ok && std::fwrite(val_soff, 4, W + 1, f) == W + 1;
    ok = ok && (T == 0 || std::fwrite(val_sidx, 4, (size_t)T * 8, f) == (size_t)T * 8);
    ok = ok && std::fwrite(val_coo_off, 4, (size_t)2 * T + 1, f) == (size_t)2 * T + 1;
    ok = ok && (nnz_pad == 0 || std::fwrite(val_coo_idx, 4, (size_t)nnz_pad, f) == (size_t)nnz_pad);
    ok = ok && (nnz_pad == 0 || std::fwrite(val_coo_val, 4, (size_t)nnz_pad, f) == (size_t)nnz_pad);
    ok = (std::fclose(f) == 0) && ok;
    return ok ? MASK_OK : fail(MASK_ERR_INVALID_ARGUMENT, "short write to checkpoint file");
}

extern "C" int mask_metcf_checkpoint_header(const char* path, int64_t* T, int64_t* nnz_pad) {
    using namespace mask;
    MASK_REQUIRE(path && T && nnz_pad, "bad arguments");
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(MASK_ERR_INVALID_ARGUMENT, "cannot open checkpoint file");
    int32_t h[2];
    const bool ok = std::fread(h, 4, 2, f) == 2;
    std::fclose(f);
    if (!ok || h[0] < 0 || h[1] < 0) return fail(MASK_ERR_INVALID_ARGUMENT, "checkpoint header unreadable");
    *T = h[0];
    *nnz_pad = h[1];
    return MASK_OK;
}

// Reads the arrays (sized from mask_metcf_checkpoint_header) and applies the reference's load-time
// validation (main.cu:586-600): offsets start at 0 and end at T / nnz_pad, columns inside [0, K).
extern "C" int mask_metcf_checkpoint_read(const char* path, int32_t M, int32_t K, int64_t T, int64_t nnz_pad,
                                          int32_t* val_soff, int32_t* val_sidx, int32_t* val_coo_off,
                                          int32_t* val_coo_idx, float* val_coo_val) {
    using namespace mask;
    MASK_REQUIRE(path && val_soff && val_coo_off && M >= 1 && K >= 1 && T >= 0 && nnz_pad >= 0, "bad arguments");
    FILE* f = std::fopen(path, "rb");
    if (!f) return fail(MASK_ERR_INVALID_ARGUMENT, "cannot open checkpoint file");
    int32_t h[2] = {-1, -1};
    const size_t W = (size_t)(M + kWinRows - 1) / kWinRows;
    bool ok = std::fread(h, 4, 2, f) == 2 && h[0] == T && h[1] == nnz_pad;
    ok = ok && std::fread(val_soff, 4, W + 1, f) == W + 1;
    ok = ok && (T == 0 || std::fread(val_sidx, 4, (size_t)T * 8, f) == (size_t)T * 8);
    ok = ok && std::fread(val_coo_off, 4, (size_t)2 * T + 1, f) == (size_t)2 * T + 1;
    ok = ok && (nnz_pad == 0 || std::fread(val_coo_idx, 4, (size_t)nnz_pad, f) == (size_t)nnz_pad);
    ok = ok && (nnz_pad == 0 || std::fread(val_coo_val, 4, (size_t)nnz_pad, f) == (size_t)nnz_pad);
    char extra;
    ok = ok && std::fread(&extra, 1, 1, f) == 0;   // nothing may follow
    std::fclose(f);
    if (!ok) return fail(MASK_ERR_INVALID_ARGUMENT, "checkpoint file does not match the expected sizes");
    if (val_soff[0] != 0 || val_soff[W] != T || val_coo_off[2 * T] != nnz_pad)
        return fail(MASK_ERR_INVALID_ARGUMENT, "checkpoint offsets are inconsistent");
    for (int64_t i = 0; i < T * 8; i++)
        if (val_sidx[i] < 0 || val_sidx[i] >= K) return fail(MASK_ERR_COLUMN_RANGE, "checkpoint column id outside [0, K)");
    return MASK_OK;
}

// ---- matrix features (the quantities the execution plan is chosen from) ----------------------------
extern "C" int mask_features_from_soff(const int32_t* h_val_soff, int32_t M, int64_t nnz, mask_features* out) {
    using namespace mask;
    MASK_REQUIRE(h_val_soff && out && M >= 1 && nnz >= 0, "bad arguments");
    const int W = (M + kWinRows - 1) / kWinRows;
    std::vector<int32_t> len((size_t)W);
    for (int w = 0; w < W; w++) len[w] = h_val_soff[w + 1] - h_val_soff[w];
    std::sort(len.begin(), len.end());
    auto pct = [&](double q) {  // same rank rule as the bridge's p95 (custom_format_e2e.cu:652-657)
        const size_t i = std::min(len.size() - 1, (size_t)std::ceil(len.size() * q) - 1);
        return len[i];
    };
    mask_features f{};
    f.row_windows = W;
    f.tiles = h_val_soff[W];
    f.nnz = nnz;
    f.tiles_mean = W ? (double)f.tiles / W : 0.0;
    f.tiles_p50 = pct(0.50);
    f.tiles_p95 = pct(0.95);
    f.tiles_p99 = pct(0.99);
    f.tiles_max = len.back();
    int64_t top5 = 0;
    for (int i = 0; i < std::min(5, W); i++) top5 += len[(size_t)W - 1 - i];
    f.top5_window_share = f.tiles ? (double)top5 / (double)f.tiles : 0.0;
    f.tile_fill = f.tiles ? (double)nnz / (128.0 * (double)f.tiles) : 0.0;
    // the bridge's heavy-tail test (custom_format_e2e.cu:659-663)
    f.heavy_tail = f.tiles_max > std::max(64, 4 * std::max(f.tiles_p95, 1)) ? 1 : 0;
    f.empty_windows = (int32_t)(std::lower_bound(len.begin(), len.end(), 1) - len.begin());
    *out = f;
    return MASK_OK;
}
