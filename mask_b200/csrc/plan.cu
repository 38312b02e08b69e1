// Task planners (host) and the execution-plan handle.
#include "plan.h"

#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.cuh"

namespace mask {

// Strict load balance: every group holds exactly `workload` tiles, windows are cut wherever a
// group fills up (examples/src_fp32/sr_bcrs/testbed/main_strict_lb_16x8.cu:208-256).
static void strict_lb(const int32_t* soff, int32_t W, int32_t workload, std::vector<int32_t>& rbo,
                      std::vector<int32_t>& rb2w, std::vector<int32_t>& go) {
    rbo.clear(); rb2w.clear(); go.clear();
    go.push_back(0);
    int32_t load = 0;
    for (int32_t w = 0; w < W; w++) {
        int32_t s = soff[w];
        const int32_t e = soff[w + 1];
        while (s < e) {
            const int32_t take = std::min(workload - load, e - s);
            rbo.push_back(s);
            rb2w.push_back(w);
            s += take;
            load += take;
            if (load == workload) {
                go.push_back((int32_t)rb2w.size());
                load = 0;
            }
        }
    }
    rbo.push_back(soff[W]);
    if (load != 0 || go.size() == 1) go.push_back((int32_t)rb2w.size());
}

// Multi-binding: windows above twice the mean tile count (mean over all windows) are cut into
// ceil(x/mean) near-equal tasks (examples/src_fp32/sr_bcrs/testbed/main_multi_bind_16x8.cu:207-271).
static void multi_bind(const int32_t* soff, int32_t W, std::vector<int32_t>& task_win,
                       std::vector<int32_t>& win_split, std::vector<int32_t>& task_soff) {
    task_win.clear(); task_soff.clear();
    win_split.assign((size_t)W, 0);
    double sum = 0.0;
    for (int32_t w = 0; w < W; w++) sum += (double)(soff[w + 1] - soff[w]);
    const double avg = W > 0 ? sum / (double)W : 0.0;
    task_soff.push_back(0);
    for (int32_t w = 0; w < W; w++) {
        const int32_t x = soff[w + 1] - soff[w];
        if (x == 0) continue;
        int32_t parts = 1;
        if (avg > 0.0 && (double)x > 2.0 * avg) {
            parts = std::max(1, std::min((int32_t)std::ceil((double)x / avg), 9999));
            if (parts > 1) win_split[w] = 1;
        }
        const int32_t base = x / parts, rem = x % parts;
        for (int32_t i = 0; i < parts; i++) {
            task_win.push_back(w);
            task_soff.push_back(task_soff.back() + base + (i < rem ? 1 : 0));
        }
    }
}

static int32_t default_group_tiles(int64_t T) {
    // The SpMM grid is resident (two blocks per SM) and deals groups round-robin, so the blocks that
    // run at the same time work on neighbouring groups.  Groups are kept SHORT on purpose: what the
    // resident blocks touch together is then a narrow band of windows, and rows of B shared by
    // neighbouring windows (stencils, banded matrices) are fetched from DRAM once and found in L2
    // by the other blocks.  Groups of 800 tiles measured twice as slow as groups of 128 on a
    // 27-point stencil and on a power-law graph for exactly that reason.
    // Small matrices: one group per resident block (every group a block takes costs it a pipeline
    // restart, and with fewer groups than blocks nothing is left to balance).
    const int64_t resident = (int64_t)sm_count() * 2;
    const int64_t g = (T + resident - 1) / resident;
    return (int32_t)std::max<int64_t>(16, std::min<int64_t>(128, g));
}

// Fills the fragment / group tables of `p` from val_soff on the host.
static void build_tables(mask_plan& p, const int32_t* soff) {
    const int32_t W = p.W;
    const int32_t G = p.group_tiles;
    auto& fo = p.h_frag_off; auto& fw = p.h_frag_win; auto& go = p.h_group_off;
    fo.clear(); fw.clear(); go.clear();
    go.push_back(0);
    constexpr int kMaxFragsPerGroup = 32;

    if (p.policy == MASK_POLICY_STRICT_LB || p.policy == MASK_POLICY_MULTI_BIND) {
        // the reference tables, plus an empty fragment for every window without tiles so that
        // its rows of C are written
        std::vector<int32_t> rbo, rb2w, rgo, tsoff, wsplit;
        if (p.policy == MASK_POLICY_STRICT_LB) {
            strict_lb(soff, W, G, rbo, rb2w, rgo);
        } else {
            multi_bind(soff, W, rb2w, wsplit, tsoff);
            rbo = tsoff;
            rgo.resize(rb2w.size() + 1);
            for (size_t i = 0; i <= rb2w.size(); i++) rgo[i] = (int32_t)i;
        }
        const size_t nf = rb2w.size();
        size_t gi = 1;  // next reference group boundary to emit
        int32_t next_w = 0;
        int in_group = 0;
        for (size_t f = 0; f < nf; f++) {
            while (next_w < rb2w[f]) {  // windows skipped by the reference tables are empty
                fo.push_back(soff[next_w]); fw.push_back(next_w); next_w++;
                if (++in_group == kMaxFragsPerGroup) { go.push_back((int32_t)fw.size()); in_group = 0; }
            }
            next_w = std::max(next_w, rb2w[f] + 1);
            fo.push_back(rbo[f]); fw.push_back(rb2w[f]); in_group++;
            if (gi < rgo.size() && (size_t)rgo[gi] == f + 1) {
                go.push_back((int32_t)fw.size()); in_group = 0; gi++;
            }
        }
        while (next_w < W) {
            fo.push_back(soff[next_w]); fw.push_back(next_w); next_w++;
            if (++in_group == kMaxFragsPerGroup) { go.push_back((int32_t)fw.size()); in_group = 0; }
        }
        if (go.back() != (int32_t)fw.size()) go.push_back((int32_t)fw.size());
    } else {
        // Groups are closed on window boundaries once their cost (tiles plus a fixed share per window
        // for the rows of C it writes) reaches G; a window of more than 5/4 G tiles is cut into
        // near-equal pieces of at most G tiles, one group each (each piece costs one partial tile in
        // scratch and the fix-up pass sums them in tile order).
        constexpr int32_t kWindowCost = 4;
        const int32_t split_above = G + G / 4;
        int32_t load = 0;
        auto close = [&]() {
            if (go.back() != (int32_t)fw.size()) go.push_back((int32_t)fw.size());
            load = 0;
        };
        for (int32_t w = 0; w < W; w++) {
            const int32_t s = soff[w], x = soff[w + 1] - s;
            if (p.policy == MASK_POLICY_ROW) {
                fo.push_back(s); fw.push_back(w); close();
                continue;
            }
            if (x > split_above) {  // split into near-equal parts, one group each
                close();
                const int32_t parts = (x + G - 1) / G, base = x / parts, rem = x % parts;
                int32_t at = s;
                for (int32_t i = 0; i < parts; i++) {
                    fo.push_back(at); fw.push_back(w); close();
                    at += base + (i < rem ? 1 : 0);
                }
                continue;
            }
            if (load > 0 && load + x + kWindowCost > G + G / 8) close();
            fo.push_back(s); fw.push_back(w);
            load += x + kWindowCost;
            if (load >= G) close();
        }
        close();
    }
    fo.push_back(soff[W]);

    p.F = (int64_t)fw.size();
    p.G = (int64_t)go.size() - 1;
    p.h_frag_slot.assign((size_t)p.F, -1);
    p.h_head_frag.clear();
    p.P = 0;
    for (int64_t f = 0; f < p.F; f++) {
        const int32_t w = fw[f];
        const bool whole = fo[f] == soff[w] && fo[f + 1] == soff[w + 1];
        if (!whole) {
            if (f == 0 || fw[f - 1] != w) p.h_head_frag.push_back((int32_t)f);
            p.h_frag_slot[f] = (int32_t)p.P++;
        }
    }
    p.H = (int64_t)p.h_head_frag.size();
    p.max_group_tiles = 0;
    p.h_group_tile.resize((size_t)p.G + 1);
    for (int64_t g = 0; g <= p.G; g++) p.h_group_tile[(size_t)g] = fo[go[g]];
    for (int64_t g = 0; g < p.G; g++)
        p.max_group_tiles = std::max<int32_t>(p.max_group_tiles, fo[go[g + 1]] - fo[go[g]]);
}

template <typename T>
static int upload(const std::vector<T>& h, T** d, cudaStream_t st) {
    const size_t n = std::max<size_t>(h.size(), 1);
    MASK_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(d), n * sizeof(T)));
    if (!h.empty()) MASK_CUDA_TRY(cudaMemcpyAsync(*d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice, st));
    return MASK_OK;
}

}  // namespace mask

extern "C" int mask_plan_strict_lb(const int32_t* h_val_soff, int32_t M, int32_t workload, int32_t* row_block_offset,
                                   int32_t* row_block_to_window, int32_t* group_offset, int64_t* n_frag,
                                   int64_t* n_groups) {
    using namespace mask;
    MASK_REQUIRE(h_val_soff != nullptr && M >= 1 && workload >= 1 && n_frag && n_groups, "bad arguments");
    std::vector<int32_t> rbo, rb2w, go;
    strict_lb(h_val_soff, (M + kWinRows - 1) / kWinRows, workload, rbo, rb2w, go);
    *n_frag = (int64_t)rb2w.size();
    *n_groups = (int64_t)go.size() - 1;
    if (row_block_offset) std::memcpy(row_block_offset, rbo.data(), rbo.size() * sizeof(int32_t));
    if (row_block_to_window && !rb2w.empty()) std::memcpy(row_block_to_window, rb2w.data(), rb2w.size() * sizeof(int32_t));
    if (group_offset) std::memcpy(group_offset, go.data(), go.size() * sizeof(int32_t));
    return MASK_OK;
}

extern "C" int mask_plan_multi_bind(const int32_t* h_val_soff, int32_t M, int32_t* task_window, int32_t* window_split,
                                    int32_t* task_soff, int64_t* n_tasks) {
    using namespace mask;
    MASK_REQUIRE(h_val_soff != nullptr && M >= 1 && n_tasks, "bad arguments");
    std::vector<int32_t> tw, ws, ts;
    multi_bind(h_val_soff, (M + kWinRows - 1) / kWinRows, tw, ws, ts);
    *n_tasks = (int64_t)tw.size();
    if (task_window && !tw.empty()) std::memcpy(task_window, tw.data(), tw.size() * sizeof(int32_t));
    if (window_split && !ws.empty()) std::memcpy(window_split, ws.data(), ws.size() * sizeof(int32_t));
    if (task_soff) std::memcpy(task_soff, ts.data(), ts.size() * sizeof(int32_t));
    return MASK_OK;
}

extern "C" int mask_plan_create(const int32_t* d_val_soff, int32_t M, int64_t T, int policy, int32_t group_tiles,
                                void* stream, mask_plan** out) {
    using namespace mask;
    MASK_REQUIRE(out != nullptr, "out is NULL");
    *out = nullptr;
    MASK_REQUIRE(d_val_soff != nullptr && M >= 1 && T >= 0, "bad arguments");
    MASK_REQUIRE(policy >= MASK_POLICY_AUTO && policy <= MASK_POLICY_REF_AUTO, "unknown policy");
    if (T >= (int64_t)1 << 31) return fail(MASK_ERR_INDEX_OVERFLOW, "T does not fit int32");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    mask_plan* p = new mask_plan();
    p->M = M;
    p->W = (M + kWinRows - 1) / kWinRows;
    p->T = T;
    p->policy = policy;
    p->group_tiles = group_tiles > 0 ? group_tiles : (policy == MASK_POLICY_STRICT_LB ? 64 : default_group_tiles(T));
    std::vector<int32_t> soff((size_t)p->W + 1);
    cudaError_t e = cudaMemcpyAsync(soff.data(), d_val_soff, soff.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        delete p;
        set_error("copying val_soff to the host failed: %s", cudaGetErrorString(e));
        return MASK_ERR_CUDA;
    }
    if (soff[0] != 0 || (int64_t)soff[p->W] != T) {
        delete p;
        return fail(MASK_ERR_INVALID_ARGUMENT, "val_soff does not start at 0 / end at T");
    }
    if (policy == MASK_POLICY_REF_AUTO) {  // the bridge's automatic choice between its own two mappings
        mask_features f;
        mask_features_from_soff(soff.data(), M, 0, &f);
        p->policy = f.heavy_tail ? MASK_POLICY_STRICT_LB : MASK_POLICY_ROW;
        if (group_tiles <= 0) p->group_tiles = 64;
    }
    build_tables(*p, soff.data());
    int rc = upload(p->h_frag_off, &p->d_frag_off, st);
    if (rc == MASK_OK) rc = upload(p->h_frag_win, &p->d_frag_win, st);
    if (rc == MASK_OK) rc = upload(p->h_frag_slot, &p->d_frag_slot, st);
    if (rc == MASK_OK) rc = upload(p->h_group_off, &p->d_group_off, st);
    if (rc == MASK_OK) rc = upload(p->h_head_frag, &p->d_head_frag, st);
    if (rc == MASK_OK) rc = upload(p->h_group_tile, &p->d_group_tile, st);
    if (rc == MASK_OK) rc = upload(std::vector<int32_t>(4, 0), &p->d_status, st);
    if (rc == MASK_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(MASK_ERR_CUDA, "plan upload failed");
    if (rc != MASK_OK) {
        mask_plan_destroy(p);
        return rc;
    }
    *out = p;
    return MASK_OK;
}

extern "C" void mask_plan_destroy(mask_plan* p) {
    if (!p) return;
    cudaFree(p->d_frag_off);
    cudaFree(p->d_frag_win);
    cudaFree(p->d_frag_slot);
    cudaFree(p->d_group_off);
    cudaFree(p->d_head_frag);
    cudaFree(p->d_group_tile);
    cudaFree(p->d_vals_tf32);
    cudaFree(p->d_status);
    delete p;
}

extern "C" size_t mask_plan_scratch_bytes(const mask_plan* p, int32_t N) {
    if (!p || N <= 0) return 0;
    return (size_t)p->P * mask::kWinRows * (size_t)N * sizeof(float);
}

extern "C" int mask_plan_info(const mask_plan* p, int64_t* n_frag, int64_t* n_groups, int64_t* n_partial,
                              int32_t* group_tiles) {
    using namespace mask;
    MASK_REQUIRE(p != nullptr, "plan is NULL");
    if (n_frag) *n_frag = p->F;
    if (n_groups) *n_groups = p->G;
    if (n_partial) *n_partial = p->P;
    if (group_tiles) *group_tiles = p->group_tiles;
    return MASK_OK;
}

extern "C" int mask_plan_set_row_map(mask_plan* p, const int32_t* d_row_order) {
    using namespace mask;
    MASK_REQUIRE(p != nullptr, "plan is NULL");
    p->d_row_map = d_row_order;
    return MASK_OK;
}

extern "C" int mask_plan_set_peer_outputs(mask_plan* p, float* const* d_peer_ptrs, int32_t n_peers) {
    using namespace mask;
    MASK_REQUIRE(p != nullptr, "plan is NULL");
    MASK_REQUIRE(n_peers >= 0 && n_peers <= 15 && (n_peers == 0 || d_peer_ptrs != nullptr), "bad peer list");
    p->d_peer_out = n_peers ? d_peer_ptrs : nullptr;
    p->n_peer_out = n_peers;
    return MASK_OK;
}

extern "C" int mask_plan_status(const mask_plan* p, int32_t* h_status, void* stream) {
    using namespace mask;
    MASK_REQUIRE(p != nullptr && h_status != nullptr, "NULL argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    MASK_CUDA_TRY(cudaMemcpyAsync(h_status, p->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    MASK_CUDA_TRY(cudaMemsetAsync(p->d_status, 0, sizeof(int32_t), st));   // one expiry must not mark every later call
    MASK_CUDA_TRY(cudaStreamSynchronize(st));
    return MASK_OK;
}

extern "C" int mask_plan_export(const mask_plan* p, int32_t* frag_offset, int32_t* frag_window, int32_t* group_offset) {
    using namespace mask;
    MASK_REQUIRE(p != nullptr, "plan is NULL");
    if (frag_offset) std::memcpy(frag_offset, p->h_frag_off.data(), p->h_frag_off.size() * sizeof(int32_t));
    if (frag_window && p->F) std::memcpy(frag_window, p->h_frag_win.data(), p->h_frag_win.size() * sizeof(int32_t));
    if (group_offset) std::memcpy(group_offset, p->h_group_off.data(), p->h_group_off.size() * sizeof(int32_t));
    return MASK_OK;
}
