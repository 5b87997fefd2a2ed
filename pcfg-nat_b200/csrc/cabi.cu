// extern "C" entry points declared in include/pcfgnat.h: argument checks, then launch.
#include <algorithm>
#include <utility>
#include <vector>

#include "common.cuh"

#include <cstdlib>
#include <mutex>

#include <nvtx3/nvToolsExt.h>

using namespace pcfgnat;

namespace pcfgnat {

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is sticky per (function, device); remember what
// was set so that steady-state launches make no driver call for it.
cudaError_t ensure_dynamic_smem_for(const void *kernel, size_t bytes) {
    constexpr int kSlots = 64, kDevs = 16;
    struct Entry {
        const void *fn;
        int bytes[kDevs];
    };
    static Entry table[kSlots] = {};
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    Entry *slot = nullptr;
    for (int i = 0; i < kSlots; i++) {
        if (table[i].fn == kernel || table[i].fn == nullptr) {
            slot = &table[i];
            break;
        }
    }
    if (slot && slot->fn == kernel && dev >= 0 && dev < kDevs && slot->bytes[dev] >= (int)bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && slot && dev >= 0 && dev < kDevs) {
        slot->fn = kernel;
        slot->bytes[dev] = (int)bytes;
    }
    return e;
}

bool exact_order_forced() {
    const char *v = getenv("PCFGNAT_EXACT_ORDER");
    return v && v[0] && v[0] != '0';
}

// Inside pass of the fused forward + backward: the table stays inside the library, so the free-order kernel
// may build it unless the caller asked for the reference's order or forced a kernel family.
int launch_loss_fwd_internal(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B,
                             int L, int T, float *S, float *loss, int *status, cudaStream_t st, float *mg,
                             bool *shares_in_mg) {
    *shares_in_mg = false;
    if (!exact_order_forced() && dp_kernel_choice() == kDpAuto) {
        float *shares = (mg && fused_grad_applies(B, L, T)) ? mg : nullptr;
        int rc = launch_loss_fwd_fast(match_all, links, ol, tl, B, L, T, S, loss, status, st, shares);
        if (rc == PCFGNAT_OK) *shares_in_mg = shares != nullptr;
        if (rc == PCFGNAT_ERR_UNSUPPORTED && shares)  // the two more arrays did not fit: without the shares
            rc = launch_loss_fwd_fast(match_all, links, ol, tl, B, L, T, S, loss, status, st, nullptr);
        if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
    }
    return launch_loss_fwd(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st);
}

DpKernel dp_kernel_choice() {
    const char *v = getenv("PCFGNAT_DP_KERNEL");
    if (v && v[0] == 'r') return kDpRows;
    if (v && v[0] == 'b') return kDpBalanced;
    if (v && v[0] == 'c') return kDpCluster;
    return kDpAuto;
}

}  // namespace pcfgnat

namespace pcfgnat {

// Forward + backward with the tables in [tables, tables + 2 * table_bytes) and the frames behind them.
int loss_fwd_bwd_in(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L, int T,
                    void *tables, size_t table_bytes, float *loss, float *mg, float *lg, int *status, cudaStream_t st) {
    float *S = static_cast<float *>(tables);
    float *G = reinterpret_cast<float *>(static_cast<char *>(tables) + table_bytes);
    float *frames = reinterpret_cast<float *>(static_cast<char *>(tables) + 2 * table_bytes);
    if (!exact_order_forced() && dp_kernel_choice() == kDpAuto && linear_dp_applies(B, L, T)) {
        // linear space first; the log-space kernels then recompute the sentences it left marked (normally none)
        int rc = launch_loss_linear(match_all, links, ol, tl, B, L, T, S, G, frames, loss, mg, lg, status, st);
        if (rc == PCFGNAT_OK) {
            rc = launch_loss_fwd_rows(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st, frames);
            if (rc) return rc;
            return launch_loss_bwd_rows(nullptr, S, match_all, links, ol, tl, B, L, T, G, mg, lg, status, st, frames);
        }
        if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
    }
    bool shares_in_mg = false;
    int rc = launch_loss_fwd_internal(match_all, links, ol, tl, B, L, T, S, loss, status, st, mg, &shares_in_mg);
    if (rc) return rc;
    return launch_loss_bwd(nullptr, S, match_all, links, ol, tl, B, L, T, G, mg, lg, status, st, shares_in_mg);
}

}  // namespace pcfgnat

namespace {

inline bool bad_dims(int B, int L, int T) { return B < 0 || L < 2 || T < 1; }

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace

namespace pcfgnat {
bool pdl_enabled() {
    static const bool on = [] {
        const char *v = getenv("PCFGNAT_PDL");
        return v && v[0] == '1';
    }();
    return on;
}
}  // namespace pcfgnat

namespace {

// The runs of rows (first row, rows; in rows of the [B * L] view) that send the real graph nodes of sentences
// [b0, b1): one per non-empty sentence, adjacent ones joined; with more runs than max_copies (> 0), neighbours are
// joined across the smallest gaps of padding rows (which are then sent along) until max_copies runs are left.
std::vector<std::pair<int64_t, int64_t>> plan_real_rows(const int64_t *host_lengths, int b0, int b1, int L, int max_copies) {
    std::vector<std::pair<int64_t, int64_t>> runs;
    runs.reserve((size_t)(b1 - b0));
    for (int b = b0; b < b1; b++) {
        int64_t m = host_lengths[b];
        m = m < 0 ? 0 : (m > L ? L : m);
        if (m == 0) continue;
        const int64_t start = (int64_t)b * L;
        if (!runs.empty() && runs.back().first + runs.back().second == start) runs.back().second += m;
        else runs.emplace_back(start, m);
    }
    // a copy costs the host several microseconds: with more runs than max_copies, neighbours are joined across the
    // smallest gaps of padding rows (which are then sent along) until max_copies runs are left
    if (max_copies > 0 && runs.size() > (size_t)max_copies) {
        std::vector<int64_t> gaps(runs.size() - 1);
        for (size_t i = 0; i + 1 < runs.size(); i++) gaps[i] = runs[i + 1].first - (runs[i].first + runs[i].second);
        std::vector<int64_t> sorted(gaps);
        const size_t join = runs.size() - (size_t)max_copies;  // that many gaps go
        std::nth_element(sorted.begin(), sorted.begin() + (join - 1), sorted.end());
        const int64_t limit = sorted[join - 1];
        size_t below = 0;
        for (int64_t g : gaps) below += g < limit;
        size_t at_limit = join - below;  // of the gaps equal to the limit, only this many are joined
        std::vector<std::pair<int64_t, int64_t>> merged;
        merged.reserve((size_t)max_copies);
        merged.push_back(runs[0]);
        for (size_t i = 0; i + 1 < runs.size(); i++) {
            bool joined = gaps[i] < limit;
            if (!joined && gaps[i] == limit && at_limit) joined = true, at_limit--;
            if (joined) merged.back().second = runs[i + 1].first + runs[i + 1].second - merged.back().first;
            else merged.push_back(runs[i + 1]);
        }
        runs.swap(merged);
    }
    return runs;
}

// NVTX range around an entry point (its host side: argument checks and launches) when PCFGNAT_NVTX=1 was set when
// the library was first called; free otherwise.  The ranges carry the entry point's name, so that a timeline of the
// host application shows which of its calls the kernels belong to.
struct ApiRange {
    static bool enabled() {
        static const bool on = [] {
            const char *v = getenv("PCFGNAT_NVTX");
            return v && v[0] == '1';
        }();
        return on;
    }
    explicit ApiRange(const char *name) : on_(enabled()) {
        if (on_) nvtxRangePushA(name);
    }
    ~ApiRange() {
        if (on_) nvtxRangePop();
    }
    ApiRange(const ApiRange &) = delete;
    ApiRange &operator=(const ApiRange &) = delete;

private:
    bool on_;
};
#define PCFGNAT_API_RANGE() ApiRange api_range_(__func__)

}  // namespace

extern "C" {

int pcfgnat_version(void) { return 100; }

const char *pcfgnat_error_string(int code) {
    switch (code) {
        case PCFGNAT_OK: return "ok";
        case PCFGNAT_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, negative or inconsistent size)";
        case PCFGNAT_ERR_UNSUPPORTED: return "unsupported configuration (max_left other than 1, a dtype other than f32/f16, or a shape this kernel cannot take)";
        case PCFGNAT_ERR_CUDA: return "a CUDA runtime call or kernel launch failed";
        case PCFGNAT_ERR_WORKSPACE: return "workspace too small";
        case PCFGNAT_ERR_TOO_LARGE: return "shape too large for the kernels";
        default: return "unknown error code";
    }
}

int pcfgnat_loss_fwd(const float *match_all, const float *links, const int64_t *output_length,
                     const int64_t *target_length, int B, int L, int T, int max_left, float *S, float *C, int *status,
                     void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (bad_dims(B, L, T)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!match_all || !links || !output_length || !target_length || !S)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_loss_fwd(match_all, links, output_length, target_length, B, L, T, S, C, nullptr, status,
                           static_cast<cudaStream_t>(stream));
}

int pcfgnat_loss_bwd(const float *grad_output, const float *S, const float *match_all, const float *links,
                     const int64_t *output_length, const int64_t *target_length, int B, int L, int T, int max_left,
                     float *S_grad, float *match_all_grad, float *links_grad, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (bad_dims(B, L, T)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!grad_output || !S || !match_all || !links || !output_length || !target_length || !S_grad ||
              !match_all_grad || !links_grad))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_loss_bwd(grad_output, S, match_all, links, output_length, target_length, B, L, T, S_grad,
                           match_all_grad, links_grad, status, static_cast<cudaStream_t>(stream));
}

size_t pcfgnat_loss_workspace_bytes(int B, int L, int T, int max_left) {
    if (max_left != 1 || bad_dims(B, L, T)) return 0;
    const size_t table = align256((size_t)B * main_slots(L, 1) * (T + 2) * sizeof(float));
    return 2 * table + linear_frames_bytes(B, T);  // two DP tables and the per-sentence frames of the linear-space pass
}


int pcfgnat_loss_fwd_bwd_kernels(int B, int L, int T, int max_left) {
    if (max_left != 1 || bad_dims(B, L, T)) return 0;
    // linear-space inside and outside kernels, then the three log-space kernels that pick up marked sentences
    if (!exact_order_forced() && dp_kernel_choice() == kDpAuto && linear_dp_applies(B, L, T)) return 5;
    // the shares the fused backward needs come from the free-order inside pass only
    const bool free_order = !exact_order_forced() && dp_kernel_choice() == kDpAuto && main_slots(L, 1) <= 256;
    return free_order && fused_grad_applies(B, L, T) ? 2 : 3;
}

int pcfgnat_loss_fwd_bwd(const float *match_all, const float *links, const int64_t *output_length,
                         const int64_t *target_length, int B, int L, int T, int max_left, void *workspace,
                         size_t workspace_bytes, float *loss, float *match_all_grad, float *links_grad, int *status,
                         void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (bad_dims(B, L, T)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!match_all || !links || !output_length || !target_length || !workspace || !loss || !match_all_grad ||
              !links_grad))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    const size_t need = pcfgnat_loss_workspace_bytes(B, L, T, max_left);
    if (workspace_bytes < need) return PCFGNAT_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) % 16) return PCFGNAT_ERR_INVALID_ARGUMENT;
    const size_t table = align256((size_t)B * main_slots(L, 1) * (T + 2) * sizeof(float));
    return loss_fwd_bwd_in(match_all, links, output_length, target_length, B, L, T, workspace, table, loss, match_all_grad,
                           links_grad, status, static_cast<cudaStream_t>(stream));
}

int pcfgnat_best_tree(const float *S, const float *match_all, const float *links, const int64_t *output_length,
                      const int64_t *target_length, int B, int L, int T, int max_left, int64_t *tree, int *status,
                      void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (bad_dims(B, L, T)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!S || !match_all || !links || !output_length || !target_length || !tree))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_best_tree(S, match_all, links, output_length, target_length, B, L, T, tree, status,
                            static_cast<cudaStream_t>(stream));
}

int pcfgnat_viterbi(const float *ob_lprob, const float *links, const int64_t *output_length, int B, int L,
                    int max_left, float *S, int64_t *R, int64_t *Lt, int64_t *Mt, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 8) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!ob_lprob || !links || !output_length || !S || !R || !Lt || !Mt)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_viterbi(ob_lprob, links, output_length, B, L, S, R, Lt, Mt, status,
                          static_cast<cudaStream_t>(stream));
}

int pcfgnat_viterbi_backtrace(const int64_t *pred_length, const int64_t *output_length, const int64_t *Lt,
                              const int64_t *R, const int64_t *Mt, const int64_t *tokens,
                              const int64_t *left_tree_mask, int mask_dim, int64_t pad_index, int B, int L, int Q,
                              int cap, int64_t *out_tokens, int64_t *out_count, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || Q < 1 || cap < 0 || mask_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!pred_length || !output_length || !Lt || !R || !Mt || !tokens || !left_tree_mask || !out_count ||
              (cap && !out_tokens)))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_backtrace(pred_length, output_length, Lt, R, Mt, tokens, left_tree_mask, mask_dim, pad_index, B, L,
                            Q, cap, out_tokens, out_count, status, static_cast<cudaStream_t>(stream));
}

int pcfgnat_viterbi_decode(const float *S, const float *penalty, const int64_t *output_length, const int64_t *Lt,
                           const int64_t *R, const int64_t *Mt, const int64_t *tokens, const int64_t *left_tree_mask,
                           int mask_dim, int64_t pad_index, int B, int L, int Q, int cap, int64_t *pred_length,
                           int64_t *out_tokens, int64_t *out_count, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 2 || Q < 2 || cap < 0 || mask_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!S || !penalty || !output_length || !Lt || !R || !Mt || !tokens || !left_tree_mask || !pred_length ||
              !out_count || (cap && !out_tokens)))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_viterbi_decode(S, penalty, output_length, Lt, R, Mt, tokens, left_tree_mask, mask_dim, pad_index, B, L,
                                 Q, cap, pred_length, out_tokens, out_count, status, static_cast<cudaStream_t>(stream));
}

int pcfgnat_lookahead_decode(const float *links, const float *ob_lprob, const int64_t *tokens,
                             const int64_t *output_length, const int64_t *left_tree_mask, int mask_dim, float beta,
                             int lookahead, int64_t pad_index, int B, int L, int max_left, int cap, int64_t *out_tokens,
                             int64_t *out_count, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 2 || cap < 0 || mask_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!links || !tokens || !output_length || !left_tree_mask || !out_count || (cap && !out_tokens) ||
              (lookahead && !ob_lprob)))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_lookahead_decode(links, ob_lprob, tokens, output_length, left_tree_mask, mask_dim, beta, lookahead != 0,
                                   pad_index, B, L, cap, out_tokens, out_count, status, static_cast<cudaStream_t>(stream));
}

int pcfgnat_logsoftmax_gather(void *logits, int dtype, const int64_t *select_idx, int64_t stride_b, int64_t stride_l,
                              int64_t stride_s, int64_t rows, int64_t rows_per_batch, int V, int slen,
                              int require_gradient, float *selected, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (rows < 0 || rows_per_batch < 1 || V < 1 || slen < 0) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (rows && (!logits || (slen && (!select_idx || !selected)))) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_logsoftmax_gather(logits, dtype, select_idx, stride_b, stride_l, stride_s, rows, rows_per_batch, V,
                                    slen, require_gradient, selected, status, static_cast<cudaStream_t>(stream));
}

size_t pcfgnat_proj_workspace_bytes(int B, int L, int T, int V) {
    if (B < 0 || L < 1 || T < 0 || V < 1) return 0;
    return proj_workspace_bytes(B, L, T, V);
}

int pcfgnat_proj_logsoftmax_gather(const void *hidden, const void *weight, const int64_t *targets,
                                   const int64_t *output_length, const int64_t *target_length, int B, int L, int T,
                                   int V, int H, float *match, float *max_lprob, int64_t *argmax, float *lse,
                                   void *workspace, size_t workspace_bytes, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || T < 0 || V < 1 || H < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if ((long long)B * L > (1ll << 30)) return PCFGNAT_ERR_TOO_LARGE;
    if (B && (!hidden || !weight || !workspace)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (match && (!targets || T < 1)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (target_length != nullptr && output_length == nullptr) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_proj(hidden, weight, targets, output_length, target_length, B, L, T, V, H, match, max_lprob, argmax,
                       lse, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

int pcfgnat_loss_stats(const float *sentence_loss, const int64_t *target_length, int B, float *stats, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || !stats || (B && (!sentence_loss || !target_length))) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_loss_stats(sentence_loss, target_length, B, stats, static_cast<cudaStream_t>(stream));
}

int pcfgnat_loss_stats_exchange(const float *sentence_loss, const int64_t *target_length, int B,
                                const uint64_t *peer_buffers, int rank, int world, float *stats, int *status,
                                void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || !stats || !peer_buffers || world < 1 || world > PCFGNAT_EXCHANGE_MAX_WORLD || rank < 0 || rank >= world ||
        (B && (!sentence_loss || !target_length)))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_loss_stats_exchange(sentence_loss, target_length, B, peer_buffers, rank, world, stats, status,
                                      static_cast<cudaStream_t>(stream));
}

int pcfgnat_glance_select(const int64_t *path, const int64_t *pred_tokens, const int64_t *tgt_tokens,
                          const int64_t *prev_output_tokens, const int64_t *target_length, const float *noise,
                          const float *uniform, int strategy, float context_p, int B, int L, int T, uint8_t *matchmask,
                          int64_t *oracle, int64_t *same_num, int64_t *glance_num, uint8_t *keep, int64_t *glat_prev,
                          void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || T < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (strategy != PCFGNAT_GLANCE_NUMBER_RANDOM && strategy != PCFGNAT_GLANCE_CMLM && strategy != PCFGNAT_GLANCE_FRACTION)
        return PCFGNAT_ERR_UNSUPPORTED;
    if (B && (!path || !pred_tokens || !tgt_tokens || !prev_output_tokens || !target_length || !matchmask || !oracle ||
              !same_num || !glance_num || !keep || !glat_prev))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && strategy != PCFGNAT_GLANCE_FRACTION && !noise) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && strategy != PCFGNAT_GLANCE_NUMBER_RANDOM && !uniform) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_glance_select(path, pred_tokens, tgt_tokens, prev_output_tokens, target_length, noise, uniform,
                                strategy, context_p, B, L, T, matchmask, oracle, same_num, glance_num, keep, glat_prev,
                                static_cast<cudaStream_t>(stream));
}

int pcfgnat_force_emit(const float *match, const uint8_t *matchmask, const uint8_t *keep, int B, int L, int T,
                       float *out, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || T < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!match || !matchmask || !keep || !out)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_force_emit(match, matchmask, keep, B, L, T, out, static_cast<cudaStream_t>(stream));
}

int pcfgnat_force_emit_grad(const float *grad, const uint8_t *keep, int B, int L, int T, float *out, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || T < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!grad || !keep || !out)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_force_emit_grad(grad, keep, B, L, T, out, static_cast<cudaStream_t>(stream));
}

int pcfgnat_copy_links_main_rows(void *dst, const void *src, int B, int L, int max_left, void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 1 || (B && (!dst || !src))) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B == 0) return PCFGNAT_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t row = (size_t)2 * L * sizeof(float);  // links[b][a]: (max_left + 1) x L
    char *d = static_cast<char *>(dst);
    const char *s = static_cast<const char *>(src);
    if (L % 2 == 0)  // odd rows of the flat [B * L] row list are the odd nodes of every sentence
        return cuda_rc(cudaMemcpy2DAsync(d + row, 2 * row, s + row, 2 * row, row, (size_t)B * L / 2, cudaMemcpyDefault, st));
    for (int b = 0; b < B; b++) {
        const size_t off = (size_t)b * L * row + row;
        cudaError_t e = cudaMemcpy2DAsync(d + off, 2 * row, s + off, 2 * row, row, (size_t)L / 2, cudaMemcpyDefault, st);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
    }
    return PCFGNAT_OK;
}

int pcfgnat_plan_real_rows(const int64_t *host_lengths, int b0, int b1, int L, int max_copies, int64_t *runs,
                           int capacity) {
    if (b0 < 0 || b1 < b0 || L < 1 || max_copies < 0 || capacity < 0) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (b1 > b0 && !host_lengths) return PCFGNAT_ERR_INVALID_ARGUMENT;
    const std::vector<std::pair<int64_t, int64_t>> plan = plan_real_rows(host_lengths, b0, b1, L, max_copies);
    if ((size_t)capacity < plan.size() || (plan.size() && !runs)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    for (size_t i = 0; i < plan.size(); i++) runs[2 * i] = plan[i].first, runs[2 * i + 1] = plan[i].second;
    return (int)plan.size();
}

int pcfgnat_copy_real_rows(void *dst, const void *src, const int64_t *host_lengths, int b0, int b1, int L,
                           size_t row_bytes, int max_copies, int64_t *rows_sent, void *stream) {
    PCFGNAT_API_RANGE();
    if (rows_sent) *rows_sent = 0;
    if (b0 < 0 || b1 < b0 || L < 1 || row_bytes == 0 || max_copies < 0) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (b1 > b0 && (!dst || !src || !host_lengths)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    const std::vector<std::pair<int64_t, int64_t>> runs = plan_real_rows(host_lengths, b0, b1, L, max_copies);
    for (const auto &r : runs) {
        const size_t off = (size_t)r.first * row_bytes;
        if (cudaMemcpyAsync(d + off, s + off, (size_t)r.second * row_bytes, cudaMemcpyDefault, st) != cudaSuccess)
            return PCFGNAT_ERR_CUDA;
        if (rows_sent) *rows_sent += r.second;
    }
    return PCFGNAT_OK;
}

int pcfgnat_stage_inputs(const void *hidden_src, void *hidden_dst, int row_bytes, const float *links_src,
                         float *links_dst, const int64_t *output_length, int B, int L, int max_left, void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 2 || row_bytes < 0 || row_bytes % 16) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!output_length || (hidden_src && !hidden_dst) || (links_src && !links_dst))) return PCFGNAT_ERR_INVALID_ARGUMENT;
    // the sources are read by the kernel itself: they must be memory the device can address (mapped pinned host
    // memory, or device memory); what the device sees may differ from the host's pointer
    const void *src[2] = {hidden_src, links_src};
    for (int i = 0; i < 2; i++) {
        if (!src[i]) continue;
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, src[i]) != cudaSuccess) {
            cudaGetLastError();
            return PCFGNAT_ERR_INVALID_ARGUMENT;
        }
        if (at.type == cudaMemoryTypeUnregistered || !at.devicePointer) return PCFGNAT_ERR_INVALID_ARGUMENT;
        src[i] = at.devicePointer;
    }
    if ((reinterpret_cast<uintptr_t>(src[0]) | reinterpret_cast<uintptr_t>(hidden_dst)) % 16) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_stage_inputs(src[0], hidden_dst, row_bytes, static_cast<const float *>(src[1]), links_dst, output_length, B,
                               L, static_cast<cudaStream_t>(stream));
}

int pcfgnat_proj_dlogits(const void *hidden, const void *weight, const int64_t *targets, const int64_t *output_length,
                         const int64_t *target_length, const float *lse, const float *grad_match, int B, int L, int T, int V,
                         int H, void *dlogits, void *workspace, size_t workspace_bytes, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || T < 1 || V < 1 || H < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if ((long long)B * L > (1ll << 30)) return PCFGNAT_ERR_TOO_LARGE;
    if (B && (!hidden || !weight || !targets || !lse || !grad_match || !dlogits || !workspace))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (target_length != nullptr && output_length == nullptr) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_proj_dlogits(hidden, weight, targets, output_length, target_length, lse, grad_match, B, L, T, V, H,
                               dlogits, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

int pcfgnat_proj_dlogits_compact(const void *hidden, const void *weight, const int64_t *targets,
                                 const int64_t *output_length, const int64_t *target_length, const float *lse,
                                 const float *grad_match, int B, int L, int T, int V, int H, int capacity, void *dlogits,
                                 int64_t *row_index, int *n_rows, void *workspace, size_t workspace_bytes, int *status,
                                 void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || L < 1 || T < 1 || V < 1 || H < 1 || capacity < 0) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if ((long long)B * L > (1ll << 30)) return PCFGNAT_ERR_TOO_LARGE;
    if (B && (!hidden || !weight || !targets || !lse || !grad_match || !workspace || !row_index)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && capacity && !dlogits) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (target_length != nullptr && output_length == nullptr) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_proj_dlogits(hidden, weight, targets, output_length, target_length, lse, grad_match, B, L, T, V, H,
                               dlogits, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream), capacity,
                               row_index, n_rows);
}

int pcfgnat_proj_backward_gemms(const void *dlogits, const void *weight_bf16, const void *rows_bf16, int n, int V, int H,
                                float *d_rows, float *d_weight, int *status, void *stream) {
    PCFGNAT_API_RANGE();
    if (n < 0 || V < 1 || H < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if ((long long)n * V > (1ll << 40)) return PCFGNAT_ERR_TOO_LARGE;
    if (n && (!dlogits || (d_rows && !weight_bf16) || (d_weight && !rows_bf16))) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_proj_backward_gemms(dlogits, weight_bf16, rows_bf16, n, V, H, d_rows, d_weight, status,
                                      static_cast<cudaStream_t>(stream));
}

int pcfgnat_links_gather_features(const void *q, const void *kl, const void *kr, int dtype, const int *nodes, int M,
                                  int B, int L, int heads, int head_dim, float *qm, float *klm, float *krm, void *stream) {
    PCFGNAT_API_RANGE();
    if (dtype != PCFGNAT_DTYPE_F32 && dtype != PCFGNAT_DTYPE_F16) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 1 || M < 0 || M > L || heads < 1 || head_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!q || !kl || !kr || !nodes || !qm || !klm || !krm)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_links_gather(q, kl, kr, dtype == PCFGNAT_DTYPE_F16, nodes, M, B, L, heads, head_dim, qm, klm, krm,
                               static_cast<cudaStream_t>(stream));
}

int pcfgnat_links_scores(const float *qm, const float *klm, const float *krm, int M, int B, int heads, int head_dim,
                         float *ac, float *bc, void *stream) {
    PCFGNAT_API_RANGE();
    if (B < 0 || M < 0 || heads < 1 || head_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && M && (!qm || !klm || !krm || !ac || !bc)) return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_links_scores(qm, klm, krm, M, B, heads, head_dim, ac, bc, static_cast<cudaStream_t>(stream));
}

int pcfgnat_links_backward(const float *links_grad, const float *ac, const float *bc, const float *qm, const float *klm,
                           const float *krm, const float *gate_logits, const uint8_t *nonpad,
                           const uint8_t *left_tree_mask, const uint8_t *right_tree_mask, const uint8_t *main_chain,
                           const int *slot_of, const int *nodes, int M, int B, int L, int heads, int head_dim, int max_left,
                           float *X0, float *X1, float *dab, float *dq, float *dkl, float *dkr, float *dgates,
                           void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 1 || M < 0 || M > L || heads < 1 || head_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!links_grad || !ac || !bc || !qm || !klm || !krm || !gate_logits || !nonpad || !left_tree_mask ||
              !right_tree_mask || !main_chain || !slot_of || !nodes || !X0 || !X1 || !dab || !dq || !dkl || !dkr || !dgates))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_links_backward(links_grad, ac, bc, qm, klm, krm, gate_logits, nonpad, left_tree_mask, right_tree_mask,
                                 main_chain, slot_of, nodes, M, B, L, heads, head_dim, X0, X1, dab, dq, dkl, dkr, dgates,
                                 static_cast<cudaStream_t>(stream));
}

int pcfgnat_links_from_scores(const float *ac, const float *bc, const float *qm, const float *klm,
                              const float *gate_logits, const uint8_t *nonpad, const uint8_t *left_tree_mask,
                              const uint8_t *right_tree_mask, const uint8_t *main_chain, const int *slot_of,
                              const int *nodes, int M, int B, int L, int heads, int head_dim, int max_left, float *links,
                              void *stream) {
    PCFGNAT_API_RANGE();
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 1 || M < 0 || M > L || heads < 1 || head_dim < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!ac || !bc || !qm || !klm || !gate_logits || !nonpad || !left_tree_mask || !right_tree_mask || !main_chain ||
              !slot_of || !nodes || !links))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    return launch_links_from_scores(ac, bc, qm, klm, gate_logits, nonpad, left_tree_mask, right_tree_mask, main_chain,
                                    slot_of, nodes, M, B, L, heads, head_dim, links, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
