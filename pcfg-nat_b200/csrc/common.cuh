// Shared helpers of the sm_100a kernels behind include/pcfgnat.h.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/pcfgnat.h"

namespace pcfgnat {

constexpr int kLanes = 4;          // virtual reduction lanes per tree node; the reduction order of the
                                   // sum-semiring tables and all arg-max tie-breaks are defined on them
constexpr int kMaxRows = 256;      // main-chain rows per CTA pass (x kLanes threads)
constexpr int kSmemLimit = 227 * 1024;

__host__ __device__ inline int main_slots(int L, int ml) { return (L - 2) / (ml + 1) + 1; }

// Number of main-chain nodes a = 2*ai+1 that are < m (max_left == 1).
__host__ __device__ inline int main_nodes_below(int m) { return m / 2; }

__device__ __forceinline__ float neg_inf() { return -CUDART_INF_F; }

__device__ __forceinline__ bool lengths_ok(int m, int n, int L, int T) { return m >= 2 && m <= L && n >= 1 && n <= T; }

__device__ __forceinline__ void flag(int *status, int bit) {
    if (status) atomicOr(status, bit);
}

// Per-sentence record the linear-space loss kernels (loss_linear.cu) leave in the workspace: kLinearFrameHead
// floats ([0] u_0[root], [1] log Z, [2] total of the sentence's emission gradients, [3] != 0: marked by the inside
// pass) followed by T + 2 column scales.  A sentence is recomputed by the log-space kernels when it was marked,
// when Z is zero or not finite, or when the emission gradients do not total the n target tokens to 1e-4.
constexpr int kLinearFrameHead = 4;
__device__ __forceinline__ bool linear_needs_redo(const float *fr, int n) {
    return fr[3] != 0.f || !(fr[0] > 0.f) || !(fabsf(fr[1]) < CUDART_INF_F) ||
           !(fabsf(fr[2] - (float)n) <= 1e-4f * (float)n);
}

// exp() through the hardware ex2 approximation (relative error ~1e-6 for the arguments met here): for the
// gradient kernels, whose results are held to 1e-3, never for the tables that must match bit for bit.
__device__ __forceinline__ float fast_exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}

// ---- column exchange without a cluster barrier: a finished node is sent to every CTA of the cluster with
// st.async, which also counts its bytes on a barrier in the receiving CTA; a CTA starts the next step when its
// own barrier has seen the whole column.  Two barriers alternate by step (a CTA can be at most one step
// ahead of a peer: it needs the peer's part of the current column), and the columns roll over four buffers, so
// that the buffer written at step t + 1 is not one that a CTA still at step t reads.  Used by the cluster DP
// kernels (Viterbi, inside pass).
__device__ __forceinline__ uint32_t dsm_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t dsm_map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void dsm_store_async(uint32_t cluster_addr, float v, uint32_t cluster_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(cluster_addr),
                 "r"(__float_as_uint(v)), "r"(cluster_bar)
                 : "memory");
}
// Bounded wait for the column of a step; false when the limit ran out (a peer that never arrives).
__device__ __forceinline__ bool dsm_wait_column(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.b32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? PCFGNAT_OK : PCFGNAT_ERR_CUDA; }

// ---- programmatic dependent launch for the chains of short kernels a step is made of.  A kernel launched with
// launch_chain() may be scheduled while the kernel before it in the stream is still running (PCFGNAT_PDL=1); it
// therefore starts with chain_begin(): wait until that kernel has finished and its memory is visible, then let the
// next kernel of the chain be scheduled in turn.  What is saved is the launch latency between the kernels.  Without
// the launch attribute both instructions do nothing.
__device__ __forceinline__ void chain_begin() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
bool pdl_enabled();  // cabi.cu: PCFGNAT_PDL=1, read once
template <class... KArgs, class... Args>
inline cudaError_t launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Raises a kernel's dynamic shared-memory limit, remembering per device the largest value already
// set so that the steady state costs no driver call (the attribute is sticky per function and device).
cudaError_t ensure_dynamic_smem_for(const void *kernel, size_t bytes);  // cabi.cu; keyed by (function, device)

template <class Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, size_t bytes) {
    return ensure_dynamic_smem_for(reinterpret_cast<const void *>(kernel), bytes);
}

// Host-side launchers shared between the translation units.
int launch_loss_fwd(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                    int T, float *S, float *C, float *loss, int *status, cudaStream_t st);
int launch_loss_bwd(const float *grad_output, const float *S, const float *match_all, const float *links,
                    const int64_t *ol, const int64_t *tl, int B, int L, int T, float *S_grad, float *mg, float *lg,
                    int *status, cudaStream_t st, bool shares_in_mg = false);
int launch_best_tree(const float *S, const float *match_all, const float *links, const int64_t *ol, const int64_t *tl,
                     int B, int L, int T, int64_t *tree, int *status, cudaStream_t st);
int launch_viterbi(const float *ob, const float *links, const int64_t *ol, int B, int L, float *S, int64_t *R,
                   int64_t *Lt, int64_t *Mt, int *status, cudaStream_t st);
int launch_backtrace(const int64_t *pred, const int64_t *ol, const int64_t *Lt, const int64_t *R, const int64_t *Mt,
                     const int64_t *tokens, const int64_t *mask, int mask_dim, int64_t pad, int B, int L, int Q,
                     int cap, int64_t *out, int64_t *cnt, int *status, cudaStream_t st);
int launch_viterbi_decode(const float *S, const float *penalty, const int64_t *ol, const int64_t *Lt, const int64_t *R,
                          const int64_t *Mt, const int64_t *tokens, const int64_t *mask, int mask_dim, int64_t pad, int B,
                          int L, int Q, int cap, int64_t *pred_out, int64_t *out, int64_t *cnt, int *status,
                          cudaStream_t st);
int launch_stage_inputs(const void *hidden_src, void *hidden_dst, int row_bytes, const float *links_src, float *links_dst,
                        const int64_t *ol, int B, int L, cudaStream_t st);
int launch_lookahead_decode(const float *links, const float *ob, const int64_t *tokens, const int64_t *ol,
                            const int64_t *mask, int mask_dim, float beta, int lookahead, int64_t pad, int B, int L,
                            int cap, int64_t *out, int64_t *cnt, int *status, cudaStream_t st);
int launch_logsoftmax_gather(void *logits, int dtype, const int64_t *sel, int64_t sb, int64_t sl, int64_t ss,
                             int64_t rows, int64_t rpb, int V, int slen, int req_grad, float *selected, int *status,
                             cudaStream_t st);

// row-per-thread family on its own; redo != nullptr: only the sentences the linear-space kernels left marked
int launch_loss_fwd_rows(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                         int T, float *S, float *C, float *loss, int *status, cudaStream_t st, const float *redo);
int launch_loss_bwd_rows(const float *grad_output, const float *S, const float *match_all, const float *links,
                         const int64_t *ol, const int64_t *tl, int B, int L, int T, float *S_grad, float *mg, float *lg,
                         int *status, cudaStream_t st, const float *redo);
int launch_grad_rows(const float *S, const float *S_grad, const float *match_all, const float *links, const int64_t *ol,
                     const int64_t *tl, int B, int L, int T, float *mg, float *lg, cudaStream_t st, const float *redo);
// linear-space inside + outside + gradients (loss_linear.cu)
bool linear_dp_applies(int B, int L, int T);
size_t linear_frames_bytes(int B, int T);
int launch_loss_linear(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                       int T, float *Y, float *O, float *frames, float *loss, float *mg, float *lg, int *status,
                       cudaStream_t st);
int mixed_width_count(int B, int Mc);

int launch_loss_fwd_balanced(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B,
                             int L, int T, float *S, float *C, float *loss, int *status, cudaStream_t st);
int launch_outside_balanced(const float *grad_output, const float *S, const float *match_all, const float *links,
                            const int64_t *ol, const int64_t *tl, int B, int L, int T, float *G, float *mg, float *lg,
                            int *status, cudaStream_t st);
int launch_loss_fwd_cluster(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B,
                            int L, int T, float *S, float *C, float *loss, int *status, cudaStream_t st);
int launch_loss_fwd_fast(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                         int T, float *S, float *loss, int *status, cudaStream_t st, float *shares = nullptr);
// Whether the backward pass of this shape runs as the one kernel that takes the emission shares the free-order
// inside pass leaves in match_all_grad (loss_bwd.cu); the inside pass asks before it writes them.
bool fused_grad_applies(int B, int L, int T);
bool outside_balanced_fits_grad(int L);
// mg: the match_all_grad buffer of the backward pass that follows; *shares_in_mg tells whether the emission
// shares were left in it (pass that on to launch_loss_bwd).
int launch_loss_fwd_internal(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B,
                             int L, int T, float *S, float *loss, int *status, cudaStream_t st, float *mg,
                             bool *shares_in_mg);
int loss_fwd_bwd_in(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L, int T,
                    void *tables, size_t table_bytes, float *loss, float *mg, float *lg, int *status, cudaStream_t st);
bool exact_order_forced();  // PCFGNAT_EXACT_ORDER=1: the fused forward + backward also keeps the reference's order
int launch_outside_cluster(const float *grad_output, const float *S, const float *match_all, const float *links,
                           const int64_t *ol, const int64_t *tl, int B, int L, int T, float *G, float *mg, float *lg,
                           int *status, cudaStream_t st);
bool outside_cluster_fits_grad(int B, int L, int T);

// Which family of DP kernels runs the inside / outside passes.  PCFGNAT_DP_KERNEL in the environment
// selects one for A/B runs and tests: "cluster" (default: warp per node, cluster per sentence),
// "balanced" (phase-balanced single CTA), "rows" (4 lanes per node, the only one without a size limit).
// A family that cannot take a shape falls through to the next one in that order.
// Unset (kDpAuto): clusters when cluster_kernels_pay(), else the measured-fastest single-CTA pair
// (row-per-thread inside pass, phase-balanced outside pass).
enum DpKernel { kDpCluster = 0, kDpBalanced = 1, kDpRows = 2, kDpAuto = 3 };
DpKernel dp_kernel_choice();
bool cluster_kernels_pay(int B, int L, int T);
bool inside_mixed_widths_pay(int B, int L, int T);

int launch_loss_stats(const float *loss, const int64_t *tl, int B, float *stats, cudaStream_t st);
int launch_loss_stats_exchange(const float *loss, const int64_t *tl, int B, const uint64_t *peer_bufs, int rank, int world,
                               float *stats, int *status, cudaStream_t st);
int launch_glance_select(const int64_t *path, const int64_t *pred, const int64_t *tgt, const int64_t *prev,
                         const int64_t *tl, const float *noise, const float *uniform, int strategy, float context_p,
                         int B, int L, int T, uint8_t *matchmask, int64_t *oracle, int64_t *same_num,
                         int64_t *glance_num, uint8_t *keep, int64_t *glat_prev, cudaStream_t st);
int launch_force_emit(const float *match, const uint8_t *matchmask, const uint8_t *keep, int B, int L, int T, float *out,
                      cudaStream_t st);
int launch_force_emit_grad(const float *grad, const uint8_t *keep, int B, int L, int T, float *out, cudaStream_t st);

size_t proj_workspace_bytes(int B, int L, int T, int V);
int launch_proj(const void *hidden, const void *weight, const int64_t *targets, const int64_t *ol, const int64_t *tl,
                int B, int L, int T, int V, int H, float *match, float *max_lprob, int64_t *argmax, float *lse,
                void *workspace, size_t ws_bytes, int *status, cudaStream_t st);

int launch_links_gather(const void *q, const void *kl, const void *kr, int is_half, const int *nodes, int M, int B, int L,
                        int H, int D, float *qm, float *klm, float *krm, cudaStream_t st);
int launch_links_scores(const float *qm, const float *klm, const float *krm, int M, int B, int H, int D, float *ac,
                        float *bc, cudaStream_t st);
int launch_links_backward(const float *links_grad, const float *ac, const float *bc, const float *qm, const float *klm,
                          const float *krm, const float *gates, const uint8_t *nonpad, const uint8_t *left_mask,
                          const uint8_t *right_mask, const uint8_t *main_chain, const int *slot_of, const int *nodes, int M,
                          int B, int L, int H, int D, float *X0, float *X1, float *dab, float *dq, float *dkl, float *dkr,
                          float *dgates, cudaStream_t st);
int launch_links_from_scores(const float *ac, const float *bc, const float *qm, const float *klm, const float *gates,
                             const uint8_t *nonpad, const uint8_t *left_mask, const uint8_t *right_mask,
                             const uint8_t *main_chain, const int *slot_of, const int *nodes, int M, int B, int L, int H,
                             int D, float *links, cudaStream_t st);
int launch_proj_dlogits(const void *hidden, const void *weight, const int64_t *targets, const int64_t *ol,
                        const int64_t *tl, const float *lse, const float *grad_match, int B, int L, int T, int V, int H,
                        void *dlogits, void *workspace, size_t ws_bytes, int *status, cudaStream_t st, int capacity = 0,
                        int64_t *row_index = nullptr, int *n_rows_out = nullptr);
int launch_proj_backward_gemms(const void *dlogits, const void *weight_bf16, const void *rows_bf16, int n, int V, int H,
                               float *d_rows, float *d_weight, int *status, cudaStream_t st);

}  // namespace pcfgnat
