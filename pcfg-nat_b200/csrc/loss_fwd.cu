// Inside pass of the PCFG loss for max_left == 1: one CTA per sentence, the whole
// dependency chain over `start` inside the kernel (no inter-CTA waits).
//
// Replaces calculate_C_kernel / calculate_S_kernel of the reference
// (fs_plugins/custom_ops/pcfg_loss.cu:263-349, :85-224).  With max_left == 1 the main-chain
// recurrence has two live terms per right child c (pcfg_loss.cu:154-160 with
// C[null][.][0] = 0, C[leaf][.][1] = match[leaf][.], everything else -inf):
//     t0 = (links[a][0][c] + S[c][start+1]) + match[a][start]
//     t1 = ((links[a][1][c] + S[c][start+2]) + match[a-1][start]) + match[a][start+1]
// The table must be bit-identical to the reference's because the best-tree arg-max
// compares sums built from it, so the reduction order is reproduced exactly: thread
// (x, y) owns row ai = y and right children ci = ai + x + 4k in increasing k, adds
// expf(t0 - max) then expf(t1 - max) sequentially, and the four lanes are combined as
// (s0 + s2) + (s1 + s3); result logf(sum) + max.  No fast-math on this file.
#include "common.cuh"

namespace pcfgnat {

namespace {

struct LinksInSmem {
    const float *p0, *p1;
    int stride;
    __device__ __forceinline__ float k0(int ai, int ci) const { return p0[ai * stride + ci]; }
    __device__ __forceinline__ float k1(int ai, int ci) const { return p1[ai * stride + ci]; }
};

struct LinksInGlobal {
    const float *base;  // links[b], [L][2][L]
    int L;
    __device__ __forceinline__ float k0(int ai, int ci) const {
        return __ldg(base + ((size_t)(2 * ai + 1) * 2 + 0) * L + 2 * ci + 1);
    }
    __device__ __forceinline__ float k1(int ai, int ci) const {
        return __ldg(base + ((size_t)(2 * ai + 1) * 2 + 1) * L + 2 * ci + 1);
    }
};

__device__ __forceinline__ float clean(float t) { return isnan(t) ? neg_inf() : t; }

// One dependent step of the recurrence for the row this thread owns.  The loop over the lane's
// right children is unrolled by kUnroll so that several loads and expf are in flight; children
// past the end contribute -inf terms, i.e. exp() = +0, which leaves max and sum bit-unchanged, and
// the additions still happen in increasing child order, t0 before t1.
constexpr int kUnroll = 4;

template <class Links>
__device__ __forceinline__ float inside_row(const Links &lk, int ai, int x, int Mb, const float *S1, const float *S2,
                                            float ma0, float ma1, float ml, bool has_leaf) {
    float mx = neg_inf();
    for (int base = ai + x; base < Mb; base += kLanes * kUnroll) {
        float t0[kUnroll], t1[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            const int ci = base + kLanes * u;
            const bool in = ci < Mb;
            const int cc = in ? ci : ai;
            const float a = clean((lk.k0(ai, cc) + S1[cc]) + ma0);
            const float b = clean(((lk.k1(ai, cc) + S2[cc]) + ml) + ma1);
            t0[u] = in ? a : neg_inf();
            t1[u] = (in && has_leaf) ? b : neg_inf();
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            if (t0[u] > mx) mx = t0[u];
            if (t1[u] > mx) mx = t1[u];
        }
    }
    // max over the 4 lanes of the row (order-free), then broadcast lane 0's value
    {
        float o = __shfl_down_sync(0xffffffffu, mx, 2, kLanes);
        if (o > mx) mx = o;
        o = __shfl_down_sync(0xffffffffu, mx, 1, kLanes);
        if (o > mx) mx = o;
        mx = __shfl_sync(0xffffffffu, mx, 0, kLanes);
    }
    float sum = 0.f;
    if (!isinf(mx)) {
        for (int base = ai + x; base < Mb; base += kLanes * kUnroll) {
            float e0[kUnroll], e1[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                const int ci = base + kLanes * u;
                const bool in = ci < Mb;
                const int cc = in ? ci : ai;
                const float a = clean(((lk.k0(ai, cc) + S1[cc]) + ma0) - mx);
                const float b = clean((((lk.k1(ai, cc) + S2[cc]) + ml) + ma1) - mx);
                e0[u] = expf(in ? a : neg_inf());
                e1[u] = expf((in && has_leaf) ? b : neg_inf());
            }
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                sum += e0[u];
                sum += e1[u];
            }
        }
    }
    sum += __shfl_down_sync(0xffffffffu, sum, 2, kLanes);
    sum += __shfl_down_sync(0xffffffffu, sum, 1, kLanes);
    return isinf(mx) ? mx : logf(sum) + mx;  // valid on lane x == 0
}

template <bool SMEM_LINKS>
__global__ void __launch_bounds__(kMaxRows *kLanes)
    loss_fwd_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                    const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *S, float *C,
                    float *loss, int *status, int Mc, int Lt, int col_stride, int lk_stride, const float *redo) {
    extern __shared__ float smem[];
    chain_begin();
    const int b = blockIdx.x;
    // redo: only the sentences the linear-space kernels left marked (loss_linear.cu)
    if (redo) {
        if (!linear_needs_redo(redo + (size_t)b * (kLinearFrameHead + T + 2), (int)tl[b])) return;
        if (threadIdx.x == 0 && threadIdx.y == 0) flag(status, PCFGNAT_STATUS_RECOMPUTED);
    }
    const int x = threadIdx.x, y = threadIdx.y;
    const int rows = blockDim.y;
    const int tid = y * kLanes + x, nthr = rows * kLanes;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const bool ok = lengths_ok(m, n, L, T);
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    float *Sb = S + (size_t)b * Mc * W;

    for (int i = tid; i < Mc * W; i += nthr) Sb[i] = neg_inf();
    if (C) {
        // C[0][t][0] = 0 for t <= n; C[leaf slot][t][1] = match[leaf][t] for t < n (pcfg_loss.cu:288-297)
        float *Cb = C + (size_t)b * Lt * W * 3;
        for (int i = tid; i < Lt * W * 3; i += nthr) {
            int g = i % 3, t = (i / 3) % W, a_id = i / (3 * W);
            float v = neg_inf();
            if (ok) {
                if (a_id == 0) {
                    if (g == 0 && t <= n) v = 0.f;
                } else if (g == 1 && 2 * a_id < m && t < n) {
                    v = __ldg(mat + (size_t)(2 * a_id) * T + t);
                }
            }
            Cb[i] = v;
        }
    }
    if (!ok) {
        if (tid == 0) {
            flag(status, PCFGNAT_STATUS_BAD_LENGTH);
            if (loss) loss[b] = neg_inf();
        }
        return;
    }
    const int Mb = main_nodes_below(m);
    const int last = (m - 2) / 2;  // slot of node m-1 (pcfg_loss.cu:144)

    float *col = smem;  // 3 rolling columns of S, indexed by slot
    float *lk0 = smem + 3 * col_stride;
    float *lk1 = lk0 + (size_t)Mc * lk_stride;
    if (SMEM_LINKS) {
        // stage links[a][k][c] for main a, main c >= a:  coalesced row reads, odd columns kept
        for (int i = tid; i < Mb * 2 * L; i += nthr) {
            int c = i % L, k = (i / L) & 1, ai = i / (2 * L);
            int a = 2 * ai + 1;
            if ((c & 1) && c >= a && c < m) {
                float v = __ldg(lkb + ((size_t)a * 2 + k) * L + c);
                (k ? lk1 : lk0)[ai * lk_stride + (c >> 1)] = v;
            }
        }
    }
    // columns n-1 and n
    for (int i = tid; i < Mc; i += nthr) {
        col[((n - 1) % 3) * col_stride + i] = neg_inf();
        col[(n % 3) * col_stride + i] = neg_inf();
    }
    __syncthreads();
    if (tid == 0) {
        float v = __ldg(mat + (size_t)(m - 1) * T + (n - 1));
        col[((n - 1) % 3) * col_stride + last] = v;
        Sb[(size_t)last * W + (n - 1)] = v;
    }
    __syncthreads();

    LinksInSmem ls{lk0, lk1, lk_stride};
    LinksInGlobal lg{lkb, L};
    const int Mpad = (Mb + rows - 1) / rows * rows;
    for (int start = n - 2; start >= 0; start--) {
        const float *S1 = col + ((start + 1) % 3) * col_stride;
        const float *S2 = col + ((start + 2) % 3) * col_stride;
        float *S0 = col + (start % 3) * col_stride;
        for (int ai = y; ai < Mpad; ai += rows) {
            const bool live = ai < Mb;
            const int a = 2 * ai + 1;
            float ma0 = 0.f, ma1 = 0.f, ml = 0.f;
            const bool has_leaf = live && a >= 3;
            if (live) {
                ma0 = __ldg(mat + (size_t)a * T + start);
                if (has_leaf) {
                    ma1 = __ldg(mat + (size_t)a * T + start + 1);
                    ml = __ldg(mat + (size_t)(a - 1) * T + start);
                }
            }
            const int lim = live ? Mb : 0;
            float res = SMEM_LINKS ? inside_row(ls, ai, x, lim, S1, S2, ma0, ma1, ml, has_leaf)
                                   : inside_row(lg, ai, x, lim, S1, S2, ma0, ma1, ml, has_leaf);
            if (live && x == 0) {
                S0[ai] = res;
                Sb[(size_t)ai * W + start] = res;
            }
        }
        // slots >= Mb of this column stay -inf
        for (int i = Mb + tid; i < Mc; i += nthr) S0[i] = neg_inf();
        __syncthreads();
    }
    if (loss && tid == 0) loss[b] = (n >= 2) ? col[0 * col_stride + 0] : Sb[0];
}

}  // namespace

int launch_loss_fwd(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                    int T, float *S, float *C, float *loss, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    // Kernel families, all producing bit-identical tables: warp-per-node clusters (loss_cluster.cu; chosen
    // when few sentences leave several SMs per sentence, or the chain is long), phase-balanced single CTA
    // (loss_balanced.cu, on request only: measured slower here) and the row-per-thread kernel below, which
    // has no size limit because it can read links from global memory.
    const DpKernel choice = dp_kernel_choice();
    if (choice == kDpCluster || (choice == kDpAuto && (cluster_kernels_pay(B, L, T) || inside_mixed_widths_pay(B, L, T)))) {
        const int rc = launch_loss_fwd_cluster(match_all, links, ol, tl, B, L, T, S, C, loss, status, st);
        if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
    }
    if (choice == kDpBalanced) {
        const int rc = launch_loss_fwd_balanced(match_all, links, ol, tl, B, L, T, S, C, loss, status, st);
        if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
    }
    return launch_loss_fwd_rows(match_all, links, ol, tl, B, L, T, S, C, loss, status, st, nullptr);
}

// The row-per-thread kernel (no size limit).  redo != nullptr: only the sentences marked in the frames of the
// linear-space kernels are computed, the others are left untouched.
int launch_loss_fwd_rows(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                         int T, float *S, float *C, float *loss, int *status, cudaStream_t st, const float *redo) {
    if (B == 0) return PCFGNAT_OK;
    const int Mc = main_slots(L, 1), Lt = L - Mc;
    int rows = (Mc + 7) / 8 * 8;
    if (rows < 8) rows = 8;
    if (rows > kMaxRows) rows = kMaxRows;
    const int col_stride = (Mc + 3) / 4 * 4;
    int lk_stride = Mc;
    while (lk_stride % 8 != 3) lk_stride++;  // rows of a warp land in distinct banks
    const size_t smem_cols = (size_t)3 * col_stride * sizeof(float);
    const size_t smem_links = (size_t)2 * Mc * lk_stride * sizeof(float);
    dim3 block(kLanes, rows), grid(B);
    cudaError_t e;
    if (smem_cols + smem_links <= (size_t)kSmemLimit - 1024) {
        auto k = loss_fwd_kernel<true>;
        e = ensure_dynamic_smem(k, smem_cols + smem_links);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        launch_chain(k, grid, block, smem_cols + smem_links, st, match_all, links, ol, tl, L, T, S, C, loss, status, Mc, Lt,
                     col_stride, lk_stride, redo);
    } else {
        if (smem_cols > (size_t)kSmemLimit - 1024) return PCFGNAT_ERR_TOO_LARGE;
        auto k = loss_fwd_kernel<false>;
        e = ensure_dynamic_smem(k, smem_cols);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        launch_chain(k, grid, block, smem_cols, st, match_all, links, ol, tl, L, T, S, C, loss, status, Mc, Lt, col_stride,
                     lk_stride, redo);
    }
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
