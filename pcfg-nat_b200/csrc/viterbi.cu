// Viterbi decode tables (max semiring over output lengths, with backpointers) and the
// back-trace, max_left == 1.
//
// viterbi_kernel replaces calculate_C_kernel / calculate_S_kernel of the reference
// (fs_plugins/custom_ops/pcfg_viterbi.cu:178-241, :23-140): one CTA per sentence loops over
// the output length inside the kernel (the reference spins on a global counter between
// lengths).  With max_left == 1 the two live expansions of node a at length len are
//     t0 = ((links[a][0][c] + 0) + S[c][len-1]) + ob[a]                (j = 0, no left child)
//     t1 = ((links[a][1][c] + ob[a-1]) + S[c][len-2]) + ob[a]          (j = 1, leaf a-1)
// Thread (x, y) owns row id = y and scans c_id = id + x + 4k in increasing k, t0 before t1,
// strict '>'; lanes are merged with shfl_down 2 then 1 under strict '>' — the reference's
// order, so values and backpointers are bit-exact.  Tables are indexed by node id; R, Lt
// hold node ids (Lt = 0 for "no left child"), Mt holds j.
//
// backtrace_kernel replaces the host function viterbi_decoding
// (fs_plugins/custom_ops/pcfg_loss.cpp:12-73): one thread per sentence does the in-order
// walk with an explicit stack, skipping pad tokens and collapsing repeats.
#include "common.cuh"

namespace pcfgnat {

namespace {

template <bool SMEM_LINKS>
__global__ void __launch_bounds__(kMaxRows *kLanes)
    viterbi_kernel(const float *__restrict__ ob_lprob, const float *__restrict__ links,
                   const int64_t *__restrict__ ol, int L, float *S, int64_t *R, int64_t *Lt, int64_t *Mt, int *status,
                   int Mc, int col_stride, int lk_stride) {
    extern __shared__ float smem[];
    const int b = blockIdx.x;
    const int x = threadIdx.x, y = threadIdx.y;
    const int rows = blockDim.y;
    const int tid = y * kLanes + x, nthr = rows * kLanes;
    const int Q = L / 4;
    const int m = (int)ol[b];
    const float *ob = ob_lprob + (size_t)b * L;
    const float *lkb = links + (size_t)b * L * 2 * L;
    float *Sb = S + (size_t)b * L * Q;
    int64_t *Rb = R + (size_t)b * L * Q, *Lb = Lt + (size_t)b * L * Q, *Mb_ = Mt + (size_t)b * L * Q;
    for (int i = tid; i < L * Q; i += nthr) {
        Sb[i] = neg_inf();
        Rb[i] = 0;
        Lb[i] = 0;
        Mb_[i] = 0;
    }
    if (m < 2 || m > L) {
        if (tid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const int Mb = main_nodes_below(m);
    float *col = smem;  // 3 rolling columns of S over main-chain slots
    float *obs = col + 3 * col_stride;  // ob of main node (slot) and of its leaf
    float *obl = obs + col_stride;
    float *lk0 = obl + col_stride;
    float *lk1 = lk0 + (size_t)Mc * lk_stride;
    if (SMEM_LINKS) {
        for (int i = tid; i < Mb * 2 * L; i += nthr) {
            int c = i % L, k = (i / L) & 1, ai = i / (2 * L);
            int a = 2 * ai + 1;
            if ((c & 1) && c >= a && c < m) (k ? lk1 : lk0)[ai * lk_stride + (c >> 1)] = __ldg(lkb + ((size_t)a * 2 + k) * L + c);
        }
    }
    for (int i = tid; i < Mc; i += nthr) {
        col[0 * col_stride + i] = neg_inf();  // length 0
        col[1 * col_stride + i] = neg_inf();  // length 1
        if (i < Mb) {
            obs[i] = __ldg(ob + 2 * i + 1);
            obl[i] = i >= 1 ? __ldg(ob + 2 * i) : neg_inf();  // C[a-1][1] = ob[a-1] (pcfg_viterbi.cu:203-205)
        }
    }
    __syncthreads();
    if (tid == 0) {
        // S[m-1][1] = ob[m-1] (pcfg_viterbi.cu:58); it feeds the recurrence only if m-1 is a main-chain node
        float v = __ldg(ob + (m - 1));
        Sb[(size_t)(m - 1) * Q + 1] = v;
        if ((m - 1) & 1) col[1 * col_stride + (m - 2) / 2] = v;
    }
    __syncthreads();
    const int Mpad = (Mb + rows - 1) / rows * rows;
    for (int len = 2; len < m / 4; len++) {
        const float *S1 = col + ((len - 1) % 3) * col_stride;
        const float *S2 = col + ((len - 2) % 3) * col_stride;
        float *S0 = col + (len % 3) * col_stride;
        for (int id = y; id < Mpad; id += rows) {
            const bool live = id < Mb;
            const int a = 2 * id + 1;
            float best = neg_inf();
            int bc = 0, bj = 0;  // max_c, max_j (max_b follows from j)
            if (live) {
                const float oa = obs[id];
                const float olf = obl[id];
                const bool has_leaf = a >= 3;
                for (int ci = id + x; ci < Mb; ci += kLanes) {
                    float l0, l1;
                    if (SMEM_LINKS) {
                        l0 = lk0[id * lk_stride + ci];
                        l1 = lk1[id * lk_stride + ci];
                    } else {
                        l0 = __ldg(lkb + ((size_t)a * 2 + 0) * L + 2 * ci + 1);
                        l1 = __ldg(lkb + ((size_t)a * 2 + 1) * L + 2 * ci + 1);
                    }
                    float t0 = ((l0 + 0.f) + S1[ci]) + oa;
                    if (isnan(t0)) t0 = neg_inf();
                    if (t0 > best) {
                        best = t0;
                        bc = 2 * ci + 1;
                        bj = 0;
                    }
                    if (has_leaf) {
                        float t1 = ((l1 + olf) + S2[ci]) + oa;
                        if (isnan(t1)) t1 = neg_inf();
                        if (t1 > best) {
                            best = t1;
                            bc = 2 * ci + 1;
                            bj = 1;
                        }
                    }
                }
            }
#pragma unroll
            for (int o = 2; o > 0; o >>= 1) {
                float ov = __shfl_down_sync(0xffffffffu, best, o, kLanes);
                int oc = __shfl_down_sync(0xffffffffu, bc, o, kLanes);
                int oj = __shfl_down_sync(0xffffffffu, bj, o, kLanes);
                if (ov > best) {
                    best = ov;
                    bc = oc;
                    bj = oj;
                }
            }
            if (live && x == 0) {
                S0[id] = best;
                if (!isinf(best)) {
                    size_t o = (size_t)a * Q + len;
                    Sb[o] = best;
                    Lb[o] = bj ? a - 1 : 0;
                    Rb[o] = bc;
                    Mb_[o] = bj;
                }
            }
        }
        for (int i = Mb + tid; i < Mc; i += nthr) S0[i] = neg_inf();
        __syncthreads();
    }
}

__global__ void backtrace_kernel(const int64_t *__restrict__ pred, const int64_t *__restrict__ ol,
                                 const int64_t *__restrict__ Lt, const int64_t *__restrict__ R,
                                 const int64_t *__restrict__ Mt, const int64_t *__restrict__ tokens,
                                 const int64_t *__restrict__ mask, int mask_dim, int64_t pad, int B, int L, int Q,
                                 int cap, int64_t *out, int64_t *cnt, int *status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B) return;
    constexpr int kStack = 32;  // the walk only stacks a node and its left spine: depth <= left_tree_layer + 2
    int stk_node[kStack], stk_len[kStack];
    int sp = 0, count = 0;
    int node = 1, len = (int)pred[i];
    const int max_h = (int)ol[i];
    int64_t last = -1;
    bool bad = false;
    long guard = 0;
    const size_t base = (size_t)i * L * Q;
    int64_t *o = out + (size_t)i * cap;
    while (!bad && ((node < max_h && node != 0) || sp > 0)) {
        while (node < max_h && node != 0) {
            if (node < 0 || node >= L || len < 0 || len >= Q || sp >= kStack || ++guard > 4L * L + 16) {
                bad = true;
                break;
            }
            stk_node[sp] = node;
            stk_len[sp] = len;
            sp++;
            int left = (int)Lt[base + (size_t)node * Q + len];
            if (left == node) left = 0;
            if (left < 0 || left >= mask_dim || node >= mask_dim) {
                bad = true;
                break;
            }
            if (mask[(size_t)node * mask_dim + left]) break;
            int nl = (int)Mt[base + (size_t)node * Q + len];
            node = left;
            len = nl;
        }
        if (bad) break;
        sp--;
        node = stk_node[sp];
        len = stk_len[sp];
        const int64_t tok = tokens[(size_t)i * L + node];
        if (tok != pad && tok != last) {
            last = tok;
            if (count < cap) o[count] = tok;
            count++;
        }
        const int right = (int)R[base + (size_t)node * Q + len];
        const int nl = len - (int)Mt[base + (size_t)node * Q + len] - 1;
        node = right;
        len = nl;
    }
    if (bad) flag(status, PCFGNAT_STATUS_BAD_TRACE);
    cnt[i] = count;
    for (int k = count < cap ? count : cap; k < cap; k++) o[k] = pad;
}

}  // namespace

int launch_viterbi(const float *ob, const float *links, const int64_t *ol, int B, int L, float *S, int64_t *R,
                   int64_t *Lt, int64_t *Mt, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    if (L < 8) return PCFGNAT_ERR_INVALID_ARGUMENT;  // column 1 of an [L][L/4] table must exist
    const int Mc = main_slots(L, 1);
    int rows = (Mc + 7) / 8 * 8;
    if (rows < 8) rows = 8;
    if (rows > kMaxRows) rows = kMaxRows;
    const int col_stride = (Mc + 3) / 4 * 4;
    int lk_stride = Mc;
    while (lk_stride % 8 != 3) lk_stride++;
    const size_t smem_cols = (size_t)5 * col_stride * sizeof(float);
    const size_t smem_links = (size_t)2 * Mc * lk_stride * sizeof(float);
    dim3 block(kLanes, rows), grid(B);
    cudaError_t e;
    if (smem_cols + smem_links <= (size_t)kSmemLimit - 1024) {
        auto k = viterbi_kernel<true>;
        e = ensure_dynamic_smem(k, smem_cols + smem_links);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        k<<<grid, block, smem_cols + smem_links, st>>>(ob, links, ol, L, S, R, Lt, Mt, status, Mc, col_stride,
                                                       lk_stride);
    } else {
        if (smem_cols > (size_t)kSmemLimit - 1024) return PCFGNAT_ERR_TOO_LARGE;
        auto k = viterbi_kernel<false>;
        e = ensure_dynamic_smem(k, smem_cols);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        k<<<grid, block, smem_cols, st>>>(ob, links, ol, L, S, R, Lt, Mt, status, Mc, col_stride, lk_stride);
    }
    return cuda_rc(cudaGetLastError());
}

int launch_backtrace(const int64_t *pred, const int64_t *ol, const int64_t *Lt, const int64_t *R, const int64_t *Mt,
                     const int64_t *tokens, const int64_t *mask, int mask_dim, int64_t pad, int B, int L, int Q,
                     int cap, int64_t *out, int64_t *cnt, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    backtrace_kernel<<<(B + 31) / 32, 32, 0, st>>>(pred, ol, Lt, R, Mt, tokens, mask, mask_dim, pad, B, L, Q, cap, out,
                                                   cnt, status);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
