// Outside pass and gradients of the PCFG loss for max_left == 1.
//
// Replaces the seven backward kernels of the reference
// (fs_plugins/custom_ops/pcfg_loss_backward.cu:29-603) with two:
//
//  1. outside_kernel — the only sequential part (reference K3, :29-121): one CTA per
//     sentence walks `start` upwards and produces the outside weights
//     G[c][t] = dLoss/dS[c][t].  Per step, thread (x, y) owns right child ci = y and parents
//     ai = x + 4k < ci.
//  2. grad_kernel — embarrassingly parallel: one warp per main-chain node a evaluates
//     every weight  w_k(a, c, s) = G[a][s] * exp(term_k - S[a][s])  exactly once and
//     reduces it three ways: over s into links_grad[a][k][c] (registers), over c into the
//     emission gradient of a and of its leaf a-1 (warp shuffles).  The reference evaluates
//     each weight four times in four kernels (K4 :160-209, K6 :326-383, K7 :429-433,
//     K8 :491-533).  Every cell of both dense gradient tensors is written, so the caller
//     does not pre-zero them.
//
// Gradients are compared by tolerance (1e-3 relative), so the summation order here is free.
#include <cstdlib>

#include "common.cuh"

namespace pcfgnat {

namespace {

// ---------------------------------------------------------------------------------------
// 1. outside weights
// ---------------------------------------------------------------------------------------
template <bool SMEM_LINKS>
__global__ void __launch_bounds__(kMaxRows *kLanes)
    outside_kernel(const float *__restrict__ grad_output, const float *__restrict__ S,
                   const float *__restrict__ match_all, const float *__restrict__ links,
                   const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *G, int *status,
                   int Mc, int col_stride, int lk_stride, const float *redo) {
    extern __shared__ float smem[];
    chain_begin();
    const int b = blockIdx.x;
    // redo: only the sentences the linear-space kernels left marked (loss_linear.cu)
    if (redo && !linear_needs_redo(redo + (size_t)b * (kLinearFrameHead + T + 2), (int)tl[b])) return;
    const int x = threadIdx.x, y = threadIdx.y;
    const int rows = blockDim.y;
    const int tid = y * kLanes + x, nthr = rows * kLanes;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    float *Gb = G + (size_t)b * Mc * W;
    for (int i = tid; i < Mc * W; i += nthr) Gb[i] = 0.f;
    if (!lengths_ok(m, n, L, T)) {
        if (tid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const int Mb = main_nodes_below(m);
    // smem: g[3][cs] rolling columns of G | ga[cs], q0[cs], q1[cs] per-parent scalars | transposed links
    float *gcol = smem;
    float *ga = gcol + 3 * col_stride;
    float *q0 = ga + col_stride;
    float *q1 = q0 + col_stride;
    float *lt0 = q1 + col_stride;  // lt0[ci][ai] = links[a][0][c]
    float *lt1 = lt0 + (size_t)Mc * lk_stride;
    if (SMEM_LINKS) {
        for (int i = tid; i < Mb * 2 * L; i += nthr) {
            int c = i % L, k = (i / L) & 1, ai = i / (2 * L);
            int a = 2 * ai + 1;
            if ((c & 1) && c > a && c < m) (k ? lt1 : lt0)[(c >> 1) * lk_stride + ai] = __ldg(lkb + ((size_t)a * 2 + k) * L + c);
        }
    }
    for (int i = tid; i < 3 * col_stride; i += nthr) gcol[i] = 0.f;
    __syncthreads();
    if (tid == 0) {
        float go = grad_output ? grad_output[b] : 1.f;
        gcol[0] = go;  // S_grad[0][0] = grad_output (pcfg_loss_backward.cu:78)
        Gb[0] = go;
    }
    __syncthreads();
    const int Mpad = (Mb + rows - 1) / rows * rows;
    for (int s = 0; s + 1 < n; s++) {
        float *g0 = gcol + (s % 3) * col_stride;
        float *g1 = gcol + ((s + 1) % 3) * col_stride;
        float *g2 = gcol + ((s + 2) % 3) * col_stride;
        // per-parent scalars for this step
        for (int ai = tid; ai < Mb; ai += nthr) {
            int a = 2 * ai + 1;
            float sa = __ldg(Sb + (size_t)ai * W + s);
            float g = g0[ai];
            bool on = g != 0.f && !isinf(sa);
            ga[ai] = on ? g : 0.f;
            float m0 = __ldg(mat + (size_t)a * T + s);
            q0[ai] = on ? m0 - sa : 0.f;
            float v1 = neg_inf();
            if (on && a >= 3 && s + 1 < n)
                v1 = (__ldg(mat + (size_t)(a - 1) * T + s) + __ldg(mat + (size_t)a * T + s + 1)) - sa;
            q1[ai] = v1;
        }
        __syncthreads();
        for (int ci = y; ci < Mpad; ci += rows) {
            float acc0 = 0.f, acc1 = 0.f;
            if (ci < Mb) {
                const float sc1 = __ldg(Sb + (size_t)ci * W + s + 1);
                const float sc2 = __ldg(Sb + (size_t)ci * W + s + 2);
                const bool f1 = !isinf(sc1), f2 = !isinf(sc2);
                const int c = 2 * ci + 1;
                if (f1 || f2) {
                    // 4 parents per trip so that several expf are in flight (summation order is free here)
                    float p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int base = x; base < ci; base += 4 * kLanes) {
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int ai = base + u * kLanes;
                            const bool in = ai < ci;
                            const int aa = in ? ai : 0;
                            const float g = in ? ga[aa] : 0.f;
                            float l0, l1;
                            if (SMEM_LINKS) {
                                l0 = lt0[ci * lk_stride + aa];
                                l1 = lt1[ci * lk_stride + aa];
                            } else {
                                l0 = __ldg(lkb + ((size_t)(2 * aa + 1) * 2 + 0) * L + c);
                                l1 = __ldg(lkb + ((size_t)(2 * aa + 1) * 2 + 1) * L + c);
                            }
                            if (g != 0.f) {
                                if (f1) p0[u] += g * fast_exp((l0 + sc1) + q0[aa]);
                                if (f2) p1[u] += g * fast_exp((l1 + sc2) + q1[aa]);
                            }
                        }
                    }
                    acc0 = (p0[0] + p0[1]) + (p0[2] + p0[3]);
                    acc1 = (p1[0] + p1[1]) + (p1[2] + p1[3]);
                }
            }
            acc0 += __shfl_down_sync(0xffffffffu, acc0, 2, kLanes);
            acc0 += __shfl_down_sync(0xffffffffu, acc0, 1, kLanes);
            acc1 += __shfl_down_sync(0xffffffffu, acc1, 2, kLanes);
            acc1 += __shfl_down_sync(0xffffffffu, acc1, 1, kLanes);
            if (x == 0 && ci < Mb) {
                float v = g1[ci] + acc0;  // column s+1 is final now
                g1[ci] = v;
                Gb[(size_t)ci * W + s + 1] = v;
                g2[ci] = acc1;  // first contribution to column s+2
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// 2. gradients
// ---------------------------------------------------------------------------------------
constexpr int kGradWarps = 8;
// kMaxCPerLane right children per lane and pass over the children: instantiated for 2, 3, 4 and 8, the
// smallest that covers the chain in one pass is launched (longer chains take several passes of 8)

template <int kMaxCPerLane>
__global__ void __launch_bounds__(kGradWarps * 32)
    grad_kernel(const float *__restrict__ S, const float *__restrict__ G, const float *__restrict__ match_all,
                const float *__restrict__ links, const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L,
                int T, float *mg, float *lg, int Mc, const float *redo) {
    extern __shared__ float smem[];  // per warp: 2 rows of T floats (emission gradients of a and a-1)
    chain_begin();
    const int b = blockIdx.y;
    if (redo && !linear_needs_redo(redo + (size_t)b * (kLinearFrameHead + T + 2), (int)tl[b])) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = blockIdx.x * kGradWarps + warp;  // node pair (2p, 2p+1)
    const int npairs = (L + 1) / 2;
    if (p >= npairs) return;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const bool ok = lengths_ok(m, n, L, T);
    const int a = 2 * p + 1, ai = p;
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    const float *Gb = G + (size_t)b * Mc * W;
    float *mgb = mg + (size_t)b * L * T;
    float *lgb = lg + (size_t)b * L * 2 * L;
    float *row_a = smem + (size_t)warp * 2 * T;
    float *row_l = row_a + T;
    for (int t = lane; t < T; t += 32) {
        row_a[t] = 0.f;
        row_l[t] = 0.f;
    }
    __syncwarp();
    const bool live = ok && a < m;
    const int Mb = ok ? main_nodes_below(m) : 0;
    // links_grad rows of the even node 2p are all zero
    for (int i = lane; i < 2 * L; i += 32) lgb[(size_t)(2 * p) * 2 * L + i] = 0.f;
    if (a < L) {
        for (int cbase = ai + 1; cbase == ai + 1 || cbase < Mb; cbase += 32 * kMaxCPerLane) {
            // this lane's right children: ci = cbase + lane + 32 q
            float l0[kMaxCPerLane], l1[kMaxCPerLane], s1[kMaxCPerLane], a0[kMaxCPerLane], a1[kMaxCPerLane];
#pragma unroll
            for (int q = 0; q < kMaxCPerLane; q++) {
                int ci = cbase + lane + 32 * q;
                bool in = live && ci < Mb;
                l0[q] = in ? __ldg(lkb + ((size_t)a * 2 + 0) * L + 2 * ci + 1) : neg_inf();
                l1[q] = in ? __ldg(lkb + ((size_t)a * 2 + 1) * L + 2 * ci + 1) : neg_inf();
                s1[q] = in ? __ldg(Sb + (size_t)ci * W + 1) : neg_inf();  // S[c][s+1] for s = 0
                a0[q] = 0.f;
                a1[q] = 0.f;
            }
            if (live) {
                for (int s = 0; s + 1 < n; s++) {
                    const float g = __ldg(Gb + (size_t)ai * W + s);
                    const float sa = __ldg(Sb + (size_t)ai * W + s);
                    const bool on = g != 0.f && !isinf(sa);  // warp-uniform
                    const float m0 = __ldg(mat + (size_t)a * T + s);
                    float qq0 = m0 - sa, qq1 = neg_inf();
                    if (a >= 3) qq1 = (__ldg(mat + (size_t)(a - 1) * T + s) + __ldg(mat + (size_t)a * T + s + 1)) - sa;
                    float r0 = 0.f, r1 = 0.f;
#pragma unroll
                    for (int q = 0; q < kMaxCPerLane; q++) {
                        int ci = cbase + lane + 32 * q;
                        if (ci < Mb) {
                            float s2 = __ldg(Sb + (size_t)ci * W + s + 2);
                            if (on) {
                                float w0 = isinf(s1[q]) ? 0.f : g * fast_exp((l0[q] + s1[q]) + qq0);
                                float w1 = isinf(s2) ? 0.f : g * fast_exp((l1[q] + s2) + qq1);
                                a0[q] += w0;
                                a1[q] += w1;
                                r0 += w0;
                                r1 += w1;
                            }
                            s1[q] = s2;
                        }
                    }
                    if (on) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            r0 += __shfl_xor_sync(0xffffffffu, r0, o);
                            r1 += __shfl_xor_sync(0xffffffffu, r1, o);
                        }
                        if (lane == 0) {
                            // w0 -> match[a][s]; w1 -> match[a][s+1] and match[a-1][s]
                            // (reference K6 pcfg_loss_backward.cu:360 drops a contribution whose
                            //  own emission is -inf; the product is exactly zero there anyway)
                            row_a[s] += r0;
                            row_a[s + 1] += r1;
                            row_l[s] += r1;
                        }
                    }
                }
            }
            // links_grad rows of node a, this block of right children
#pragma unroll
            for (int q = 0; q < kMaxCPerLane; q++) {
                int ci = cbase + lane + 32 * q;
                if (live && ci < Mb) {
                    lgb[((size_t)a * 2 + 0) * L + 2 * ci + 1] = a0[q];
                    lgb[((size_t)a * 2 + 1) * L + 2 * ci + 1] = a1[q];
                }
            }
        }
        // remaining cells of rows (a, 0) and (a, 1): even columns, columns <= a, columns >= m
        for (int i = lane; i < 2 * L; i += 32) {
            int c = i % L;
            bool computed = live && (c & 1) && c > a && c < m;
            if (!computed) lgb[(size_t)a * 2 * L + i] = 0.f;
        }
    }
    __syncwarp();
    // terminal cell: match_all_grad[m-1][n-1] += S_grad[slot of m-1][n-1] (pcfg_loss_backward.cu:379-382)
    const float term = ok ? __ldg(Gb + (size_t)((m - 2) / 2) * W + (n - 1)) : 0.f;
    // emission gradient rows 2p (leaf) and 2p+1 (main); node 0 and nodes >= m get zeros
    for (int t = lane; t < T; t += 32) {
        float vl = (live && p >= 1) ? row_l[t] : 0.f;
        if (ok && 2 * p == m - 1 && t == n - 1) vl += term;
        mgb[(size_t)(2 * p) * T + t] = vl;
        if (a < L) {
            float va = live ? row_a[t] : 0.f;
            if (ok && a == m - 1 && t == n - 1) va += term;
            mgb[(size_t)a * T + t] = va;
        }
    }
}

}  // namespace

bool fused_grad_applies(int B, int L, int T) {
    const char *fused = std::getenv("PCFGNAT_FUSED_GRAD");  // 0: outside pass, then the gradient kernel
    if (fused && fused[0] == '0') return false;
    const DpKernel choice = dp_kernel_choice();
    if (choice == kDpRows || choice == kDpCluster) return false;
    if (choice == kDpAuto && cluster_kernels_pay(B, L, T)) return outside_cluster_fits_grad(B, L, T);
    return outside_balanced_fits_grad(L);
}

int launch_loss_bwd(const float *grad_output, const float *S, const float *match_all, const float *links,
                    const int64_t *ol, const int64_t *tl, int B, int L, int T, float *S_grad, float *mg, float *lg,
                    int *status, cudaStream_t st, bool shares_in_mg) {
    if (B == 0) return PCFGNAT_OK;
    int brc = PCFGNAT_ERR_UNSUPPORTED;
    const DpKernel choice = dp_kernel_choice();
    if (choice == kDpCluster || (choice == kDpAuto && cluster_kernels_pay(B, L, T))) {  // loss_cluster.cu
        // with the emission shares of the inside pass at hand the same kernel sums up both gradients
        if (shares_in_mg && fused_grad_applies(B, L, T)) {
            const int rc = launch_outside_cluster(grad_output, S, match_all, links, ol, tl, B, L, T, S_grad, mg, lg, status, st);
            if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;  // else: two kernels; the second overwrites the shares
        }
        brc = launch_outside_cluster(grad_output, S, match_all, links, ol, tl, B, L, T, S_grad, nullptr, nullptr, status, st);
    }
    if (brc == PCFGNAT_ERR_UNSUPPORTED && choice != kDpRows) {  // evenly spread phases in one CTA (loss_balanced.cu)
        // with the emission shares of the inside pass at hand the same kernel sums up both gradients
        if (shares_in_mg && fused_grad_applies(B, L, T) && outside_balanced_fits_grad(L)) {
            const int rc = launch_outside_balanced(grad_output, S, match_all, links, ol, tl, B, L, T, S_grad, mg, lg, status, st);
            if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;  // else: two kernels; the second overwrites the shares
        }
        brc = launch_outside_balanced(grad_output, S, match_all, links, ol, tl, B, L, T, S_grad, nullptr, nullptr, status, st);
    }
    if (brc != PCFGNAT_ERR_UNSUPPORTED) {
        if (brc != PCFGNAT_OK) return brc;
        return launch_grad_rows(S, S_grad, match_all, links, ol, tl, B, L, T, mg, lg, st, nullptr);
    }
    return launch_loss_bwd_rows(grad_output, S, match_all, links, ol, tl, B, L, T, S_grad, mg, lg, status, st, nullptr);
}

// Gradient kernel over (S, G).  redo: see launch_loss_bwd_rows.
int launch_grad_rows(const float *S, const float *S_grad, const float *match_all, const float *links, const int64_t *ol,
                     const int64_t *tl, int B, int L, int T, float *mg, float *lg, cudaStream_t st, const float *redo) {
    const int Mc = main_slots(L, 1);
    const int npairs = (L + 1) / 2;
    const size_t gsm = (size_t)kGradWarps * 2 * T * sizeof(float);
    if (gsm > (size_t)kSmemLimit - 1024) return PCFGNAT_ERR_TOO_LARGE;
    dim3 ggrid((npairs + kGradWarps - 1) / kGradWarps, B);
    auto launch = [&](auto kernel) {
        if (ensure_dynamic_smem(kernel, gsm) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        return cuda_rc(launch_chain(kernel, ggrid, dim3(kGradWarps * 32), gsm, st, S, S_grad, match_all, links, ol, tl, L, T,
                                    mg, lg, Mc, redo));
    };
    if (Mc <= 64) return launch(grad_kernel<2>);
    if (Mc <= 96) return launch(grad_kernel<3>);
    if (Mc <= 128) return launch(grad_kernel<4>);
    return launch(grad_kernel<8>);
}

// Outside pass of the row-per-thread family (no size limit) + the gradient kernel.  redo != nullptr: only the
// sentences marked in the frames of the linear-space kernels are computed, the others are left untouched.
int launch_loss_bwd_rows(const float *grad_output, const float *S, const float *match_all, const float *links,
                         const int64_t *ol, const int64_t *tl, int B, int L, int T, float *S_grad, float *mg, float *lg,
                         int *status, cudaStream_t st, const float *redo) {
    if (B == 0) return PCFGNAT_OK;
    const int Mc = main_slots(L, 1);
    int rows = (Mc + 7) / 8 * 8;
    if (rows < 8) rows = 8;
    if (rows > kMaxRows) rows = kMaxRows;
    const int col_stride = (Mc + 3) / 4 * 4;
    int lk_stride = Mc;
    while (lk_stride % 8 != 4) lk_stride++;  // transposed tile: 8 rows x 4 lanes of a warp in distinct banks
    const size_t smem_cols = (size_t)6 * col_stride * sizeof(float);
    const size_t smem_links = (size_t)2 * Mc * lk_stride * sizeof(float);
    dim3 block(kLanes, rows), grid(B);
    cudaError_t e;
    if (smem_cols + smem_links <= (size_t)kSmemLimit - 1024) {
        auto k = outside_kernel<true>;
        e = ensure_dynamic_smem(k, smem_cols + smem_links);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        launch_chain(k, grid, block, smem_cols + smem_links, st, grad_output, S, match_all, links, ol, tl, L, T, S_grad,
                     status, Mc, col_stride, lk_stride, redo);
    } else {
        if (smem_cols > (size_t)kSmemLimit - 1024) return PCFGNAT_ERR_TOO_LARGE;
        auto k = outside_kernel<false>;
        e = ensure_dynamic_smem(k, smem_cols);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        launch_chain(k, grid, block, smem_cols, st, grad_output, S, match_all, links, ol, tl, L, T, S_grad, status, Mc,
                     col_stride, lk_stride, redo);
    }
    if (cudaGetLastError() != cudaSuccess) return PCFGNAT_ERR_CUDA;
    return launch_grad_rows(S, S_grad, match_all, links, ol, tl, B, L, T, mg, lg, st, redo);
}

}  // namespace pcfgnat
