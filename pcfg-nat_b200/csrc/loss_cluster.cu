// Inside and outside passes of the PCFG loss, one WARP per tree node and one thread-block CLUSTER
// per sentence (max_left == 1).  Same tables as loss_fwd.cu / loss_bwd.cu.
//
// Why: with 4 lanes per node (the reference's layout) the first node of a sentence walks M/4 right
// children one after the other and sets the time of every dependent step; a single SM also caps the
// step at ~16 us for a 256-node chain.  Here
//   * a warp owns a node: lane l takes the children c = a + l + 32 i, so a step costs ceil(M/32)
//     trips on its critical path instead of M/4;
//   * the nodes of a sentence are dealt round-robin to the 1..16 CTAs of a cluster (one cluster per
//     sentence, sized so that the batch fills the GPU).  Every CTA keeps the rolling S (or G)
//     columns of the WHOLE chain in its shared memory; a warp that finishes a node stores the value
//     into every CTA's copy through distributed shared memory and the cluster meets at a hardware
//     barrier once per step.  Only the links rows of a CTA's own nodes are staged in its shared memory.
//
// Bit-exactness of the inside table (pcfg_loss.cu:149-213): the reference's lane x adds the
// exponentials of children k = 0, 1, 2, ... (c = a + x + 4k), t0 before t1.  Lane l = x + 4h here
// holds k = h + 8i, so after each trip i the eight lanes h = 0..7 of a virtual lane x are visited in
// order with shuffles and every lane keeps the running sum of its virtual lane: the same additions
// in the same order.  Lanes 0..3 are then combined (s0 + s2) + (s1 + s3).  max is order-free.
//
// inside_cluster_kernel<TRIPS > 0> is the inside pass for callers that never see the table (the fused
// forward + backward): same layout, but every lane keeps its own partial sum of exponentials and the warp
// is reduced with a shuffle tree, exp and log are the hardware ex2 / lg2 approximations.  The table then
// agrees with the reference's to a few ulp instead of bit for bit, and the pass costs about a quarter of
// the instructions.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace pcfgnat {

namespace {

constexpr int kCThreads = 1024;
constexpr int kCWarps = kCThreads / 32;

__device__ __forceinline__ float clean(float t) { return isnan(t) ? neg_inf() : t; }

__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Warp maximum with the hardware integer reduction on an order-preserving image of the floats (no NaN).
__device__ __forceinline__ float warp_max_redux(float v) {
    unsigned u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    u = __reduce_max_sync(0xffffffffu, u);
    return __uint_as_float((u & 0x80000000u) ? (u ^ 0x80000000u) : ~u);
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------------------
// inside pass
// ---------------------------------------------------------------------------------------
// One node of the inside pass in the reference's summation order (see the head of this file), for a node
// whose children fit TR trips of 32.  The terms of the first pass (NaN -> -inf already applied; -inf for
// absent children, whose exponential is the reference's +0) stay in registers for the second.
template <int TR>
__device__ __forceinline__ float inside_node_exact(const float *r0, const float *r1, const float *S1, const float *S2,
                                                   int ai, int Mb, int lane, bool has_leaf, float ma0, float ma1,
                                                   float ml) {
    float t0[TR], t1[TR];
    float mx = neg_inf();
#pragma unroll
    for (int i = 0; i < TR; i++) {
        const int ci = ai + lane + 32 * i;
        t0[i] = t1[i] = neg_inf();
        if (ci < Mb) {
            t0[i] = clean((r0[ci] + S1[ci]) + ma0);
            if (t0[i] > mx) mx = t0[i];
            if (has_leaf) {
                t1[i] = clean(((r1[ci] + S2[ci]) + ml) + ma1);
                if (t1[i] > mx) mx = t1[i];
            }
        }
    }
    mx = warp_max(mx);
    if (isinf(mx)) return mx;  // warp-uniform
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < TR; i++) {
        const float e0 = expf(t0[i] - mx), e1 = expf(t1[i] - mx);
        // children k = 8i .. 8i+7 of every virtual lane, in order
#pragma unroll
        for (int h = 0; h < 8; h++) {
            const float v0 = __shfl_sync(0xffffffffu, e0, (lane & 3) + 4 * h);
            const float v1 = __shfl_sync(0xffffffffu, e1, (lane & 3) + 4 * h);
            sum += v0;
            sum += v1;
        }
    }
    sum += __shfl_down_sync(0xffffffffu, sum, 2, 4);  // lanes 0..3 hold the four virtual-lane sums
    sum += __shfl_down_sync(0xffffffffu, sum, 1, 4);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    return logf(sum) + mx;
}

// One node of the inside pass in free summation order; TR trips of 32 children cover the node's children.
// SH: also the shares of the j = 0 terms (returned in lane 0) and of the j = 1 terms (in lane 16) in the
// node's value, which the backward pass turns into emission gradients.
template <int TR, bool SH>
__device__ __forceinline__ float inside_node_free(const float *r0, const float *r1, const float *S1, const float *S2,
                                                  int ai, int Mb, int lane, bool has_leaf, float ma0, float ma1,
                                                  float ml, float &share) {
    constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
    float t0[TR], t1[TR];
    float mx = neg_inf();
#pragma unroll
    for (int i = 0; i < TR; i++) {
        const int ci = ai + lane + 32 * i;
        const bool in = ci < Mb;
        const int cc = in ? ci : ai;
        // fmaxf drops a NaN operand: the reference's NaN -> -inf cleaning
        const float a = fmaxf((r0[cc] + S1[cc]) + ma0, neg_inf());
        const float b = fmaxf(((r1[cc] + S2[cc]) + ml) + ma1, neg_inf());
        t0[i] = in ? a : neg_inf();
        t1[i] = (in && has_leaf) ? b : neg_inf();
        mx = fmaxf(mx, fmaxf(t0[i], t1[i]));
    }
    mx = warp_max_redux(mx);
    if (SH) share = 0.f;
    if (isinf(mx)) return mx;  // warp-uniform
    if (SH) {
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int i = 0; i < TR; i++) {
            sum0 += fast_ex2((t0[i] - mx) * kLog2e);
            sum1 += fast_ex2((t1[i] - mx) * kLog2e);
        }
        const float sum = warp_sum(sum0 + sum1);
        // both partial sums in one tree: after the first round the lower half-warp carries the j = 0 sums and
        // the upper one the j = 1 sums
        const bool upper = lane & 16;
        float v = upper ? sum1 : sum0;
        v += __shfl_xor_sync(0xffffffffu, upper ? sum0 : sum1, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        share = __fdividef(v, sum);
        return fmaf(fast_lg2(sum), kLn2, mx);
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < TR; i++) {  // the difference first: it is small, so its rounding error is too
        sum += fast_ex2((t0[i] - mx) * kLog2e);  // ex2(-inf) = +0
        sum += fast_ex2((t1[i] - mx) * kLog2e);
    }
    sum = warp_sum(sum);
    return fmaf(fast_lg2(sum), kLn2, mx);
}

// TRIPS == 0: the reference's summation order (bit-exact table).  TRIPS > 0: free order, for chains of at
// most 32 * TRIPS main nodes (a lane holds the terms of its TRIPS children in registers between the passes).
// SHARES (free order only): `shares` is a [B][L][T] buffer; the share of the j = 0 terms in S[a][t] goes to
// [a][t] and that of the j = 1 terms to [a-1][t] (the cells of match_all_grad those terms contribute to).  The
// shared memory then holds two more [rows_cap][W] arrays.
template <int TRIPS, bool SHARES = false>
__global__ void __launch_bounds__(kCThreads, 1)
    inside_cluster_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                          const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *S,
                          float *C, float *loss, int *status, int Mc, int Lt, int cs, int rows_cap, int lk_stride,
                          int B, int wide, float *shares) {
    extern __shared__ float smem[];
    cg::cluster_group cluster = cg::this_cluster();
    int crank = (int)cluster.block_rank();  // below: the rank among the CTAs that work on this sentence
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // wide < 0: every sentence gets the whole cluster.  wide >= 0 (batches with more sentences than half the
    // SMs; clusters of two): the sentences are taken in order of decreasing cost m * n, the `wide` costliest get a
    // cluster each and the others share clusters, one CTA per sentence, so that the grid is one CTA per SM: the
    // long sentences, which set the kernel's time, run on two SMs while every sentence still starts at once.
    // (A second CTA that merely left would not make room for clusters still waiting: a new cluster needs both of
    // its SMs free together.)
    int NC = (int)cluster.num_blocks();
    int b = blockIdx.x / NC;
    if (wide >= 0) {
        __shared__ int s_b;
        const int want = b < wide ? b : wide + 2 * (b - wide) + crank;  // the cost rank this CTA serves
        if (want >= B) return;  // the odd CTA of the last shared cluster
        if (b >= wide) {
            NC = 1;
            crank = 0;
        }
        for (int i = tid; i < B; i += kCThreads) {
            const long long mi = ol[i], ni = tl[i];
            const long long ci = lengths_ok((int)mi, (int)ni, L, T) ? mi * ni : 0;
            int before = 0;
            for (int j = 0; j < B; j++) {
                const long long mj = ol[j], nj = tl[j];
                const long long cj = lengths_ok((int)mj, (int)nj, L, T) ? mj * nj : 0;
                before += cj > ci || (cj == ci && j < i);
            }
            if (before == want) s_b = i;
        }
        __syncthreads();
        b = s_b;
    }
    const int ctid = crank * kCThreads + tid, cthreads = NC * kCThreads;  // thread index inside the cluster
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const bool ok = lengths_ok(m, n, L, T);
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    float *Sb = S + (size_t)b * Mc * W;

    for (int i = ctid; i < Mc * W; i += cthreads) Sb[i] = neg_inf();
    if (C) {  // C[0][t][0] = 0 for t <= n; C[leaf slot][t][1] = match[leaf][t] for t < n (pcfg_loss.cu:288-297)
        float *Cb = C + (size_t)b * Lt * W * 3;
        for (int i = ctid; i < Lt * W * 3; i += cthreads) {
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
    if (!ok) {  // uniform over the cluster: nobody reaches a cluster barrier
        if (ctid == 0) {
            flag(status, PCFGNAT_STATUS_BAD_LENGTH);
            if (loss) loss[b] = neg_inf();
        }
        return;
    }
    const int Mb = main_nodes_below(m);
    const int last = (m - 2) / 2;
    const int my_rows = Mb > crank ? (Mb - crank + NC - 1) / NC : 0;  // nodes ai = crank + NC * r
    float *col = smem;                 // [4][cs] rolling S columns of the whole chain (replicated per CTA)
    float *lk0 = col + 4 * cs;         // [rows_cap][lk_stride] links[a][0][c] of this CTA's nodes, by child slot
    float *lk1 = lk0 + (size_t)rows_cap * lk_stride;
    // S entries of this CTA's nodes, flushed to global memory after the last step: a global store
    // inside the step loop would make every cluster barrier (a release) wait for it to reach L2
    float *own = lk1 + (size_t)rows_cap * lk_stride;  // [rows_cap][W]
    // emissions of this CTA's nodes and of their leaves, so that a step reads them from shared memory
    // instead of chasing three global addresses per node
    float *em0 = own + (size_t)rows_cap * W, *eml = em0 + (size_t)rows_cap * W;  // [rows_cap][W] each
    float *own0 = eml + (size_t)rows_cap * W, *own1 = own0 + (size_t)rows_cap * W;  // SHARES only: [rows_cap][W] each
    for (int i = tid; i < my_rows * T; i += kCThreads) {
        const int r = i / T, t = i - r * T, a = 2 * (crank + NC * r) + 1;
        em0[r * W + t] = __ldg(mat + (size_t)a * T + t);
        eml[r * W + t] = a >= 3 ? __ldg(mat + (size_t)(a - 1) * T + t) : 0.f;
    }

    for (int r = warp; r < my_rows; r += kCWarps) {
        const int ai = crank + NC * r;
        const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L;
        for (int ci = ai + lane; ci < Mb; ci += 32) {
            lk0[r * lk_stride + ci] = __ldg(row + 2 * ci + 1);
            lk1[r * lk_stride + ci] = __ldg(row + L + 2 * ci + 1);
        }
    }
    // columns are exchanged with st.async counted on two alternating barriers (common.cuh), not a cluster barrier
    __shared__ __align__(8) uint64_t col_bar[2];
    __shared__ int s_timeout;
    for (int i = tid; i < 4 * cs; i += kCThreads) col[i] = neg_inf();
    if (tid == 0) {
        s_timeout = 0;
        for (int i = 0; i < 2; i++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dsm_smem_u32(&col_bar[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        const float v = __ldg(mat + (size_t)(m - 1) * T + (n - 1));
        col[((n - 1) & 3) * cs + last] = v;  // every CTA fills its own copy
    }
    // all copies initialised before anybody stores into a neighbour's; also orders the -inf fill of the
    // global table (done by threads of any CTA of the cluster) before the cells written below
    if (NC > 1) cluster.sync(); else __syncthreads();
    if (ctid == 0) Sb[(size_t)last * W + (n - 1)] = __ldg(mat + (size_t)(m - 1) * T + (n - 1));

    for (int start = n - 2; start >= 0; start--) {
        const float *S1 = col + ((start + 1) & 3) * cs;
        const float *S2 = col + ((start + 2) & 3) * cs;
        float *S0 = col + (start & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[start & 1]);
        if (NC > 1 && tid == 0)  // this CTA expects the whole column of this step: one value per node of the chain
            asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(4 * Mb)
                         : "memory");
        for (int r = warp; r < my_rows; r += kCWarps) {
            const int ai = crank + NC * r, a = 2 * ai + 1;
            const bool has_leaf = a >= 3;
            const float ma0 = em0[r * W + start];
            const float ma1 = has_leaf ? em0[r * W + start + 1] : 0.f;
            const float ml = eml[r * W + start];  // 0 for the first node, which has no leaf
            const float *r0 = lk0 + r * lk_stride, *r1 = lk1 + r * lk_stride;
            float res;
            if constexpr (TRIPS > 0) {
                // warp-uniform dispatch on the number of trips this node needs: each case is straight-line code
                float share = 0.f;
                switch ((Mb - ai + 31) / 32) {
#define PCFGNAT_NODE(TR) res = inside_node_free<(TR), SHARES>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml, share)
                    case 1: PCFGNAT_NODE(1); break;
                    case 2: PCFGNAT_NODE(2); break;
                    case 3: PCFGNAT_NODE(TRIPS >= 4 ? 3 : TRIPS); break;
                    case 4: PCFGNAT_NODE(TRIPS >= 4 ? 4 : TRIPS); break;
                    case 5:
                    case 6: PCFGNAT_NODE(TRIPS >= 8 ? 6 : TRIPS); break;
                    default: PCFGNAT_NODE(TRIPS); break;
#undef PCFGNAT_NODE
                }
                if (SHARES && (lane & 15) == 0) (lane ? own1 : own0)[r * W + start] = share;
            } else {
            const int trips = (Mb - ai + 31) / 32;
            if (trips <= 8) {  // straight-line code per trip count, terms kept in registers between the passes
                switch (trips) {
                    case 1: res = inside_node_exact<1>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml); break;
                    case 2: res = inside_node_exact<2>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml); break;
                    case 3: res = inside_node_exact<3>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml); break;
                    case 4: res = inside_node_exact<4>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml); break;
                    case 5:
                    case 6: res = inside_node_exact<6>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml); break;
                    default: res = inside_node_exact<8>(r0, r1, S1, S2, ai, Mb, lane, has_leaf, ma0, ma1, ml); break;
                }
            } else {
            float mx = neg_inf();
            for (int i = 0; i < trips; i++) {
                const int ci = ai + lane + 32 * i;
                if (ci < Mb) {
                    const float t0 = clean((r0[ci] + S1[ci]) + ma0);
                    if (t0 > mx) mx = t0;
                    if (has_leaf) {
                        const float t1 = clean(((r1[ci] + S2[ci]) + ml) + ma1);
                        if (t1 > mx) mx = t1;
                    }
                }
            }
            mx = warp_max(mx);
            float sum = 0.f;
            if (!isinf(mx)) {
                for (int i = 0; i < trips; i++) {
                    const int ci = ai + lane + 32 * i;
                    float e0 = 0.f, e1 = 0.f;  // exp(-inf) of the reference's absent / -inf terms
                    if (ci < Mb) {
                        e0 = expf(clean(((r0[ci] + S1[ci]) + ma0) - mx));
                        if (has_leaf) e1 = expf(clean((((r1[ci] + S2[ci]) + ml) + ma1) - mx));
                    }
                    // children k = 8i .. 8i+7 of every virtual lane, in order
#pragma unroll
                    for (int h = 0; h < 8; h++) {
                        const float v0 = __shfl_sync(0xffffffffu, e0, (lane & 3) + 4 * h);
                        const float v1 = __shfl_sync(0xffffffffu, e1, (lane & 3) + 4 * h);
                        sum += v0;
                        sum += v1;
                    }
                }
            }
            sum += __shfl_down_sync(0xffffffffu, sum, 2, 4);  // lanes 0..3 hold the four virtual-lane sums
            sum += __shfl_down_sync(0xffffffffu, sum, 1, 4);
            sum = __shfl_sync(0xffffffffu, sum, 0);
            res = isinf(mx) ? mx : logf(sum) + mx;
            }
            }
            if (NC > 1) {  // into every CTA's column, counted on that CTA's barrier of this step
                if (lane < NC) dsm_store_async(dsm_map_to_cta(dsm_smem_u32(S0 + ai), lane), res, dsm_map_to_cta(bar, lane));
            } else if (lane == 0) {
                S0[ai] = res;
            }
            if (lane == 0) own[r * W + start] = res;
        }
        // one warp waits for the column on the byte-counting barrier, the block barrier releases the others
        if (NC > 1 && warp == kCWarps - 1 && !dsm_wait_column(bar, (((n - 2) - start) >> 1) & 1)) s_timeout = 1;
        __syncthreads();
    }
    if (s_timeout && tid == 0) flag(status, PCFGNAT_STATUS_TIMEOUT);
    // no CTA leaves (its shared memory with it) while a peer may still send to it; every wait above is bounded,
    // so every CTA gets here
    if (NC > 1) cluster.sync();
    for (int i = tid; i < my_rows * (n - 1); i += kCThreads) {  // computed cells: columns 0 .. n-2
        const int r = i / (n - 1), t = i - r * (n - 1);
        Sb[(size_t)(crank + NC * r) * W + t] = own[r * W + t];
    }
    if (SHARES) {
        float *sb = shares + (size_t)b * L * T;
        for (int i = tid; i < my_rows * (n - 1); i += kCThreads) {
            const int r = i / (n - 1), t = i - r * (n - 1), a = 2 * (crank + NC * r) + 1;
            sb[(size_t)a * T + t] = own0[r * W + t];
            if (a >= 3) sb[(size_t)(a - 1) * T + t] = own1[r * W + t];
        }
    }
    if (loss && ctid == 0) loss[b] = (n >= 2) ? col[0] : Sb[0];
}

// ---------------------------------------------------------------------------------------
// outside pass
// ---------------------------------------------------------------------------------------
// GRAD: the kernel also sums up both gradients (the weights of a step are their terms): a (parent, child) pair's
// weights over the steps, in shared memory, give links_grad (same values and order as grad_kernel); the emission
// gradients are G[a][s] times the shares of the j = 0 / j = 1 terms in S[a][s] that the free-order inside kernel
// left in the cells [a][s] / [a-1][s] of match_all_grad.  The dense gradients are zero-filled first.
template <bool GRAD>
__global__ void __launch_bounds__(kCThreads, 1)
    outside_cluster_kernel(const float *__restrict__ grad_output, const float *__restrict__ S,
                           const float *__restrict__ match_all, const float *__restrict__ links,
                           const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *G,
                           float *mg, float *lg, int *status, int Mc, int cs, int rows_cap, int lk_stride) {
    extern __shared__ float smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int NC = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    const int b = blockIdx.x / NC;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ctid = crank * kCThreads + tid, cthreads = NC * kCThreads;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    float *Gb = G + (size_t)b * Mc * W;
    for (int i = ctid; i < Mc * W; i += cthreads) Gb[i] = 0.f;
    float *mgb = GRAD ? mg + (size_t)b * L * T : nullptr;
    float *lgb = GRAD ? lg + (size_t)b * L * 2 * L : nullptr;
    if (GRAD) {
        const size_t n_lg = (size_t)L * 2 * L;
        if ((n_lg & 3) == 0 && (reinterpret_cast<uintptr_t>(lgb) & 15) == 0) {
            for (size_t i = ctid; i < n_lg / 4; i += cthreads) reinterpret_cast<float4 *>(lgb)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (size_t i = ctid; i < n_lg; i += cthreads) lgb[i] = 0.f;
        }
        // emission gradients: every cell that does not hold a share (for an unusable sentence: every cell)
        const int live_rows = lengths_ok(m, n, L, T) ? 2 * main_nodes_below(m) : 0;
        for (int row = ctid / T, t = ctid - row * T; row < L;) {
            const bool share = row >= 1 && row < live_rows && t < n - 1;
            if (!share) mgb[(size_t)row * T + t] = 0.f;
            t += cthreads;
            while (t >= T) {
                t -= T;
                row++;
            }
        }
    }
    if (!lengths_ok(m, n, L, T)) {
        if (ctid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const int Mb = main_nodes_below(m);
    const int my_rows = Mb > crank ? (Mb - crank + NC - 1) / NC : 0;  // children ci = crank + NC * r
    float *gcol = smem;            // [4][cs] rolling G columns of the whole chain (replicated per CTA)
    // per-parent scalars of a step, for the whole chain (every CTA needs all of them), double-buffered: those of
    // step s+1 are fetched from global memory while step s is computed
    float *q0 = gcol + 4 * cs;     // [2][cs] match[a][s] - S[a][s]; -inf where S[a][s] is
    float *q1 = q0 + 2 * cs;       // [2][cs] match[a-1][s] + match[a][s+1] - S[a][s]; -inf without a leaf
    float *lt0 = q1 + 2 * cs;      // [rows_cap][lk_stride] links[a][0][c] of this CTA's children, by parent slot
    float *lt1 = lt0 + (size_t)rows_cap * lk_stride;
    float *own = lt1 + (size_t)rows_cap * lk_stride;  // [rows_cap][W] G entries of this CTA's nodes, flushed at the end
    float *sown = own + (size_t)rows_cap * W;         // [rows_cap][W] inside values of this CTA's nodes
    float *D0 = sown + (size_t)rows_cap * W;          // GRAD only: [rows_cap][lk_stride] weights summed over the steps
    float *D1 = D0 + (size_t)rows_cap * lk_stride;
    // the scalars of parent ai at step s (thread ai computes them; chains of more than kCThreads nodes are not
    // launched with this kernel)
    auto parent_scalars = [&](int ai, int s, float &v0, float &v1) {
        const int a = 2 * ai + 1;
        const float sa = __ldg(Sb + (size_t)ai * W + s);
        const float m0 = __ldg(mat + (size_t)a * T + s);
        v0 = isinf(sa) ? neg_inf() : m0 - sa;
        v1 = neg_inf();
        if (!isinf(sa) && a >= 3) v1 = (__ldg(mat + (size_t)(a - 1) * T + s) + __ldg(mat + (size_t)a * T + s + 1)) - sa;
    };

    for (int r = warp; r < my_rows; r += kCWarps) {
        const int ci = crank + NC * r, c = 2 * ci + 1;
        for (int ai = lane; ai < ci; ai += 32) {
            const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L + c;
            lt0[r * lk_stride + ai] = __ldg(row);
            lt1[r * lk_stride + ai] = __ldg(row + L);
            if (GRAD) {
                D0[r * lk_stride + ai] = 0.f;
                D1[r * lk_stride + ai] = 0.f;
            }
        }
    }
    for (int i = tid; i < my_rows * W; i += kCThreads) {
        const int r = i / W, t = i - r * W;
        sown[i] = __ldg(Sb + (size_t)(crank + NC * r) * W + t);
    }
    // GRAD: thread kCThreads - 1 - r finishes the emission gradients of this CTA's node r
    const int h_r = kCThreads - 1 - tid;
    const bool h_live = GRAD && h_r < my_rows;
    const int h_ai = crank + NC * h_r, h_a = 2 * h_ai + 1;
    float sh0 = 0.f, sh1 = 0.f, carry = 0.f;  // shares of the j = 0 / j = 1 terms in S[h_ai][s]; last step's j = 1 weight
    if (h_live && n >= 2) {
        sh0 = mgb[(size_t)h_a * T];
        if (h_a >= 3) sh1 = mgb[(size_t)(h_a - 1) * T];
    }
    if (tid < Mb && n >= 2) parent_scalars(tid, 0, q0[tid], q1[tid]);
    // columns are exchanged with st.async counted on two alternating barriers (common.cuh), not a cluster barrier
    __shared__ __align__(8) uint64_t col_bar[2];
    for (int i = tid; i < 4 * cs; i += kCThreads) gcol[i] = 0.f;
    if (tid == 0) {
        for (int i = 0; i < 2; i++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dsm_smem_u32(&col_bar[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0) {
        const float go = grad_output ? grad_output[b] : 1.f;
        gcol[0] = go;  // S_grad[0][0] = grad_output (pcfg_loss_backward.cu:78); every CTA fills its own copy
    }
    if (NC > 1) cluster.sync(); else __syncthreads();  // also orders the zero fill of G before the flush below

    bool arrived = true;
    for (int s = 0; s + 1 < n; s++) {
        // four rolling columns: the one that receives the first contributions to column s + 3 at step s + 1 is
        // not the one (column s) that a CTA still at step s reads
        const float *g0 = gcol + (s & 3) * cs;
        float *g1 = gcol + ((s + 1) & 3) * cs;
        float *g2 = gcol + ((s + 2) & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[s & 1]);
        if (NC > 1 && tid == 0)  // this CTA expects two values per node of the chain (columns s + 1 and s + 2)
            asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(8 * Mb)
                         : "memory");
        const float *c0 = q0 + (s & 1) * cs, *c1 = q1 + (s & 1) * cs;
        // the next step's scalars: the loads are in flight while this step's nodes are computed
        float n0 = 0.f, n1 = 0.f;
        const bool fetch = tid < Mb && s + 2 < n;
        if (fetch) parent_scalars(tid, s + 1, n0, n1);
        for (int r = warp; r < my_rows; r += kCWarps) {
            const int ci = crank + NC * r;
            const float sc1 = sown[r * W + s + 1];
            const float sc2 = sown[r * W + s + 2];
            const float *r0 = lt0 + r * lk_stride, *r1 = lt1 + r * lk_stride;
            float acc0 = 0.f, acc1 = 0.f;
            if (!isinf(sc1) || !isinf(sc2)) {
                for (int ai = lane; ai < ci; ai += 32) {
                    const float g = g0[ai];
                    if (g != 0.f) {  // exp(-inf) = 0 where the parent's inside value is -inf
                        const float w0 = g * fast_exp((r0[ai] + sc1) + c0[ai]);
                        const float w1 = g * fast_exp((r1[ai] + sc2) + c1[ai]);
                        acc0 += w0;
                        acc1 += w1;
                        if (GRAD) {  // the slot is this lane's alone
                            D0[r * lk_stride + ai] += w0;
                            D1[r * lk_stride + ai] += w1;
                        }
                    }
                }
            }
            acc0 = warp_sum(acc0);
            acc1 = warp_sum(acc1);
            const float v = g1[ci] + acc0;  // column s+1 is final now (g1[ci] holds the j = 1 part from step s-1)
            __syncwarp();                   // every lane has read g1[ci] before the local copy is overwritten
            if (NC > 1) {
                if (lane < NC) {
                    const uint32_t peer_bar = dsm_map_to_cta(bar, lane);
                    dsm_store_async(dsm_map_to_cta(dsm_smem_u32(g1 + ci), lane), v, peer_bar);
                    dsm_store_async(dsm_map_to_cta(dsm_smem_u32(g2 + ci), lane), acc1, peer_bar);  // first part of column s+2
                }
            } else if (lane == 0) {
                g1[ci] = v;
                g2[ci] = acc1;
            }
            if (lane == 0) own[r * W + s + 1] = v;
        }
        if (fetch) {
            q0[((s + 1) & 1) * cs + tid] = n0;
            q1[((s + 1) & 1) * cs + tid] = n1;
        }
        if (h_live) {
            // j = 0 weights are match[a][s]'s; j = 1 weights are match[a][s+1]'s and match[a-1][s]'s
            // (pcfg_loss_backward.cu:339-382); a share next to a zero G may be anything
            const float g = g0[h_ai];
            const float w0 = g != 0.f ? g * sh0 : 0.f, w1 = g != 0.f ? g * sh1 : 0.f;
            mgb[(size_t)h_a * T + s] = w0 + carry;
            if (h_a >= 3) mgb[(size_t)(h_a - 1) * T + s] = w1;
            carry = w1;
            if (s + 2 < n) {  // shares of the next step
                sh0 = mgb[(size_t)h_a * T + s + 1];
                if (h_a >= 3) sh1 = mgb[(size_t)(h_a - 1) * T + s + 1];
            }
        }
        __syncthreads();  // the next step's scalars are written before any thread of this CTA reads them
        if (NC > 1) arrived = dsm_wait_column(bar, (s >> 1) & 1) && arrived;
    }
    if (!arrived) flag(status, PCFGNAT_STATUS_TIMEOUT);
    if (NC > 1) cluster.sync();  // as in the inside pass: nobody exits while a peer may still send to it
    for (int i = tid; i < my_rows * (n - 1); i += kCThreads) {  // columns 1 .. n-1 of this CTA's nodes
        const int r = i / (n - 1), t = 1 + (i - r * (n - 1));
        Gb[(size_t)(crank + NC * r) * W + t] = own[r * W + t];
    }
    if (ctid == 0) Gb[0] = grad_output ? grad_output[b] : 1.f;
    if (GRAD) {
        if (h_live) {
            // terminal cell: match_all_grad[m-1][n-1] += S_grad[slot of m-1][n-1] (pcfg_loss_backward.cu:379-382);
            // the slot's own row holds no j = 1 weight there (the last node has no children)
            float v = carry;
            if (h_ai == (m - 2) / 2) {
                const float go = grad_output ? grad_output[b] : 1.f;
                const float term = n >= 2 ? own[h_r * W + n - 1] : (h_ai == 0 ? go : 0.f);
                if (h_a == m - 1) v += term;
                else mgb[(size_t)(m - 1) * T + n - 1] = term;  // odd m: an even node
            }
            mgb[(size_t)h_a * T + n - 1] = v;
        }
        for (int r = warp; r < my_rows; r += kCWarps) {
            const int ci = crank + NC * r;
            for (int ai = lane; ai < ci; ai += 32) {
                float *cell = lgb + (size_t)(2 * ai + 1) * 2 * L + (2 * ci + 1);
                cell[0] = D0[r * lk_stride + ai];
                cell[L] = D1[r * lk_stride + ai];
            }
        }
    }
}

struct ClusterGeometry {
    int nc, cs, rows_cap, lk_stride;
    size_t smem_in, smem_out;
};

// Cluster size: the largest power of two <= 16 that still lets all sentences run at once, raised if a
// CTA's share of the links would not fit shared memory; nc = 0 when no size fits.
ClusterGeometry cluster_geometry(int B, int Mc, int W) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    ClusterGeometry g;
    g.cs = (Mc + 3) / 4 * 4;
    g.lk_stride = (Mc + 31) / 32 * 32 + 1;
    int nc = 1;
    // measured on 8 sentences x 256 nodes: 8 CTAs per sentence 1.12 ms, 16 CTAs 1.85 ms (the barrier of a
    // 16-CTA cluster costs more than the extra SMs give), 4 CTAs 1.65 ms: stop at 8
    while (nc < 8 && (long long)B * nc * 2 <= sms && Mc > 8 * nc) nc *= 2;
    if (const char *v = getenv("PCFGNAT_DP_CLUSTER_SIZE")) {  // experiments: 1, 2, 4, 8 or 16
        const int want = atoi(v);
        if (want == 1 || want == 2 || want == 4 || want == 8 || want == 16) nc = want;
    }
    for (;; nc *= 2) {
        g.nc = nc;
        g.rows_cap = (Mc + nc - 1) / nc;
        const size_t lk = (size_t)2 * g.rows_cap * g.lk_stride * sizeof(float);
        const size_t own = (size_t)g.rows_cap * W * sizeof(float);
        g.smem_in = (size_t)4 * g.cs * sizeof(float) + lk + 3 * own;
        g.smem_out = (size_t)8 * g.cs * sizeof(float) + lk + 2 * own;
        if (g.smem_out <= (size_t)kSmemLimit - 1024) break;
        if (nc >= 16) {
            g.nc = 0;
            break;
        }
    }
    return g;
}

template <class Kernel, class... Args>
int launch_cluster(Kernel kernel, int B, int nc, size_t smem, cudaStream_t st, Args... args) {
    if (ensure_dynamic_smem(kernel, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
    if (nc > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return PCFGNAT_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(B * nc));
    cfg.blockDim = dim3(kCThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)nc;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg) != cudaSuccess || max_clusters < 1) {
        cudaGetLastError();
        return PCFGNAT_ERR_UNSUPPORTED;  // this cluster size cannot be scheduled on this GPU
    }
    return cuda_rc(cudaLaunchKernelEx(&cfg, kernel, args...));
}

}  // namespace

// Number of sentences that get both CTAs of a cluster of two when the batch has more sentences than half the
// SMs (so that one cluster size for all would leave SMs idle or sentences waiting), or 0 when that mode does not
// apply: the SMs left over once every sentence has one.
static int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

int mixed_width_count(int B, int Mc) {
    const int sms = sm_count();
    if (B * 2 <= sms || B >= sms || B > 256 || Mc <= 16 || getenv("PCFGNAT_DP_CLUSTER_SIZE")) return 0;
    return sms - B;
}

// True when the inside pass should run on the cluster kernel although cluster_kernels_pay() is false: batches
// between half the SMs and all of them, where the costliest sentences get a second CTA (mixed widths).
bool inside_mixed_widths_pay(int B, int L, int T) {
    const int Mc = main_slots(L, 1);
    const ClusterGeometry g = cluster_geometry(B, Mc, T + 2);
    return g.nc == 1 && mixed_width_count(B, Mc) > 0 && g.smem_in <= (size_t)kSmemLimit - 1024;
}

// True when the batch is small enough that several CTAs per sentence are available (cluster size >= 2),
// or the chain is too long for the single-CTA kernels to keep its links in shared memory.
bool cluster_kernels_pay(int B, int L, int T) {
    const int Mc = main_slots(L, 1);
    const ClusterGeometry g = cluster_geometry(B, Mc, T + 2);
    return g.nc >= 2 || Mc > 160;
}

// Both return PCFGNAT_ERR_UNSUPPORTED when the shape does not fit any cluster size (the caller then
// uses the row-per-thread kernels that read links from global memory).
template <int TRIPS, bool SHARES = false>
int launch_inside(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L, int T,
                  float *S, float *C, float *loss, int *status, cudaStream_t st, float *shares = nullptr) {
    const int Mc = main_slots(L, 1), Lt = L - Mc;
    ClusterGeometry g = cluster_geometry(B, Mc, T + 2);
    for (; g.nc >= 1; g.nc /= 2) {  // fall back to smaller clusters if the GPU cannot co-schedule this size
        g.rows_cap = (Mc + g.nc - 1) / g.nc;
        g.smem_in = ((size_t)4 * g.cs + (size_t)2 * g.rows_cap * g.lk_stride + (size_t)(SHARES ? 5 : 3) * g.rows_cap * (T + 2)) *
                    sizeof(float);
        if (g.smem_in > (size_t)kSmemLimit - 1024) break;
        if (g.nc == 1) {
            // more sentences than half the SMs: clusters of two, which the costliest sentences have to themselves
            // and the others share (see the kernel); every CTA can hold a whole chain, so the shared memory is that of one CTA
            const int wide = mixed_width_count(B, Mc);
            if (wide > 0) {
                int rc = launch_cluster(inside_cluster_kernel<TRIPS, SHARES>, wide + (B - wide + 1) / 2, 2, g.smem_in, st, match_all, links, ol, tl,
                                        L, T, S, C, loss, status, Mc, Lt, g.cs, g.rows_cap, g.lk_stride, B, wide, shares);
                if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
            }
        }
        // more CTAs than SMs: sentences by decreasing cost, so that the clusters that wait for a place get the cheapest
        const int ranked = (long long)B * g.nc > sm_count() && B <= 256 ? B : -1;
        int rc = launch_cluster(inside_cluster_kernel<TRIPS, SHARES>, B, g.nc, g.smem_in, st, match_all, links, ol, tl, L,
                                T, S, C, loss, status, Mc, Lt, g.cs, g.rows_cap, g.lk_stride, B, ranked, shares);
        if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
    }
    return PCFGNAT_ERR_UNSUPPORTED;
}

int launch_loss_fwd_cluster(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B,
                            int L, int T, float *S, float *C, float *loss, int *status, cudaStream_t st) {
    return launch_inside<0>(match_all, links, ol, tl, B, L, T, S, C, loss, status, st);
}

// Inside pass in free summation order (table equal to the reference's to a few ulp, not bit for bit): for
// callers that use the table only to form the loss and the gradients.  PCFGNAT_ERR_UNSUPPORTED when the
// shape does not fit (chains above 256 main nodes, or links beyond the cluster's shared memory).
int launch_loss_fwd_fast(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                         int T, float *S, float *loss, int *status, cudaStream_t st, float *shares) {
    const int Mc = main_slots(L, 1);
    if (shares) {  // [B][L][T]: the shares of the two kinds of terms in every value, for the backward pass
        if (Mc <= 64) return launch_inside<2, true>(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st, shares);
        if (Mc <= 128) return launch_inside<4, true>(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st, shares);
        if (Mc <= 256) return launch_inside<8, true>(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st, shares);
        return PCFGNAT_ERR_UNSUPPORTED;
    }
    if (Mc <= 64) return launch_inside<2>(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st);
    if (Mc <= 128) return launch_inside<4>(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st);
    if (Mc <= 256) return launch_inside<8>(match_all, links, ol, tl, B, L, T, S, nullptr, loss, status, st);
    return PCFGNAT_ERR_UNSUPPORTED;
}

// Shared memory of the outside kernel at the cluster size the geometry picks first, with the gradient sums.
static size_t outside_grad_smem(const ClusterGeometry &g, int T) {
    return ((size_t)8 * g.cs + (size_t)4 * g.rows_cap * g.lk_stride + (size_t)2 * g.rows_cap * (T + 2)) * sizeof(float);
}

bool outside_cluster_fits_grad(int B, int L, int T) {
    const int Mc = main_slots(L, 1);
    if (Mc > kCThreads / 2) return false;  // parents' scalars from the low threads, emission gradients from the high ones
    const ClusterGeometry g = cluster_geometry(B, Mc, T + 2);
    return g.nc >= 2 && outside_grad_smem(g, T) <= (size_t)kSmemLimit - 1024;
}

// mg, lg both given: the kernel also writes both gradients from the emission shares the inside pass left in mg;
// only at the first cluster size (PCFGNAT_ERR_UNSUPPORTED otherwise: the caller then runs the two kernels).
int launch_outside_cluster(const float *grad_output, const float *S, const float *match_all, const float *links,
                           const int64_t *ol, const int64_t *tl, int B, int L, int T, float *G, float *mg, float *lg,
                           int *status, cudaStream_t st) {
    const int Mc = main_slots(L, 1);
    if (Mc > kCThreads) return PCFGNAT_ERR_UNSUPPORTED;  // one thread per parent fetches the step's scalars
    ClusterGeometry g = cluster_geometry(B, Mc, T + 2);
    if (mg && lg) {
        if (!outside_cluster_fits_grad(B, L, T)) return PCFGNAT_ERR_UNSUPPORTED;
        return launch_cluster(outside_cluster_kernel<true>, B, g.nc, outside_grad_smem(g, T), st, grad_output, S, match_all,
                              links, ol, tl, L, T, G, mg, lg, status, Mc, g.cs, g.rows_cap, g.lk_stride);
    }
    for (; g.nc >= 1; g.nc /= 2) {
        g.rows_cap = (Mc + g.nc - 1) / g.nc;
        g.smem_out = ((size_t)8 * g.cs + (size_t)2 * g.rows_cap * g.lk_stride + (size_t)2 * g.rows_cap * (T + 2)) * sizeof(float);
        if (g.smem_out > (size_t)kSmemLimit - 1024) break;
        int rc = launch_cluster(outside_cluster_kernel<false>, B, g.nc, g.smem_out, st, grad_output, S, match_all, links, ol,
                                tl, L, T, G, nullptr, nullptr, status, Mc, g.cs, g.rows_cap, g.lk_stride);
        if (rc != PCFGNAT_ERR_UNSUPPORTED) return rc;
    }
    return PCFGNAT_ERR_UNSUPPORTED;
}

}  // namespace pcfgnat
