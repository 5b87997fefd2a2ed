// Inside pass, outside pass and both gradients of the PCFG loss in LINEAR space (max_left == 1), for the
// fused forward + backward, whose tables never leave the library (pcfg_loss.cu:149-213 and
// pcfg_loss_backward.cu:58-119 compute the same quantities term by term in log space).
//
// The log-space recurrence  S[a][t] = LSE_c( links[a][0][c] + S[c][t+1] + match[a][t],
//                                            links[a][1][c] + S[c][t+2] + match[a-1][t] + match[a][t+1] )
// costs one exponential per (node, child, term) and step.  With P0 = exp(links[.][0][.]), P1 = exp(links[.][1][.])
// staged once per sentence and E0[a][t] = exp(match[a][t]), E1[a][t] = exp(match[a-1][t] + match[a][t+1]) once per
// cell, a step is two matrix-vector products:
//     s_t[a] = E0[a][t] * sum_c P0[a][c] s_{t+1}[c]  +  E1[a][t] * sum_c P1[a][c] s_{t+2}[c]
// i.e. one fused multiply-add per term and O(M) transcendentals per step instead of O(M^2).
//
// Scaling.  s_t spans hundreds of e-folds over a sentence, so every column is kept relative to the maximum of
// the column computed before it: the kernel stores u_t[a] = s_t[a] / Phi_{t+1}, Phi_t = N_t Phi_{t+1},
// N_t = max_a u_t[a], and the recurrence becomes
//     u_t[a] = E0 inv_{t+1} sum_c P0 u_{t+1}[c] + E1 inv_{t+1} inv_{t+2} sum_c P1 u_{t+2}[c],   inv_t = 1 / N_t.
// Every warp reads the whole column for its dot products anyway, so it takes the column maximum from the same
// registers (one integer warp reduction): no extra exchange, and all warps of all CTAs get the identical N_t.
// log Z = log u_0[root] + sum_t log N_t.
//
// The outside pass needs no inside values in linear space.  With o_t[a] = out_t[a] Phi_{t+1} / Z the posterior
// of a cell is simply o_t[a] u_t[a], and
//     o_{t+1}[c] = inv_{t+1} ( sum_a x0_t[a] P0[a][c] + inv_t sum_a x1_{t-1}[a] P1[a][c] ),
//     x0_t[a] = o_t[a] E0[a][t],  x1_t[a] = o_t[a] E1[a][t],  o_0[root] = 1 / u_0[root]:
// two transposed matrix-vector products per step with the frames the inside pass recorded.  The gradients are
// then sums of products over the steps, which need no dependent chain and run after the loop on all threads:
//     links_grad[a][0][c] = P0[a][c] sum_t x0_t[a] y_{t+1}[c],   y_t[c] = u_t[c] inv_t
//     links_grad[a][1][c] = P1[a][c] sum_t x1_t[a] inv_{t+1} y_{t+2}[c]
//     match_grad[a][t]    = o_t[a] p0_t[a] + o_{t-1}[a] p1_{t-1}[a]      (p0, p1: the two halves of u_t[a])
//     match_grad[a-1][t]  = o_t[a] p1_t[a]
//
// Cells more than ~87 e-folds below their column's maximum flush to zero.  They carry no measurable posterior
// mass in a normal sentence, but the kernels do not rely on that: the outside kernel adds up the emission
// gradients of the sentence, which must total the number of target tokens; when they do not (to 1e-4), when Z
// is zero or not finite, when an input overflowed exp(), or when the lengths are unusual (odd graph length, one
// target token, out of range), the sentence is marked and recomputed by the log-space kernels in the same call
// (loss_fwd.cu / loss_bwd.cu, which skip unmarked sentences).
//
// Layout: one WARP per node, one thread-block CLUSTER per sentence, nodes dealt round-robin to the CTAs; the
// columns are exchanged with st.async counted on alternating mbarriers exactly as in loss_cluster.cu; a lane
// covers four consecutive children with 16-byte shared-memory loads.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace pcfgnat {

namespace {

constexpr int kLThreads = 1024;
constexpr int kLWarps = kLThreads / 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2f(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// exp of a log-probability; NaN counts as -inf (the reference's cleaning of NaN terms, pcfg_loss.cu:162)
__device__ __forceinline__ float exp_clean(float x) { return ex2f(fmaxf(x, neg_inf()) * kLog2e); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// maximum of non-negative floats over the warp: their bit patterns order like unsigned integers
__device__ __forceinline__ float warp_max_nonneg(float v) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
}
__device__ __forceinline__ float dot4(const float4 &a, const float4 &b) {
    return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}

// The sentence of this cluster and the number of its CTAs that work on it (the mixed-width rule of
// loss_cluster.cu: with `wide` >= 0 the clusters take the sentences by decreasing cost and only the `wide`
// costliest use every CTA).  False: this CTA has nothing to do and must return at once.
__device__ __forceinline__ bool pick_sentence(const int64_t *ol, const int64_t *tl, int B, int L, int T, int wide,
                                              int cluster_blocks, int crank, int &b, int &NC) {
    NC = cluster_blocks;
    b = blockIdx.x / cluster_blocks;
    if (wide < 0) return true;
    __shared__ int s_b;
    const int want = b;
    for (int i = threadIdx.x; i < B; i += kLThreads) {
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
    if (want >= wide) {
        if (crank > 0) return false;
        NC = 1;
    }
    return true;
}

__device__ __forceinline__ void bar_init(uint64_t *bars, int count) {
    for (int i = 0; i < count; i++)
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dsm_smem_u32(&bars[i])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void bar_expect(uint32_t bar, int bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------------------------------
// inside pass
// ---------------------------------------------------------------------------------------
// Y      [B][W][Mc]   y_t[c] = u_t[c] inv_t for t = 1 .. n-1 (column-major: a column is contiguous)
// frames [B][F], F = kLinearFrameHead + W:  [0] u_0[root]  [1] log Z  [2] emission-gradient mass (outside pass)
//                     [3] != 0: an input overflowed  [4 + t] inv_t
// shares [B][L][T]    (the match_all_grad buffer) p0_t[a] in cell [a][t], p1_t[a] in cell [a-1][t], t <= n-2
template <int TR>
__global__ void __launch_bounds__(kLThreads, 1)
    inside_linear_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                         const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *Y,
                         float *frames, float *loss, float *shares, int *status, int Mc, int cs, int rows_cap, int B,
                         int wide) {
    extern __shared__ float4 smem4[];
    float *smem = reinterpret_cast<float *>(smem4);
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int b, NC;
    if (!pick_sentence(ol, tl, B, L, T, wide, (int)cluster.num_blocks(), crank, b, NC)) return;
    const int ctid = crank * kLThreads + tid;
    const int W = T + 2, F = kLinearFrameHead + W;
    const int m = (int)ol[b], n = (int)tl[b];
    float *fr = frames + (size_t)b * F;
    // unusual lengths go to the log-space kernels: mark and leave (uniform over the cluster, before any barrier)
    if (!lengths_ok(m, n, L, T) || n < 2 || (m & 1)) {
        if (ctid == 0) {
            fr[0] = 0.f;
            fr[1] = neg_inf();
            fr[2] = 0.f;
            fr[3] = 1.f;
        }
        return;
    }
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const int Mb = m / 2, last = (m - 2) / 2;
    const int my_rows = Mb > crank ? (Mb - crank + NC - 1) / NC : 0;  // nodes ai = crank + NC * r
    float *col = smem;                          // [4][cs] rolling columns of the whole chain (every CTA has a copy)
    float *P0 = col + 4 * cs;                   // [rows_cap][cs] exp(links[a][0][c]) of this CTA's nodes, 0 for c <= a
    float *P1 = P0 + (size_t)rows_cap * cs;
    float *ownu = P1 + (size_t)rows_cap * cs;   // [rows_cap][W] u_t of this CTA's nodes
    float *own0 = ownu + (size_t)rows_cap * W;  // its two halves
    float *own1 = own0 + (size_t)rows_cap * W;
    float *e0 = own1 + (size_t)rows_cap * W;    // [rows_cap][W] E0, E1
    float *e1 = e0 + (size_t)rows_cap * W;
    float *invs = e1 + (size_t)rows_cap * W;    // [W]
    __shared__ __align__(8) uint64_t col_bar[2];
    __shared__ int s_overflow;
    if (tid == 0) s_overflow = 0;
    __syncthreads();

    bool big = false;
    for (int i = tid; i < my_rows * W; i += kLThreads) {
        const int r = i / W, t = i - r * W, a = 2 * (crank + NC * r) + 1;
        float v0 = 0.f, v1 = 0.f;
        if (t < n) {
            const float ma = __ldg(mat + (size_t)a * T + t);
            v0 = exp_clean(ma);
            if (a >= 3 && t + 1 < n)
                v1 = exp_clean(fmaxf(__ldg(mat + (size_t)(a - 1) * T + t), neg_inf()) +
                               fmaxf(__ldg(mat + (size_t)a * T + t + 1), neg_inf()));
        }
        big |= !(v0 < 1e30f) || !(v1 < 1e30f);
        e0[i] = v0;
        e1[i] = v1;
        ownu[i] = 0.f;
    }
    for (int r = warp; r < my_rows; r += kLWarps) {
        const int ai = crank + NC * r;
        const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L;
        for (int ci = lane; ci < cs; ci += 32) {
            float p0 = 0.f, p1 = 0.f;
            if (ci > ai && ci < Mb) {
                p0 = exp_clean(__ldg(row + 2 * ci + 1));
                if (ai >= 1) p1 = exp_clean(__ldg(row + L + 2 * ci + 1));
            }
            big |= !(p0 < 1e30f) || !(p1 < 1e30f);
            P0[(size_t)r * cs + ci] = p0;
            P1[(size_t)r * cs + ci] = p1;
        }
    }
    if (big) s_overflow = 1;
    for (int i = tid; i < 4 * cs; i += kLThreads) col[i] = 0.f;
    for (int i = tid; i < W; i += kLThreads) invs[i] = 0.f;
    if (tid == 0) bar_init(col_bar, 2);
    if (ctid == 0) {
        fr[2] = 0.f;
        fr[3] = 0.f;
    }
    __syncthreads();
    const float base = exp_clean(__ldg(mat + (size_t)(m - 1) * T + (n - 1)));
    if (tid == 0) {
        col[((n - 1) & 3) * cs + last] = base;  // every CTA fills its own copy
        if (last % NC == crank) ownu[(size_t)(last / NC) * W + (n - 1)] = base;
    }
    if (NC > 1) cluster.sync(); else __syncthreads();
    if (s_overflow && tid == 0) fr[3] = 1.f;  // after the reset above (ordered by the barrier)

    bool arrived = true;
    float inv_prev = 0.f, sumlog = 0.f;
    for (int t = n - 2; t >= 0; t--) {
        const float *S1 = col + ((t + 1) & 3) * cs;
        const float *S2 = col + ((t + 2) & 3) * cs;
        float *S0 = col + (t & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[t & 1]);
        if (NC > 1 && tid == 0) bar_expect(bar, 4 * Mb);
        float4 s1[TR], s2[TR];
        float mx = 0.f;
#pragma unroll
        for (int i = 0; i < TR; i++) {
            const int c4 = 4 * lane + 128 * i;
            s1[i] = s2[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c4 < cs) {
                s1[i] = *reinterpret_cast<const float4 *>(S1 + c4);
                s2[i] = *reinterpret_cast<const float4 *>(S2 + c4);
            }
            mx = fmaxf(fmaxf(mx, fmaxf(s1[i].x, s1[i].y)), fmaxf(s1[i].z, s1[i].w));
        }
        const float N1 = warp_max_nonneg(mx);  // N_{t+1}: the same value in every warp of every CTA
        // inv_{t+1}; a column below 1e-36 counts as empty (its reciprocal would leave the range; Z then comes
        // out zero and the sentence is recomputed in log space)
        const float inv1 = N1 > 1e-36f ? __frcp_rn(N1) : 0.f;
        for (int r = warp; r < my_rows; r += kLWarps) {
            const int ai = crank + NC * r;
            const float *p0 = P0 + (size_t)r * cs, *p1 = P1 + (size_t)r * cs;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < TR; i++) {
                const int c4 = 4 * lane + 128 * i;
                if (c4 < cs) {
                    acc0 += dot4(*reinterpret_cast<const float4 *>(p0 + c4), s1[i]);
                    acc1 += dot4(*reinterpret_cast<const float4 *>(p1 + c4), s2[i]);
                }
            }
            acc0 = warp_sum(acc0);
            acc1 = warp_sum(acc1);
            // one scale at a time: the product of two reciprocals can leave the range although the result does not
            const float v0 = e0[(size_t)r * W + t] * (acc0 * inv1);
            const float v1 = e1[(size_t)r * W + t] * ((acc1 * inv_prev) * inv1);
            const float u = v0 + v1;
            if (NC > 1) {  // into every CTA's column, counted on that CTA's barrier of this step
                if (lane < NC) dsm_store_async(dsm_map_to_cta(dsm_smem_u32(S0 + ai), lane), u, dsm_map_to_cta(bar, lane));
            } else if (lane == 0) {
                S0[ai] = u;
            }
            if (lane == 0) {
                ownu[(size_t)r * W + t] = u;
                own0[(size_t)r * W + t] = v0;
                own1[(size_t)r * W + t] = v1;
            }
        }
        if (tid == 0) {
            invs[t + 1] = inv1;
            sumlog += lg2f(N1);
        }
        inv_prev = inv1;
        if (NC > 1) arrived = dsm_wait_column(bar, (((n - 2) - t) >> 1) & 1) && arrived;
        else __syncthreads();
    }
    if (!arrived) flag(status, PCFGNAT_STATUS_TIMEOUT);
    // no CTA leaves (its shared memory with it) while a peer may still send to it; every wait above is bounded
    if (NC > 1) cluster.sync(); else __syncthreads();

    float *Yb = Y + (size_t)b * W * Mc;
    for (int i = tid; i < my_rows * (n - 1); i += kLThreads) {  // columns 1 .. n-1 of this CTA's nodes, normalised
        const int r = i / (n - 1), t = 1 + (i - r * (n - 1));
        Yb[(size_t)t * Mc + (crank + NC * r)] = ownu[(size_t)r * W + t] * invs[t];
    }
    float *sb = shares + (size_t)b * L * T;
    for (int i = tid; i < my_rows * (n - 1); i += kLThreads) {  // the halves of columns 0 .. n-2
        const int r = i / (n - 1), t = i - r * (n - 1), a = 2 * (crank + NC * r) + 1;
        sb[(size_t)a * T + t] = own0[(size_t)r * W + t];
        if (a >= 3) sb[(size_t)(a - 1) * T + t] = own1[(size_t)r * W + t];
    }
    if (crank == 0) {
        for (int t = tid; t < W; t += kLThreads) fr[kLinearFrameHead + t] = invs[t];
        if (tid == 0) {
            const float u00 = ownu[0];  // row 0 of rank 0 is the root, column 0
            const float lz = u00 > 0.f ? (lg2f(u00) + sumlog) * kLn2 : neg_inf();
            fr[0] = arrived ? u00 : 0.f;
            fr[1] = lz;
            if (loss) loss[b] = lz;
        }
    }
}

// ---------------------------------------------------------------------------------------
// outside pass + gradients
// ---------------------------------------------------------------------------------------
// J = children per lane in the links-gradient sums (32 J >= main-chain nodes).
template <int TR>
__global__ void __launch_bounds__(kLThreads, 1)
    outside_linear_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                          const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T,
                          const float *__restrict__ Y, float *O, float *frames, float *mg, float *lg, int *status, int Mc,
                          int cs, int rows_cap, int B, int wide) {
    constexpr int J = 4 * TR;
    extern __shared__ float4 smem4[];
    float *smem = reinterpret_cast<float *>(smem4);
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int b, NC;
    if (!pick_sentence(ol, tl, B, L, T, wide, (int)cluster.num_blocks(), crank, b, NC)) return;
    const int ctid = crank * kLThreads + tid, cthreads = NC * kLThreads;
    const int W = T + 2, F = kLinearFrameHead + W;
    const int m = (int)ol[b], n = (int)tl[b];
    float *fr = frames + (size_t)b * F;
    // what the inside pass marked, or could not finish, is left to the log-space kernels (uniform over the cluster)
    const float u00 = fr[0];
    if (fr[3] != 0.f || !(u00 > 0.f) || !(fabsf(fr[1]) < CUDART_INF_F)) return;
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const int Mb = m / 2, last = (m - 2) / 2;
    const int my_rows = Mb > crank ? (Mb - crank + NC - 1) / NC : 0;  // nodes ci = crank + NC * r
    float *xc0 = smem;                           // [4][cs] rolling columns x0_s of the whole chain
    float *xc1 = xc0 + 4 * cs;                   // [4][cs] x1_s
    float *PT0 = xc1 + 4 * cs;                   // [rows_cap][cs] exp(links[a][0][c]) of this CTA's CHILDREN c, by parent
    float *PT1 = PT0 + (size_t)rows_cap * cs;
    float *owno = PT1 + (size_t)rows_cap * cs;   // [rows_cap][W] o_t of this CTA's nodes
    float *e0 = owno + (size_t)rows_cap * W;     // [rows_cap][W] E0, E1; after the loop x0_t and x1_t inv_{t+1}
    float *e1 = e0 + (size_t)rows_cap * W;
    float *invs = e1 + (size_t)rows_cap * W;     // [W]
    __shared__ __align__(8) uint64_t col_bar[2];
    __shared__ float red[kLWarps];

    for (int i = tid; i < my_rows * W; i += kLThreads) {
        const int r = i / W, t = i - r * W, a = 2 * (crank + NC * r) + 1;
        float v0 = 0.f, v1 = 0.f;
        if (t < n) {
            v0 = exp_clean(__ldg(mat + (size_t)a * T + t));
            if (a >= 3 && t + 1 < n)
                v1 = exp_clean(fmaxf(__ldg(mat + (size_t)(a - 1) * T + t), neg_inf()) +
                               fmaxf(__ldg(mat + (size_t)a * T + t + 1), neg_inf()));
        }
        e0[i] = v0;
        e1[i] = v1;
        owno[i] = 0.f;
    }
    for (int r = warp; r < my_rows; r += kLWarps) {
        const int ci = crank + NC * r;
        for (int ai = lane; ai < cs; ai += 32) {
            float p0 = 0.f, p1 = 0.f;
            if (ai < ci) {
                const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L + (2 * ci + 1);
                p0 = exp_clean(__ldg(row));
                if (ai >= 1) p1 = exp_clean(__ldg(row + L));
            }
            PT0[(size_t)r * cs + ai] = p0;
            PT1[(size_t)r * cs + ai] = p1;
        }
    }
    for (int i = tid; i < 8 * cs; i += kLThreads) xc0[i] = 0.f;  // both column sets
    for (int t = tid; t < W; t += kLThreads) invs[t] = t >= 1 && t < n ? fr[kLinearFrameHead + t] : 0.f;
    if (tid == 0) bar_init(col_bar, 2);
    __syncthreads();
    const float o_root = __frcp_rn(u00);
    if (tid == 0) {
        xc0[0] = o_root * exp_clean(__ldg(mat + (size_t)1 * T + 0));  // x0_0[root]; the root has no left child: x1 = 0
        if (crank == 0) owno[0] = o_root;
    }
    if (NC > 1) cluster.sync(); else __syncthreads();

    bool arrived = true;
    for (int s = 0; s <= n - 2; s++) {  // step s forms column s + 1
        const float *X0 = xc0 + (s & 3) * cs;
        const float *X1 = xc1 + ((s + 3) & 3) * cs;  // column s - 1 (all zero at s = 0)
        float *D0 = xc0 + ((s + 1) & 3) * cs, *D1 = xc1 + ((s + 1) & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[s & 1]);
        if (NC > 1 && tid == 0) bar_expect(bar, 8 * Mb);
        float4 x0[TR], x1[TR];
#pragma unroll
        for (int i = 0; i < TR; i++) {
            const int c4 = 4 * lane + 128 * i;
            x0[i] = x1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c4 < cs) {
                x0[i] = *reinterpret_cast<const float4 *>(X0 + c4);
                x1[i] = *reinterpret_cast<const float4 *>(X1 + c4);
            }
        }
        const float k0 = invs[s + 1], k1 = invs[s];
        for (int r = warp; r < my_rows; r += kLWarps) {
            const int ci = crank + NC * r;
            const float *p0 = PT0 + (size_t)r * cs, *p1 = PT1 + (size_t)r * cs;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < TR; i++) {
                const int c4 = 4 * lane + 128 * i;
                if (c4 < cs) {
                    acc0 += dot4(*reinterpret_cast<const float4 *>(p0 + c4), x0[i]);
                    acc1 += dot4(*reinterpret_cast<const float4 *>(p1 + c4), x1[i]);
                }
            }
            // o_{s+1}[c] = inv_{s+1} (acc0 + inv_s acc1).  o u is a posterior (<= 1), so o only grows beyond 1e30 on
            // cells whose inside value is below 1e-30 of its column: clamped (also NaN), so that no infinity enters
            // the products below; the mass check at the end notices if that ever cost anything
            float o = warp_sum(fmaf(k1, acc1, acc0)) * k0;
            o = o < 1e30f ? o : 1e30f;
            const float n0 = o * e0[(size_t)r * W + s + 1], n1 = o * e1[(size_t)r * W + s + 1];
            if (NC > 1) {
                if (lane < NC) {
                    const uint32_t rb = dsm_map_to_cta(bar, lane);
                    dsm_store_async(dsm_map_to_cta(dsm_smem_u32(D0 + ci), lane), n0, rb);
                    dsm_store_async(dsm_map_to_cta(dsm_smem_u32(D1 + ci), lane), n1, rb);
                }
            } else if (lane == 0) {
                D0[ci] = n0;
                D1[ci] = n1;
            }
            if (lane == 0) owno[(size_t)r * W + s + 1] = o;
        }
        if (NC > 1) arrived = dsm_wait_column(bar, (s >> 1) & 1) && arrived;
        else __syncthreads();
    }
    if (!arrived) flag(status, PCFGNAT_STATUS_TIMEOUT);
    if (NC > 1) cluster.sync(); else __syncthreads();  // nobody exits while a peer may still send to it

    // ---- o table to global memory (the emission gradients of a node need it from whichever CTA sweeps the cell)
    float *Ob = O + (size_t)b * Mc * W;
    for (int i = tid; i < my_rows * n; i += kLThreads) {
        const int r = i / n, t = i - r * n;
        Ob[(size_t)(crank + NC * r) * W + t] = owno[(size_t)r * W + t];
    }
    // x0_t and x1_t inv_{t+1} of this CTA's nodes, now as PARENTS, in place of E0 / E1
    for (int i = tid; i < my_rows * W; i += kLThreads) {
        const int t = i % W;
        const float o = owno[i];
        e0[i] = e0[i] * o;
        e1[i] = (e1[i] * o) * (t + 1 < W ? invs[t + 1] : 0.f);
    }
    __syncthreads();

    // ---- links_grad rows of this CTA's nodes: sums over the steps, J children per lane
    const float *Yb = Y + (size_t)b * W * Mc;
    float *lgb = lg + (size_t)b * L * 2 * L;
    for (int r = warp; r < my_rows; r += kLWarps) {
        const int ai = crank + NC * r, a = 2 * ai + 1;
        float acc0[J], acc1[J], y1[J];
        bool live[J];
#pragma unroll
        for (int j = 0; j < J; j++) {
            const int ci = lane + 32 * j;
            live[j] = ci > ai && ci < Mb;
            acc0[j] = acc1[j] = 0.f;
            y1[j] = live[j] ? __ldg(Yb + (size_t)1 * Mc + ci) : 0.f;
        }
        const float *x0r = e0 + (size_t)r * W, *x1r = e1 + (size_t)r * W;
        for (int t = 0; t <= n - 2; t++) {
            const float x0 = x0r[t], x1 = x1r[t];
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int ci = lane + 32 * j;
                const float y2 = (live[j] && t + 2 <= n - 1) ? __ldg(Yb + (size_t)(t + 2) * Mc + ci) : 0.f;
                acc0[j] = fmaf(x0, y1[j], acc0[j]);
                acc1[j] = fmaf(x1, y2, acc1[j]);
                y1[j] = y2;
            }
        }
        float *row = lgb + (size_t)a * 2 * L;
        const float *lrow = lkb + (size_t)a * 2 * L;
#pragma unroll
        for (int j = 0; j < J; j++) {
            const int ci = lane + 32 * j;
            if (2 * ci < L) {
                row[2 * ci] = 0.f;
                row[L + 2 * ci] = 0.f;
            }
            if (2 * ci + 1 < L) {
                float g0 = 0.f, g1 = 0.f;
                if (live[j]) {
                    g0 = exp_clean(__ldg(lrow + 2 * ci + 1)) * acc0[j];
                    if (ai >= 1) g1 = exp_clean(__ldg(lrow + L + 2 * ci + 1)) * acc1[j];
                }
                row[2 * ci + 1] = g0;
                row[L + 2 * ci + 1] = g1;
            }
        }
        for (int c = 64 * J + lane; c < L; c += 32) {  // columns beyond the main chain's reach (never with L <= 64 J)
            row[c] = 0.f;
            row[L + c] = 0.f;
        }
    }
    // rows of links_grad that belong to no main-chain node in use
    for (int a = crank * kLWarps + warp; a < L; a += NC * kLWarps) {
        if ((a & 1) && a < m) continue;
        float *row = lgb + (size_t)a * 2 * L;
        for (int c = lane; c < 2 * L; c += 32) row[c] = 0.f;
    }

    // ---- emission gradients, pass 1: every cell times the o of its main-chain node (cells without a share: 0)
    if (NC > 1) cluster.sync(); else __syncthreads();  // the o table is complete
    float *mgb = mg + (size_t)b * L * T;
    for (int i = ctid; i < L * T; i += cthreads) {
        const int node = i / T, t = i - node * T;
        float v = 0.f;
        if (node >= 1 && node < m && t <= n - 2) {
            const int a = node | 1;  // the main-chain node of the cell: itself, or the parent of the leaf
            if (a < m && (node & 1 || node >= 2)) v = mgb[i] * Ob[(size_t)((a - 1) / 2) * W + t];
        }
        mgb[i] = v;
    }
    if (NC > 1) cluster.sync(); else __syncthreads();
    // pass 2: a node that emitted y_t after its leaf emitted y_{t-1} (the same posterior), the terminal cell, and
    // the total mass of the sentence's emission gradients (= n when nothing was lost)
    float mass = 0.f;
    for (int i = ctid; i < L * T; i += cthreads) {
        const int node = i / T, t = i - node * T;
        if (node >= m || t >= n) continue;
        float v = mgb[i];
        if ((node & 1) && node >= 3 && t >= 1) v += mgb[(size_t)(node - 1) * T + t - 1];
        if (node == m - 1 && t == n - 1) v += Ob[(size_t)last * W + n - 1] * (invs[n - 1] > 0.f ? __frcp_rn(invs[n - 1]) : 0.f);
        if ((node & 1) && t >= 1) mgb[i] = v;
        mass += v;
    }
    mass = warp_sum(mass);
    if (lane == 0) red[warp] = mass;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.f;
        for (int i = 0; i < kLWarps; i++) tot += red[i];
        atomicAdd(fr + 2, tot);
    }
}

struct LinearGeometry {
    int nc, cs, rows_cap, wide;
    size_t smem_in, smem_out;
};

// Cluster size as for the log-space cluster kernels: the largest power of two <= 8 that lets all sentences run
// at once, raised while a CTA's share of the matrices does not fit shared memory; nc = 0: no size fits.
LinearGeometry linear_geometry(int B, int Mc, int W) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    LinearGeometry g;
    g.cs = (Mc + 3) / 4 * 4;
    g.wide = -1;
    int nc = 1;
    while (nc < 8 && (long long)B * nc * 2 <= sms && Mc > 8 * nc) nc *= 2;
    if (const char *v = getenv("PCFGNAT_DP_CLUSTER_SIZE")) {
        const int want = atoi(v);
        if (want == 1 || want == 2 || want == 4 || want == 8 || want == 16) nc = want;
    }
    for (;; nc *= 2) {
        g.nc = nc;
        g.rows_cap = (Mc + nc - 1) / nc;
        const size_t mat = (size_t)2 * g.rows_cap * g.cs, own = (size_t)g.rows_cap * W;
        g.smem_in = ((size_t)4 * g.cs + mat + 5 * own + W) * sizeof(float);
        g.smem_out = ((size_t)8 * g.cs + mat + 3 * own + W) * sizeof(float);
        if (g.smem_in <= (size_t)kSmemLimit - 1024 && g.smem_out <= (size_t)kSmemLimit - 1024) break;
        if (nc >= 16) {
            g.nc = 0;
            break;
        }
    }
    if (g.nc == 1) {
        const int wide = mixed_width_count(B, Mc);
        if (wide > 0) g.wide = wide;
    }
    return g;
}

template <class Kernel, class... Args>
int launch_linear_cluster(Kernel kernel, int B, int nc, size_t smem, cudaStream_t st, Args... args) {
    if (ensure_dynamic_smem(kernel, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
    if (nc > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return PCFGNAT_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(B * nc));
    cfg.blockDim = dim3(kLThreads);
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
        return PCFGNAT_ERR_UNSUPPORTED;
    }
    return cuda_rc(cudaLaunchKernelEx(&cfg, kernel, args...));
}

template <int TR>
int launch_linear(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L, int T,
                  float *Y, float *O, float *frames, float *loss, float *mg, float *lg, int *status, cudaStream_t st) {
    const int Mc = main_slots(L, 1);
    const LinearGeometry g = linear_geometry(B, Mc, T + 2);
    if (g.nc == 0) return PCFGNAT_ERR_UNSUPPORTED;
    const int nc = g.wide >= 0 ? 2 : g.nc;  // mixed widths: clusters of two of which only the costliest use both CTAs
    int rc = launch_linear_cluster(inside_linear_kernel<TR>, B, nc, g.smem_in, st, match_all, links, ol, tl, L, T, Y, frames,
                                   loss, mg, status, Mc, g.cs, g.rows_cap, B, g.wide);
    if (rc) return rc;
    return launch_linear_cluster(outside_linear_kernel<TR>, B, nc, g.smem_out, st, match_all, links, ol, tl, L, T,
                                 (const float *)Y, O, frames, mg, lg, status, Mc, g.cs, g.rows_cap, B, g.wide);
}

}  // namespace

bool linear_dp_applies(int B, int L, int T) {
    if (B == 0) return false;
    if (const char *v = getenv("PCFGNAT_LINEAR_DP"))
        if (v[0] == '0') return false;
    const int Mc = main_slots(L, 1);
    if (Mc > 256) return false;
    return linear_geometry(B, Mc, T + 2).nc != 0;
}

size_t linear_frames_bytes(int B, int T) {
    return ((size_t)B * (kLinearFrameHead + T + 2) * sizeof(float) + 255) / 256 * 256;
}

// Inside pass, outside pass and both gradients of every sentence the linear-space kernels can take; the others
// are left marked in `frames` for the log-space kernels (launch_loss_redo).  PCFGNAT_ERR_UNSUPPORTED: nothing
// was launched.
int launch_loss_linear(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B, int L,
                       int T, float *Y, float *O, float *frames, float *loss, float *mg, float *lg, int *status,
                       cudaStream_t st) {
    const int Mc = main_slots(L, 1);
    if (Mc <= 128) return launch_linear<1>(match_all, links, ol, tl, B, L, T, Y, O, frames, loss, mg, lg, status, st);
    if (Mc <= 256) return launch_linear<2>(match_all, links, ol, tl, B, L, T, Y, O, frames, loss, mg, lg, status, st);
    return PCFGNAT_ERR_UNSUPPORTED;
}

}  // namespace pcfgnat
