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
// Scaling.  s_t spans hundreds of e-folds over a sentence, so every column is stored with a scale of its own:
// the kernel keeps u_t[a] = s_t[a] / G_t, G_t = G_{t+1} / rho_t, and the recurrence becomes
//     u_t[a] = rho_t ( E0 sum_c P0 u_{t+1}[c] + rho_{t+1} E1 sum_c P1 u_{t+2}[c] ).
// Any positive rho_t that all warps agree on is exact; it only has to keep the numbers in range.  rho_t is
// taken from the maximum of column t + 2 (column_scale), which every warp reads off the finished column one
// step ahead of need, after its own nodes of the step are on their way: finding it costs the chain of dependent
// steps nothing, and all warps of all CTAs get the identical value.  log Z = log u_0[root] - sum_t log rho_t.
// (In the code inv_{t+1} names rho_t.)
//
// The outside pass needs no inside values in linear space.  With o_t[a] = out_t[a] G_t / Z the posterior
// of a cell is simply o_t[a] u_t[a], and
//     o_{t+1}[c] = rho_t ( sum_a x0_t[a] P0[a][c] + rho_{t-1} sum_a x1_{t-1}[a] P1[a][c] ),
//     x0_t[a] = o_t[a] E0[a][t],  x1_t[a] = o_t[a] E1[a][t],  o_0[root] = 1 / u_0[root]:
// two transposed matrix-vector products per step with the frames the inside pass recorded.  The gradients are
// then sums of products over the steps, which need no dependent chain and run after the loop on all threads:
//     links_grad[a][0][c] = P0[a][c] sum_t x0_t[a] y_{t+1}[c],   y_t[c] = u_t[c] rho_{t-1}
//     links_grad[a][1][c] = P1[a][c] sum_t x1_t[a] rho_t y_{t+2}[c]
//     match_grad[a][t]    = o_t[a] p0_t[a] + o_{t-1}[a] p1_{t-1}[a]      (p0, p1: the two halves of u_t[a])
//     match_grad[a-1][t]  = o_t[a] p1_t[a]
//
// Cells some 60 e-folds below their column's maximum flush to zero.  They carry no measurable posterior
// mass in a normal sentence, but the kernels do not rely on that: the outside kernel adds up the emission
// gradients of the sentence, which must total the number of target tokens; when they do not (to 1e-4), when Z
// is zero or not finite, when an input overflowed exp(), or when the lengths are unusual (odd graph length, one
// target token, out of range), the sentence is marked and recomputed by the log-space kernels in the same call
// (loss_fwd.cu / loss_bwd.cu, which skip unmarked sentences).
//
// Layout: G = 8 or 16 lanes per node (a lane covers groups of four consecutive children, its part of the node's
// matrix rows in registers), one thread-block CLUSTER per sentence, nodes dealt round-robin to the CTAs; the
// columns are exchanged with st.async counted on alternating mbarriers exactly as in loss_cluster.cu.  Batches
// between half and all of the SMs run clusters of two, which the costliest sentences have to themselves and the
// others share, one CTA per sentence (pick_sentence).
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

// Development aid, compiled out of the library: with -DPCFGNAT_TIMING the first thread of every sentence's first
// CTA records clock64() stamps of the kernel's phases.
#ifdef PCFGNAT_TIMING
__device__ long long g_linear_timing[2][256][16];
#define PCFGNAT_STAMP(k, i) \
    if (tid == 0 && crank == 0 && b < 256) g_linear_timing[k][b][i] = clock64();
#define PCFGNAT_ACC(k, i, v) \
    if (tid == 0 && crank == 0 && b < 256) g_linear_timing[k][b][i] += (v);
extern "C" int pcfgnat_debug_linear_timing(long long *host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_linear_timing, sizeof(g_linear_timing));
}
extern "C" int pcfgnat_debug_linear_timing_reset() {
    static long long zeros[2 * 256 * 16];
    return (int)cudaMemcpyToSymbol(g_linear_timing, zeros, sizeof(zeros));
}
#else
#define PCFGNAT_STAMP(k, i)
#define PCFGNAT_ACC(k, i, v)
#endif

namespace pcfgnat {

namespace {

constexpr int kLThreads = 512;
constexpr int kLWarps = kLThreads / 32;
constexpr int kMaxMixedBatch = 256;                // mixed cluster widths only up to this many sentences (mixed_width_count)
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
// Scale applied to column t, from the maximum m of column t + 2 (known a whole step earlier, so that finding it
// is not on the chain of dependent steps): m^(-3/4).  With x_t = log max of column t the columns then follow
// x_t = e_t + x_{t+1} - 0.75 x_{t+2} (e_t: log of a typical emission x transition), a damped recurrence: the maxima
// settle around exp(4/3 e) instead of drifting, with fluctuations of the order of those of e_t.  A column below
// 1e-36 counts as empty (Z then comes out zero and the sentence is recomputed in log space).
__device__ __forceinline__ float column_scale(float m) { return m > 1e-36f ? ex2f(-0.75f * lg2f(m)) : 0.f; }
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

// Floats the outside kernel keeps in front of its step-loop memory (E0, E1 and the column scales), a multiple of 4.
__host__ __device__ inline int linear_outside_head(int rows_cap, int W) { return (2 * rows_cap * W + W + 3) & ~3; }

// The sentence of this CTA, the number of CTAs that work on it and this CTA's rank among them.  wide < 0: cluster
// k takes sentence k with all its CTAs.  wide >= 0: the sentences are taken by decreasing cost; the `wide`
// costliest get a cluster each, the others (clusters of two only) share clusters, one CTA per sentence, so that
// the grid is one CTA per SM and every sentence starts at once.  (A second CTA that merely left would not make
// room for the clusters still waiting: a new cluster needs both of its SMs free together.)  wide = B is the plain
// ranking for grids larger than the GPU: the clusters that wait for a place get the cheapest sentences.  False:
// nothing for this CTA.
__device__ __forceinline__ bool pick_sentence(const int64_t *ol, const int64_t *tl, int B, int L, int T, int wide,
                                              int cluster_blocks, int &crank, int &b, int &NC) {
    NC = cluster_blocks;
    b = blockIdx.x / cluster_blocks;
    if (wide < 0) return true;
    const int want = b < wide ? b : wide + 2 * (b - wide) + crank;  // the cost rank this CTA serves
    if (want >= B) return false;
    if (b >= wide) {
        NC = 1;
        crank = 0;
    }
    __shared__ int s_b;
    __shared__ int s_cost[kMaxMixedBatch];  // m n of every sentence (0: lengths out of range)
    for (int i = threadIdx.x; i < B; i += kLThreads) {
        const long long mi = ol[i], ni = tl[i];
        s_cost[i] = lengths_ok((int)mi, (int)ni, L, T) ? (int)(mi * ni) : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < B; i += kLThreads) {
        const int ci = s_cost[i];
        int before = 0;
        for (int j = 0; j < B; j++) {
            const int cj = s_cost[j];
            before += cj > ci || (cj == ci && j < i);
        }
        if (before == want) s_b = i;
    }
    __syncthreads();
    b = s_b;
    return true;
}

// lmx[t] = max over the main-chain nodes in use of match[a][t] (0 when the token has no finite emission): the
// emissions of token t are taken relative to it, which only changes the units of s_t (posteriors do not notice,
// log Z gets the sum back) but keeps the columns of both passes centred in the range of the floats however
// peaked the emissions are.  Both kernels compute it the same way, so nothing has to be handed over.
__device__ __forceinline__ void token_maxima(const float *__restrict__ mat, int m, int n, int T, int W, float *lmx) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int *enc = reinterpret_cast<int *>(lmx);  // order-preserving integer image of the floats while the maxima are taken
    for (int t = threadIdx.x; t < W; t += kLThreads) enc[t] = (int)0x80000000;
    __syncthreads();
    // lanes over tokens (coalesced rows), warps over nodes; the warps meet in shared-memory integer maxima
    for (int t0 = 0; t0 < n; t0 += 128) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = neg_inf();
        for (int a = 2 * warp + 1; a < m; a += 2 * kLWarps) {
            const float *row = mat + (size_t)a * T + t0 + lane;
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (t0 + lane + 32 * j < n) v[j] = fmaxf(v[j], __ldg(row + 32 * j));
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int t = t0 + lane + 32 * j;
            if (t < n) {
                const int i = __float_as_int(v[j]);
                atomicMax(enc + t, i >= 0 ? i : i ^ 0x7fffffff);
            }
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < W; t += kLThreads) {
        const int i = enc[t];
        const float v = __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
        lmx[t] = (t < n && v > neg_inf() && v < CUDART_INF_F) ? v : 0.f;
    }
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
template <int G, int TRIPS>
__global__ void __launch_bounds__(kLThreads, 1)
    inside_linear_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                         const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *Y,
                         float *frames, float *loss, float *shares, int *status, int Mc, int cs, int rows_cap, int B,
                         int wide) {
    extern __shared__ float4 smem4[];
    float *smem = reinterpret_cast<float *>(smem4);
    chain_begin();
    cg::cluster_group cluster = cg::this_cluster();
    int crank = (int)cluster.block_rank();  // from pick_sentence on: the rank among the CTAs of this sentence
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef PCFGNAT_TIMING
    const long long t_start = clock64();
#endif
    int b, NC;
    if (!pick_sentence(ol, tl, B, L, T, wide, (int)cluster.num_blocks(), crank, b, NC)) return;
#ifdef PCFGNAT_TIMING
    if (tid == 0 && crank == 0 && b < 256) g_linear_timing[0][b][0] = t_start;
#endif
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
    PCFGNAT_STAMP(0, 1)
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
    __shared__ int s_overflow, s_timeout;
    __shared__ float s_rho[4], s_sumlog;  // scales of the steps in flight (slot t & 3); - sum of their log2
    __shared__ float s_lmx_sum, s_lmx_last;
    if (tid == 0) {
        s_overflow = 0;
        s_lmx_sum = 0.f;
    }
    __syncthreads();

    token_maxima(mat, m, n, T, W, invs);  // borrowed until the scales are written: invs[t] = lmx[t]
    __syncthreads();
    bool big = false;
    for (int i = tid; i < my_rows * W; i += kLThreads) {
        const int r = i / W, t = i - r * W, a = 2 * (crank + NC * r) + 1;
        float v0 = 0.f, v1 = 0.f;
        if (t < n) {
            const float ma = __ldg(mat + (size_t)a * T + t);
            v0 = exp_clean(ma - invs[t]);
            if (a >= 3 && t + 1 < n)
                v1 = exp_clean((fmaxf(__ldg(mat + (size_t)(a - 1) * T + t), neg_inf()) - invs[t]) +
                               (fmaxf(__ldg(mat + (size_t)a * T + t + 1), neg_inf()) - invs[t + 1]));
        }
        big |= !(v0 < 1e30f) || !(v1 < 1e30f);
        e0[i] = v0;
        e1[i] = v1;
        ownu[i] = 0.f;
    }
    for (int r = warp; r < my_rows; r += kLWarps) {
        const int ai = crank + NC * r;
        const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L;
#pragma unroll 4
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
    __syncthreads();  // E0 and E1 are formed: the per-token maxima make room for the scales
    float lmx_part = 0.f;  // this thread's part of sum_t lmx[t]
    for (int i = tid; i < W; i += kLThreads) {
        lmx_part += i < n ? invs[i] : 0.f;
        if (i == n - 1) s_lmx_last = invs[i];
    }
    lmx_part = warp_sum(lmx_part);
    if (lane == 0 && lmx_part != 0.f) atomicAdd(&s_lmx_sum, lmx_part);
    __syncthreads();
    for (int i = tid; i < W; i += kLThreads) invs[i] = 0.f;
    if (tid == 0) bar_init(col_bar, 2);
    if (ctid == 0) {
        fr[2] = 0.f;
        fr[3] = 0.f;
    }
    __syncthreads();
    const float base = exp_clean(__ldg(mat + (size_t)(m - 1) * T + (n - 1)) - s_lmx_last);
    if (tid == 0) {
        col[((n - 1) & 3) * cs + last] = base;  // every CTA fills its own copy
        if (last % NC == crank) ownu[(size_t)(last / NC) * W + (n - 1)] = base;
    }
    PCFGNAT_STAMP(0, 2)
    if (NC > 1) cluster.sync(); else __syncthreads();
    PCFGNAT_STAMP(0, 3)
    if (s_overflow && tid == 0) fr[3] = 1.f;  // after the reset above (ordered by the barrier)

    // Step loop.  G lanes share a node (lane q of them covers the groups of four children q, q + G, ...), so a warp
    // does 32 / G nodes at once, always the same ones: their rows of P0 and P1 stay in REGISTERS for the whole loop
    // (TRIPS float4 each per lane), and a step reads only the two columns from shared memory.  Nodes beyond what
    // the warps can hold that way (long chains on few CTAs) take their rows from shared memory every step.
    // The last warp does not compute nodes unless the chain is that long: it derives the scale two steps ahead
    // from the finished column, keeps the books of the scales, and waits for the column of the step on the
    // byte-counting barrier; the block barrier then releases the others, so nobody else spins.
    constexpr int R = 32 / G;  // nodes per warp
    const int cs4 = cs >> 2;
    const int groups = (my_rows + R - 1) / R;
    const int q = lane % G, sub = lane / G;
    const float4 *P0v = reinterpret_cast<const float4 *>(P0), *P1v = reinterpret_cast<const float4 *>(P1);
    const int r_own = warp * R + sub;
    const bool live_own = r_own < my_rows;
    float4 rp0[TRIPS], rp1[TRIPS];
#pragma unroll
    for (int i = 0; i < TRIPS; i++) {
        const int c4 = q + G * i;
        rp0[i] = rp1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live_own && c4 < cs4) {
            rp0[i] = P0v[r_own * cs4 + c4];
            rp1[i] = P1v[r_own * cs4 + c4];
        }
    }
    uint32_t rcol = 0, rbar0 = 0, rbar1 = 0;  // lane q < NC: this CTA's columns and barriers as CTA q maps them
    if (NC > 1 && q < NC) {
        rcol = dsm_map_to_cta(dsm_smem_u32(col), q);
        rbar0 = dsm_map_to_cta(dsm_smem_u32(&col_bar[0]), q);
        rbar1 = dsm_map_to_cta(dsm_smem_u32(&col_bar[1]), q);
    }
    if (tid == 0) {
        s_timeout = 0;
        s_rho[(n - 2) & 3] = column_scale(base);  // the first step's scale comes from the terminal cell
        s_rho[(n - 1) & 3] = 0.f;
    }
    __syncthreads();
    float sumlog = 0.f;  // lane 0 of the last warp: - sum of log2 rho_t
#ifdef PCFGNAT_TIMING
    long long tA = 0, tB = 0, tC = 0, tD = 0, tq = clock64();
#define PCFGNAT_LAP(acc) { const long long now_ = clock64(); acc += now_ - tq; tq = now_; }
#else
#define PCFGNAT_LAP(acc)
#endif
    for (int t = n - 2; t >= 0; t--) {
        const float4 *S1v = reinterpret_cast<const float4 *>(col + ((t + 1) & 3) * cs);
        const float4 *S2v = reinterpret_cast<const float4 *>(col + ((t + 2) & 3) * cs);
        float *S0 = col + (t & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[t & 1]);
        if (NC > 1 && tid == 0) bar_expect(bar, 4 * Mb);
        if (warp < groups) {
            const float rho = s_rho[t & 3], rho_prev = s_rho[(t + 1) & 3];
            const uint32_t rS0 = rcol + 4u * ((t & 3) * cs), rbar = (t & 1) ? rbar1 : rbar0;
            PCFGNAT_LAP(tA)
            for (int g = warp; g < groups; g += kLWarps) {
                const int r = g * R + sub;
                const bool live = r < my_rows;
                const int rr = live ? r : 0;
                float acc0 = 0.f, acc1 = 0.f;
                if (g == warp) {  // this warp's resident nodes
                    float a[TRIPS], c[TRIPS];
#pragma unroll
                    for (int i = 0; i < TRIPS; i++) {
                        const int c4 = q + G * i;
                        a[i] = c[i] = 0.f;
                        if (c4 < cs4) {
                            a[i] = dot4(rp0[i], S1v[c4]);
                            c[i] = dot4(rp1[i], S2v[c4]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < TRIPS; i++) {
                        acc0 += a[i];
                        acc1 += c[i];
                    }
                } else {  // further nodes of a long chain: rows from shared memory, children ci > ai only
                    const float4 *p0 = P0v + rr * cs4, *p1 = P1v + rr * cs4;
                    for (int c4 = q + ((crank + NC * rr + 1) >> 2) / G * G; c4 < cs4; c4 += G) {
                        acc0 += dot4(p0[c4], S1v[c4]);
                        acc1 += dot4(p1[c4], S2v[c4]);
                    }
                }
                PCFGNAT_LAP(tB)
                // one scale at a time: the product of two scales can leave the range although the result does not
                float v0 = e0[rr * W + t] * (acc0 * rho);
                float v1 = e1[rr * W + t] * ((acc1 * rho_prev) * rho);
#pragma unroll
                for (int o = G / 2; o > 0; o >>= 1) {
                    v0 += __shfl_xor_sync(0xffffffffu, v0, o);
                    v1 += __shfl_xor_sync(0xffffffffu, v1, o);
                }
                const float u = v0 + v1;
                if (live) {
                    const int ai = crank + NC * r;
                    if (NC > 1) {  // lane q of the node sends to CTA q: into its column, counted on its barrier of this step
                        if (q < NC) dsm_store_async(rS0 + 4u * ai, u, rbar);
                    } else if (q == 0) {
                        S0[ai] = u;
                    }
                    if (q == 0) {
                        ownu[r * W + t] = u;
                        own0[r * W + t] = v0;
                        own1[r * W + t] = v1;
                    }
                }
            }
        }
        PCFGNAT_LAP(tC)
        if (warp == kLWarps - 1) {
            // The scale of step t - 1, from the column that has been complete since the previous barrier (t + 1).
            // Every CTA's last warp reads the same column and gets the same value.
            float mx = 0.f;
            for (int c4 = lane; c4 < cs4; c4 += 32) {
                const float4 v = S1v[c4];
                mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
            }
            mx = warp_max_nonneg(mx);
            if (lane == 0) {
                const float rho = s_rho[t & 3];
                s_rho[(t + 3) & 3] = column_scale(mx);  // slot of step t - 1
                invs[t + 1] = rho;
                sumlog -= lg2f(rho);
            }
            if (NC > 1 && !dsm_wait_column(bar, (((n - 2) - t) >> 1) & 1)) s_timeout = 1;
        }
        __syncthreads();
        PCFGNAT_LAP(tD)
    }
    if (warp == kLWarps - 1 && lane == 0) s_sumlog = sumlog;
#ifdef PCFGNAT_TIMING
    if (tid == 0 && crank == 0 && b < 256) {
        g_linear_timing[0][b][8] = tD;
        g_linear_timing[0][b][11] = tA;
        g_linear_timing[0][b][12] = tB;
        g_linear_timing[0][b][13] = tC;
    }
#endif
    PCFGNAT_STAMP(0, 4)
    const bool arrived = s_timeout == 0;
    if (!arrived && tid == 0) flag(status, PCFGNAT_STATUS_TIMEOUT);
    // no CTA leaves (its shared memory with it) while a peer may still send to it; every wait above is bounded
    if (NC > 1) cluster.sync(); else __syncthreads();
    PCFGNAT_STAMP(0, 5)

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
            const float lz = u00 > 0.f ? (lg2f(u00) + s_sumlog) * kLn2 + s_lmx_sum : neg_inf();
            fr[0] = arrived ? u00 : 0.f;
            fr[1] = lz;
            if (loss) loss[b] = lz;
        }
    }
    PCFGNAT_STAMP(0, 6)
    PCFGNAT_ACC(0, 9, NC)
}

// ---------------------------------------------------------------------------------------
// outside pass + gradients
// ---------------------------------------------------------------------------------------
// Sums of the links gradient of one node over the steps: acc0[j] = sum_tc x0[tc - 1] y_tc[c], acc1[j] = sum_tc
// x1[tc - 2] y_tc[c] for the children c = lane + 32 j of C groups, of which the first D are skipped (all at or
// below the node).  Column tc of y meets x0 of step tc - 1 and x1 of step tc - 2: one load per column and child.
// Four columns at a time, all their loads issued before the sums: a warp has few neighbours on its scheduler
// here, so it has to cover the shared-memory latency itself; the phase is bound by instruction issue.
template <int C, int D>
__device__ __forceinline__ void links_grad_sums(const float *x0r, const float *x1r, const float *ycol, int cs, int n,
                                                const bool (&in)[C], float (&acc0)[C], float (&acc1)[C]) {
    {  // column 1 has no x1 partner
        const float xa = x0r[0];
#pragma unroll
        for (int j = D; j < C; j++) acc0[j] = xa * (in[j] ? ycol[32 * j] : 0.f);
    }
    int tc = 2;
    for (; tc + 3 <= n - 1; tc += 4) {
        float xa[4], xb[4], y[4][C];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            xa[u] = x0r[tc + u - 1];
            xb[u] = x1r[tc + u - 2];
#pragma unroll
            for (int j = D; j < C; j++) y[u][j] = in[j] ? ycol[(tc + u - 1) * cs + 32 * j] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int j = D; j < C; j++) {
                acc0[j] = fmaf(xa[u], y[u][j], acc0[j]);
                acc1[j] = fmaf(xb[u], y[u][j], acc1[j]);
            }
    }
    for (; tc <= n - 1; tc++) {
        const float xa = x0r[tc - 1], xb = x1r[tc - 2];
#pragma unroll
        for (int j = D; j < C; j++) {
            const float y = in[j] ? ycol[(tc - 1) * cs + 32 * j] : 0.f;
            acc0[j] = fmaf(xa, y, acc0[j]);
            acc1[j] = fmaf(xb, y, acc1[j]);
        }
    }
}
// the instance for `dead` skipped groups (warp-uniform); dead = C: nothing to sum
template <int C, int D>
__device__ __forceinline__ void links_grad_dispatch(int dead, const float *x0r, const float *x1r, const float *ycol, int cs,
                                                    int n, const bool (&in)[C], float (&acc0)[C], float (&acc1)[C]) {
    if constexpr (D < C) {
        if (dead == D)
            links_grad_sums<C, D>(x0r, x1r, ycol, cs, n, in, acc0, acc1);
        else
            links_grad_dispatch<C, D + 1>(dead, x0r, x1r, ycol, cs, n, in, acc0, acc1);
    }
}

template <int G, int TRIPS>
__global__ void __launch_bounds__(kLThreads, 1)
    outside_linear_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                          const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T,
                          const float *__restrict__ Y, float *O, float *frames, float *mg, float *lg, int *status, int Mc,
                          int cs, int rows_cap, int B, int wide) {
    // groups of 32 children a lane sums in one pass over the steps of the links gradient: all the kernel's row
    // width allows (4 G TRIPS children), in two passes when that is more than four
    constexpr int kChunksMax = (4 * G * TRIPS + 31) / 32;
    constexpr int kGradChunk = kChunksMax <= 4 ? kChunksMax : (kChunksMax + 1) / 2;
    extern __shared__ float4 smem4[];
    float *smem = reinterpret_cast<float *>(smem4);
    chain_begin();
    cg::cluster_group cluster = cg::this_cluster();
    int crank = (int)cluster.block_rank();  // from pick_sentence on: the rank among the CTAs of this sentence
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef PCFGNAT_TIMING
    const long long t_start = clock64();
#endif
    int b, NC;
    if (!pick_sentence(ol, tl, B, L, T, wide, (int)cluster.num_blocks(), crank, b, NC)) return;
#ifdef PCFGNAT_TIMING
    if (tid == 0 && crank == 0 && b < 256) g_linear_timing[1][b][0] = t_start;
#endif
    const int W = T + 2, F = kLinearFrameHead + W;
    const int m = (int)ol[b], n = (int)tl[b];
    float *fr = frames + (size_t)b * F;
    // what the inside pass marked, or could not finish, is left to the log-space kernels (uniform over the cluster)
    const float u00 = fr[0];
    if (fr[3] != 0.f || !(u00 > 0.f) || !(fabsf(fr[1]) < CUDART_INF_F)) return;
    PCFGNAT_STAMP(1, 1)
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const int Mb = m / 2, last = (m - 2) / 2;
    const int my_rows = Mb > crank ? (Mb - crank + NC - 1) / NC : 0;  // nodes ci = crank + NC * r
    float *e0 = smem;                            // [rows_cap][W] E0, E1; after the loop x0_t and x1_t inv_{t+1}
    float *e1 = e0 + (size_t)rows_cap * W;
    float *invs = e1 + (size_t)rows_cap * W;     // [W]
    float *loop_mem = smem + linear_outside_head(rows_cap, W);  // what follows is only needed by the step loop
    float *xc0 = loop_mem;                       // [4][cs] rolling columns x0_s of the whole chain
    float *xc1 = xc0 + 4 * cs;                   // [4][cs] x1_s
    float *PT0 = xc1 + 4 * cs;                   // [rows_cap][cs] exp(links[a][0][c]) of this CTA's CHILDREN c, by parent
    float *PT1 = PT0 + (size_t)rows_cap * cs;
    float *owno = PT1 + (size_t)rows_cap * cs;   // [rows_cap][W] o_t of this CTA's nodes
    __shared__ __align__(8) uint64_t col_bar[2];
    __shared__ float red[kLWarps];
    __shared__ int s_timeout, s_range;

    token_maxima(mat, m, n, T, W, invs);  // borrowed until the scales are loaded: invs[t] = lmx[t]
    __syncthreads();
    for (int i = tid; i < my_rows * W; i += kLThreads) {
        const int r = i / W, t = i - r * W, a = 2 * (crank + NC * r) + 1;
        float v0 = 0.f, v1 = 0.f;
        if (t < n) {
            v0 = exp_clean(__ldg(mat + (size_t)a * T + t) - invs[t]);
            if (a >= 3 && t + 1 < n)
                v1 = exp_clean((fmaxf(__ldg(mat + (size_t)(a - 1) * T + t), neg_inf()) - invs[t]) +
                               (fmaxf(__ldg(mat + (size_t)a * T + t + 1), neg_inf()) - invs[t + 1]));
        }
        e0[i] = v0;
        e1[i] = v1;
        owno[i] = 0.f;
    }
    const float e_root = exp_clean(__ldg(mat + (size_t)1 * T + 0) - invs[0]);       // E0 of the root at token 0
    const float e_term = exp_clean(__ldg(mat + (size_t)(m - 1) * T + (n - 1)) - invs[n - 1]);  // u of the terminal cell
    __syncthreads();  // the maxima are used up: invs takes the scales below
    for (int r = warp; r < my_rows; r += kLWarps) {
        const int ci = crank + NC * r;
#pragma unroll 4
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
        xc0[0] = o_root * e_root;  // x0_0[root]; the root has no left child: x1 = 0
        if (crank == 0) owno[0] = o_root;
    }
    PCFGNAT_STAMP(1, 2)
    if (NC > 1) cluster.sync(); else __syncthreads();
    PCFGNAT_STAMP(1, 3)

    // Step loop, laid out as in the inside pass: G lanes per node, the node's rows of the transposed matrices in
    // registers, the last warp waits for the columns of the step.
    constexpr int R = 32 / G;
    const int cs4 = cs >> 2;
    const int groups = (my_rows + R - 1) / R;
    const int q = lane % G, sub = lane / G;
    const float4 *PT0v = reinterpret_cast<const float4 *>(PT0), *PT1v = reinterpret_cast<const float4 *>(PT1);
    const int r_own = warp * R + sub;
    const bool live_own = r_own < my_rows;
    float4 rp0[TRIPS], rp1[TRIPS];
#pragma unroll
    for (int i = 0; i < TRIPS; i++) {
        const int c4 = q + G * i;
        rp0[i] = rp1[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live_own && c4 < cs4) {
            rp0[i] = PT0v[r_own * cs4 + c4];
            rp1[i] = PT1v[r_own * cs4 + c4];
        }
    }
    uint32_t rx0 = 0, rx1 = 0, rbar0 = 0, rbar1 = 0;  // lane q < NC: this CTA's columns and barriers as CTA q maps them
    if (NC > 1 && q < NC) {
        rx0 = dsm_map_to_cta(dsm_smem_u32(xc0), q);
        rx1 = dsm_map_to_cta(dsm_smem_u32(xc1), q);
        rbar0 = dsm_map_to_cta(dsm_smem_u32(&col_bar[0]), q);
        rbar1 = dsm_map_to_cta(dsm_smem_u32(&col_bar[1]), q);
    }
    if (tid == 0) s_timeout = s_range = 0;
    __syncthreads();
    for (int s = 0; s <= n - 2; s++) {  // step s forms column s + 1
        const float4 *X0v = reinterpret_cast<const float4 *>(xc0 + (s & 3) * cs);
        const float4 *X1v = reinterpret_cast<const float4 *>(xc1 + ((s + 3) & 3) * cs);  // column s - 1 (all zero at s = 0)
        float *D0 = xc0 + ((s + 1) & 3) * cs, *D1 = xc1 + ((s + 1) & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[s & 1]);
        if (NC > 1 && tid == 0) bar_expect(bar, 8 * Mb);
        if (warp < groups) {
            const float k0 = invs[s + 1], k1 = invs[s];
            const uint32_t off = 4u * (((s + 1) & 3) * cs);
            const uint32_t rD0 = rx0 + off, rD1 = rx1 + off, rbar = (s & 1) ? rbar1 : rbar0;
            for (int g = warp; g < groups; g += kLWarps) {
                const int r = g * R + sub;
                const bool live = r < my_rows;
                const int rr = live ? r : 0;
                float acc0 = 0.f, acc1 = 0.f;
                if (g == warp) {
                    float a[TRIPS], c[TRIPS];
#pragma unroll
                    for (int i = 0; i < TRIPS; i++) {
                        const int c4 = q + G * i;
                        a[i] = c[i] = 0.f;
                        if (c4 < cs4) {
                            a[i] = dot4(rp0[i], X0v[c4]);
                            c[i] = dot4(rp1[i], X1v[c4]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < TRIPS; i++) {
                        acc0 += a[i];
                        acc1 += c[i];
                    }
                } else {  // further nodes of a long chain: rows from shared memory, parents ai < ci only
                    const float4 *p0 = PT0v + rr * cs4, *p1 = PT1v + rr * cs4;
                    const int end4 = min(cs4, (crank + NC * rr + 3) >> 2);
                    for (int c4 = q; c4 < end4; c4 += G) {
                        acc0 += dot4(p0[c4], X0v[c4]);
                        acc1 += dot4(p1[c4], X1v[c4]);
                    }
                }
                float o = fmaf(k1, acc1, acc0);
#pragma unroll
                for (int w = G / 2; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
                // o_{s+1}[c] = rho_s (acc0 + rho_{s-1} acc1).  o u is a posterior (<= 1): as long as o stays inside the
                // floats, what the inside pass flushed to zero or kept as a denormal costs less than 1e-7 of posterior
                // per cell.  An o at the edge of the range (or NaN) means the cell's inside value was below ~1e-37
                // while it still carries mass: the sentence goes to the log-space kernels.  Clamped so that the
                // products below stay finite until then.
                o *= k0;
                if (!(o < 1e37f)) {
                    o = 1e37f;
                    if (live) s_range = 1;
                }
                if (live) {
                    const int ci = crank + NC * r;
                    const float n0 = o * e0[r * W + s + 1], n1 = o * e1[r * W + s + 1];
                    if (NC > 1) {
                        if (q < NC) {
                            dsm_store_async(rD0 + 4u * ci, n0, rbar);
                            dsm_store_async(rD1 + 4u * ci, n1, rbar);
                        }
                    } else if (q == 0) {
                        D0[ci] = n0;
                        D1[ci] = n1;
                    }
                    if (q == 0) owno[r * W + s + 1] = o;
                }
            }
        }
        if (NC > 1 && warp == kLWarps - 1 && !dsm_wait_column(bar, (s >> 1) & 1)) s_timeout = 1;
        __syncthreads();
    }
    PCFGNAT_STAMP(1, 4)
    if (s_timeout && tid == 0) flag(status, PCFGNAT_STATUS_TIMEOUT);
    if ((s_range || s_timeout) && tid == 0) fr[3] = 1.f;  // marked: the log-space kernels recompute the sentence
    if (NC > 1) cluster.sync(); else __syncthreads();  // nobody exits while a peer may still send to it
    PCFGNAT_STAMP(1, 5)

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
    PCFGNAT_STAMP(1, 11)

    // ---- links_grad rows of this CTA's nodes: sums over the steps.  The y table of the whole chain is staged in
    // the shared memory the matrices and columns no longer need (the launcher sizes the kernel for it).
    const float *Yb = Y + (size_t)b * W * Mc;
    float *ys = loop_mem;  // [n - 1][cs]: y_t[c] in row t - 1, over the columns and matrices of the step loop
    float *lgb = lg + (size_t)b * L * 2 * L;
    const bool pairs_ok = !(L & 1) && !(reinterpret_cast<uintptr_t>(lg) & 7);  // rows and half rows start on 8 bytes
#pragma unroll 4
    for (int i = tid; i < (n - 1) * cs; i += kLThreads) {
        const int tc = 1 + i / cs, c = i - (tc - 1) * cs;
        ys[i] = c < Mb ? __ldg(Yb + (size_t)tc * Mc + c) : 0.f;
    }
    __syncthreads();
    PCFGNAT_STAMP(1, 12)
    for (int r = warp; r < my_rows; r += kLWarps) {
        const int ai = crank + NC * r, a = 2 * ai + 1;
        const float *x0r = e0 + r * W, *x1r = e1 + r * W;
        float *row = lgb + (size_t)a * 2 * L;
        const float *lrow = lkb + (size_t)a * 2 * L;
        for (int j0 = 0; j0 * 32 < cs; j0 += kGradChunk) {  // kGradChunk x 32 children per pass over the steps
            float acc0[kGradChunk], acc1[kGradChunk], l0[kGradChunk], l1[kGradChunk];
#pragma unroll
            for (int j = 0; j < kGradChunk; j++) {  // the links of these pairs, on their way while the sums run
                const int ci = lane + 32 * (j0 + j);
                acc0[j] = acc1[j] = 0.f;
                l0[j] = l1[j] = neg_inf();
                if (ci > ai && ci < Mb) {
                    l0[j] = __ldg(lrow + 2 * ci + 1);
                    if (ai >= 1) l1[j] = __ldg(lrow + L + 2 * ci + 1);
                }
            }
            // groups of 32 children that lie at or below the node itself have no pair with it: skipped as a whole
            const int dead = min(max((ai + 1) / 32 - j0, 0), kGradChunk);
            bool in[kGradChunk];
#pragma unroll
            for (int j = 0; j < kGradChunk; j++) in[j] = 32 * (j0 + j) + lane < cs;
            links_grad_dispatch<kGradChunk, 0>(dead, x0r, x1r, ys + 32 * j0 + lane, cs, n, in, acc0, acc1);
#pragma unroll
            for (int j = 0; j < kGradChunk; j++) {
                const int ci = lane + 32 * (j0 + j);
                const float g0 = exp_clean(l0[j]) * acc0[j];  // exp(-inf) = 0 where there is no pair
                const float g1 = exp_clean(l1[j]) * acc1[j];
                if (pairs_ok && 2 * ci + 1 < L) {  // the leaf's zero and the child's value in one 8-byte store
                    *reinterpret_cast<float2 *>(row + 2 * ci) = make_float2(0.f, g0);
                    *reinterpret_cast<float2 *>(row + L + 2 * ci) = make_float2(0.f, g1);
                } else {
                    if (2 * ci < L) {
                        row[2 * ci] = 0.f;
                        row[L + 2 * ci] = 0.f;
                    }
                    if (2 * ci + 1 < L) {
                        row[2 * ci + 1] = g0;
                        row[L + 2 * ci + 1] = g1;
                    }
                }
            }
        }
        for (int c = 2 * ((cs + 31) / 32 * 32) + lane; c < L; c += 32) {  // an odd last column beyond the chain
            row[c] = 0.f;
            row[L + c] = 0.f;
        }
    }
    PCFGNAT_STAMP(1, 13)
    // rows of links_grad that belong to no main-chain node in use
    const bool quads_ok = !(L & 1) && !(reinterpret_cast<uintptr_t>(lg) & 15);  // rows of 2 L floats start on 16 bytes
    for (int a = crank * kLWarps + warp; a < L; a += NC * kLWarps) {
        if ((a & 1) && a < m) continue;
        float *row = lgb + (size_t)a * 2 * L;
        if (quads_ok) {
            float4 *row4 = reinterpret_cast<float4 *>(row);
            for (int c = lane; c < L / 2; c += 32) row4[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int c = lane; c < 2 * L; c += 32) row[c] = 0.f;
        }
    }

    // ---- emission gradients: a warp per main-chain node a takes the rows of a and of its leaf a - 1, lanes over the
    // tokens.  The inside pass left the shares p0_t[a] in cell [a][t] and p1_t[a] in cell [a-1][t]; with o = o_t[a]
    // the leaf's gradient is p1 o, and the node's p0 o plus the leaf's of token t - 1 (a node that emitted y_t after
    // its leaf emitted y_{t-1}: the same posterior), which comes from the neighbouring lane: no cell is read
    // that another thread writes.  The terminal cell gets o u on top; everything else is zero.  `mass` = the total
    // of the sentence's emission gradients (= n when nothing was lost).
    PCFGNAT_STAMP(1, 6)
    if (NC > 1) cluster.sync(); else __syncthreads();  // the o table is complete
    PCFGNAT_STAMP(1, 7)
    float *mgb = mg + (size_t)b * L * T;
    const int cwarp = crank * kLWarps + warp, cwarps = NC * kLWarps;
    float mass = 0.f;
    for (int ai = cwarp; ai < Mb; ai += cwarps) {
        const int a = 2 * ai + 1;
        float *rown = mgb + (size_t)a * T, *rowl = rown - T;
        const float *orow = Ob + (size_t)ai * W;
        const float term = ai == last ? orow[n - 1] * e_term : 0.f;
        float carry = 0.f;  // the leaf's gradient at the token before this group of 64
        for (int t0 = 0; t0 < T; t0 += 64) {
            float p0[2], p1[2], o[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {  // both halves' loads before any use
                const int t = t0 + 32 * u + lane;
                p0[u] = p1[u] = o[u] = 0.f;
                if (t <= n - 2) {
                    o[u] = orow[t];
                    p0[u] = rown[t];
                    if (a >= 3) p1[u] = rowl[t];
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int t = t0 + 32 * u + lane;
                const float leafv = p1[u] * o[u];
                float nodev = p0[u] * o[u];
                float prev = __shfl_up_sync(0xffffffffu, leafv, 1);
                if (lane == 0) prev = carry;
                carry = __shfl_sync(0xffffffffu, leafv, 31);
                if (a >= 3 && t >= 1) nodev += prev;
                if (t == n - 1) nodev += term;
                if (t < T) {
                    rown[t] = t < n ? nodev : 0.f;
                    rowl[t] = t < n ? leafv : 0.f;
                }
                if (t < n) mass += nodev + leafv;
            }
        }
    }
    for (int node = m + cwarp; node < L; node += cwarps)  // rows beyond the graph
        for (int t = lane; t < T; t += 32) mgb[(size_t)node * T + t] = 0.f;
    mass = warp_sum(mass);
    if (lane == 0) red[warp] = mass;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.f;
        for (int i = 0; i < kLWarps; i++) tot += red[i];
        atomicAdd(fr + 2, tot);
    }
    PCFGNAT_STAMP(1, 10)
    PCFGNAT_ACC(1, 9, NC)
}

struct LinearGeometry {
    int nc, cs, rows_cap;
    int wide;                 // -1: cluster k takes sentence k; else the sentences are taken by cost (pick_sentence)
    int launch_nc, clusters;  // cluster size and number of clusters of the launch
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
        // the step loop's columns, matrices and o table, later overlaid by the y table of the gradient sums
        const size_t loop_mem = (size_t)8 * g.cs + mat + own, y_table = (size_t)W * g.cs;
        g.smem_out = ((size_t)linear_outside_head(g.rows_cap, W) + (loop_mem > y_table ? loop_mem : y_table)) * sizeof(float);
        if (g.smem_in <= (size_t)kSmemLimit - 1024 && g.smem_out <= (size_t)kSmemLimit - 1024) break;
        if (nc >= 16) {
            g.nc = 0;
            break;
        }
    }
    g.launch_nc = g.nc;
    g.clusters = B;
    if (g.nc == 1) {
        // mixed widths: clusters of two; the costliest sentences have one to themselves, the others share them in pairs
        const int wide = mixed_width_count(B, Mc);
        if (wide > 0) {
            g.wide = wide;
            g.launch_nc = 2;
            g.clusters = wide + (B - wide + 1) / 2;
        }
    }
    // more CTAs than SMs: the clusters that have to wait for a place take the cheapest sentences
    if (g.wide < 0 && g.nc >= 1 && (long long)B * g.nc > sms && B <= kMaxMixedBatch) g.wide = B;
    return g;
}

template <class Kernel, class... Args>
int launch_linear_cluster(Kernel kernel, int clusters, int nc, size_t smem, cudaStream_t st, Args... args) {
    if (ensure_dynamic_smem(kernel, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
    if (nc > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return PCFGNAT_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(clusters * nc));
    cfg.blockDim = dim3(kLThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)nc;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernels start with chain_begin()
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg) != cudaSuccess || max_clusters < 1) {
        cudaGetLastError();
        return PCFGNAT_ERR_UNSUPPORTED;
    }
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cuda_rc(cudaLaunchKernelEx(&cfg, kernel, args...));
}

template <int G, int TRIPS>
int launch_linear(const LinearGeometry &g, const float *match_all, const float *links, const int64_t *ol, const int64_t *tl,
                  int B, int L, int T, float *Y, float *O, float *frames, float *loss, float *mg, float *lg, int *status,
                  cudaStream_t st) {
    const int Mc = main_slots(L, 1);
    const int nc = g.launch_nc, clusters = g.clusters;
    int rc = launch_linear_cluster(inside_linear_kernel<G, TRIPS>, clusters, nc, g.smem_in, st, match_all, links, ol, tl, L, T,
                                   Y, frames, loss, mg, status, Mc, g.cs, g.rows_cap, B, g.wide);
    if (rc) return rc;
    return launch_linear_cluster(outside_linear_kernel<G, TRIPS>, clusters, nc, g.smem_out, st, match_all, links, ol, tl, L, T,
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
    if (Mc > 256) return PCFGNAT_ERR_UNSUPPORTED;
    const LinearGeometry g = linear_geometry(B, Mc, T + 2);
    if (g.nc == 0) return PCFGNAT_ERR_UNSUPPORTED;
    // lanes per node and float4 per lane so that a node's row of g.cs / 4 groups of four children fits the lanes' registers
    const int cs4 = g.cs / 4;
#define PCFGNAT_LINEAR_CASE(G_, TRIPS_) \
    return launch_linear<G_, TRIPS_>(g, match_all, links, ol, tl, B, L, T, Y, O, frames, loss, mg, lg, status, st)
    if (cs4 <= 8) PCFGNAT_LINEAR_CASE(8, 1);
    if (cs4 <= 16) PCFGNAT_LINEAR_CASE(8, 2);
    if (cs4 <= 24) PCFGNAT_LINEAR_CASE(8, 3);
    if (cs4 <= 32) PCFGNAT_LINEAR_CASE(8, 4);
    if (cs4 <= 48) PCFGNAT_LINEAR_CASE(16, 3);
    PCFGNAT_LINEAR_CASE(16, 4);
#undef PCFGNAT_LINEAR_CASE
}

}  // namespace pcfgnat
