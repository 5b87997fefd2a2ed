// Inside and outside passes of the PCFG loss for sentences whose main chain fits shared memory
// (max_left == 1, up to ~160 main-chain nodes): same tables as loss_fwd.cu / loss_bwd.cu, different
// work distribution.
//
// The row-per-thread kernels give node a the (M - a) terms of its own row, so the first rows set
// the step time and most lanes idle (triangular work).  Here every dependent step is split in
// phases separated by __syncthreads, and the expensive phase is spread evenly over all 1024
// threads of the CTA by folding the triangle (row r is paired with row M-1-r: constant length):
//   inside,  step `start`:  P1 terms t0/t1 of every (a, c) pair -> smem, row max by warp-aggregated
//                              atomicMax;  P2 exp(t - max) in place;  P3 four lanes per row add the
//                              exponentials in the reference's order (c = a + x + 4k ascending, t0
//                              before t1, lanes (s0+s2)+(s1+s3)), logf(sum)+max -> S column.
//   outside, step s:        P1 weight of every (a < c) pair -> smem;  P2 four lanes per column add
//                              them in a fixed order -> G columns s+1, s+2.
// The inside table stays bit-identical to the reference kernel's (pcfg_loss.cu:149-213): the same
// float expression per term, the same max, expf/logf without fast-math, the same order of
// additions.  Per-row scalars of the next step (emissions, S entries) are loaded one step ahead
// into registers so that no global-memory latency sits between two barriers.
#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kBalThreads = 1024;
constexpr int kKeyNegInf = (int)0x807fffffu;  // f2key(-inf)

__device__ __forceinline__ int f2key(float f) {  // monotonic float -> int map (no NaN)
    int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float key2f(int k) { return __int_as_float(k >= 0 ? k : k ^ 0x7fffffff); }
__device__ __forceinline__ float clean(float t) { return isnan(t) ? neg_inf() : t; }

// Walks the folded triangle: position q -> (combined row r, offset j) with j < len.
struct FoldIter {
    int r, j, dr, dj, len;
    __device__ FoldIter(int tid, int nthr, int len_) : len(len_) {
        r = tid / len;
        j = tid - r * len;
        dr = nthr / len;
        dj = nthr - dr * len;
    }
    __device__ __forceinline__ void next() {
        j += dj;
        r += dr;
        if (j >= len) {
            j -= len;
            r++;
        }
    }
};

// ---------------------------------------------------------------------------------------
// inside pass
// ---------------------------------------------------------------------------------------
template <int NIT>
__global__ void __launch_bounds__(kBalThreads, 1)
    inside_balanced_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                           const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *S,
                           float *C, float *loss, int *status, int Mc, int Lt, int cs, int P) {
    extern __shared__ float smem[];
    const int b = blockIdx.x;
    const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const bool ok = lengths_ok(m, n, L, T);
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    float *Sb = S + (size_t)b * Mc * W;

    for (int i = tid; i < Mc * W; i += nthr) Sb[i] = neg_inf();
    if (C) {  // C[0][t][0] = 0 for t <= n; C[leaf slot][t][1] = match[leaf][t] for t < n (pcfg_loss.cu:288-297)
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
    const int last = (m - 2) / 2;
    float *col = smem;                                      // [3][cs] rolling S columns
    int *rowmax = reinterpret_cast<int *>(col + 3 * cs);    // [cs]
    float *ma = reinterpret_cast<float *>(rowmax + cs);     // [2][cs] match[a][t], buffer t & 1
    float *ml = ma + 2 * cs;                                // [cs] match[a-1][start]
    float *lk0 = ml + cs;                                   // [P] packed upper triangle incl. diagonal
    float *lk1 = lk0 + P;
    float *T0 = lk1 + P;
    float *T1 = T0 + P;

    const int fold_len = Mb + 1, fold_rows = (Mb + 1) / 2;
    auto decode = [&](const FoldIter &f, int &ai, int &ci) -> bool {
        if (f.r >= fold_rows) return false;
        if (f.j < Mb - f.r) {
            ai = f.r;
            ci = f.r + f.j;
            return true;
        }
        if (2 * f.r == Mb - 1) return false;  // middle row of an odd triangle is its own partner
        ai = Mb - 1 - f.r;
        ci = ai + (f.j - (Mb - f.r));
        return true;
    };
    auto rowstart = [&](int ai) { return ai * Mb - (ai * (ai - 1)) / 2; };

    // The pairs a thread handles are the same at every step: decode them once.  pk = a-slot | c-slot << 8 |
    // first lane << 16 | last lane << 21 of the warp's lanes that hold the same row in this trip (they are
    // contiguous), or -1 when the thread has no pair in this trip.
    int pk[NIT];
    {
        FoldIter f(tid, nthr, fold_len);
#pragma unroll
        for (int it = 0; it < NIT; it++, f.next()) {
            int ai = 0, ci = 0;
            const bool valid = decode(f, ai, ci);
            const unsigned peers = __match_any_sync(0xffffffffu, valid ? ai : -1 - lane);
            pk[it] = valid ? (ai | (ci << 8) | ((__ffs(peers) - 1) << 16) | ((31 - __clz(peers)) << 21)) : -1;
            if (valid) {
                const int p = rowstart(ai) + (ci - ai);
                const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L + (2 * ci + 1);
                lk0[p] = __ldg(row);
                lk1[p] = __ldg(row + L);
            }
        }
    }
    for (int i = tid; i < 3 * cs; i += nthr) col[i] = neg_inf();
    for (int i = tid; i < cs; i += nthr) rowmax[i] = kKeyNegInf;
    __syncthreads();

    // P3 geometry: thread (x, ai) = (tid & 3, tid >> 2); the thread with x == 0 owns the row's scalars
    const int x = tid & 3, my_row = tid >> 2;
    const bool p3_warp = tid < ((4 * Mb + 31) / 32) * 32;
    const bool row_live = my_row < Mb;
    const bool owner = row_live && x == 0;
    const int a_node = 2 * my_row + 1;
    float nxt_ma = 0.f, nxt_ml = 0.f;  // emissions of the step after the next one
    if (tid == 0) {
        float v = __ldg(mat + (size_t)(m - 1) * T + (n - 1));
        col[((n - 1) % 3) * cs + last] = v;
        Sb[(size_t)last * W + (n - 1)] = v;
    }
    if (owner && n >= 2) {
        ma[((n - 1) & 1) * cs + my_row] = __ldg(mat + (size_t)a_node * T + (n - 1));
        ma[((n - 2) & 1) * cs + my_row] = __ldg(mat + (size_t)a_node * T + (n - 2));
        ml[my_row] = a_node >= 3 ? __ldg(mat + (size_t)(a_node - 1) * T + (n - 2)) : 0.f;
        if (n >= 3) {
            nxt_ma = __ldg(mat + (size_t)a_node * T + (n - 3));
            nxt_ml = a_node >= 3 ? __ldg(mat + (size_t)(a_node - 1) * T + (n - 3)) : 0.f;
        }
    }
    __syncthreads();

    for (int start = n - 2; start >= 0; start--) {
        const float *S1 = col + ((start + 1) % 3) * cs;
        const float *S2 = col + ((start + 2) % 3) * cs;
        float *S0 = col + (start % 3) * cs;
        const float *ma0 = ma + (start & 1) * cs;
        const float *ma1 = ma + ((start + 1) & 1) * cs;
        // ---- P1: terms and row maxima -------------------------------------------------------
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            const int q = pk[it];
            int key = kKeyNegInf, ai = 0;
            unsigned mask = 1u << lane;
            if (q >= 0) {
                ai = q & 0xff;
                const int ci = (q >> 8) & 0xff;
                mask = (0xffffffffu >> (31 - ((q >> 21) & 31))) & (0xffffffffu << ((q >> 16) & 31));
                const int p = rowstart(ai) + (ci - ai);
                const float t0 = clean((lk0[p] + S1[ci]) + ma0[ai]);
                const float t1 = ai >= 1 ? clean(((lk1[p] + S2[ci]) + ml[ai]) + ma1[ai]) : neg_inf();
                T0[p] = t0;
                T1[p] = t1;
                key = f2key(fmaxf(t0, t1));
            }
            // one atomic per (warp, row): the lanes holding the same row combine first
            const int mk = __reduce_max_sync(mask, key);
            if (q >= 0 && ((q >> 16) & 31) == lane && mk > kKeyNegInf) atomicMax(&rowmax[ai], mk);
        }
        __syncthreads();
        // ---- P2: exponentials in place --------------------------------------------------------
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            const int q = pk[it];
            if (q < 0) continue;
            const int ai = q & 0xff, ci = (q >> 8) & 0xff;
            const float mx = key2f(rowmax[ai]);
            if (isinf(mx)) continue;
            const int p = rowstart(ai) + (ci - ai);
            T0[p] = expf(clean(T0[p] - mx));
            T1[p] = expf(clean(T1[p] - mx));
        }
        __syncthreads();
        // ---- P3: ordered sums, new S column, scalars of the next step ---------------------------
        if (p3_warp) {
            float sum = 0.f;
            float mx = neg_inf();
            if (row_live) {
                mx = key2f(rowmax[my_row]);
                if (!isinf(mx)) {
                    const int rs = rowstart(my_row);
                    const int cnt = Mb - my_row;  // children my_row .. Mb-1 at offsets 0 .. cnt-1
                    for (int k = x; k < cnt; k += 16) {
                        float e0[4], e1[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int kk = k + 4 * u;
                            const bool in = kk < cnt;
                            e0[u] = in ? T0[rs + kk] : 0.f;
                            e1[u] = in ? T1[rs + kk] : 0.f;
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            sum += e0[u];
                            sum += e1[u];
                        }
                    }
                }
            }
            sum += __shfl_down_sync(0xffffffffu, sum, 2, 4);
            sum += __shfl_down_sync(0xffffffffu, sum, 1, 4);
            if (owner) {
                const float res = isinf(mx) ? mx : logf(sum) + mx;
                S0[my_row] = res;
                Sb[(size_t)my_row * W + start] = res;
                rowmax[my_row] = kKeyNegInf;
                if (start >= 1) {  // scalars of step start-1 were loaded one step ago
                    ma[((start - 1) & 1) * cs + my_row] = nxt_ma;
                    ml[my_row] = nxt_ml;
                    if (start >= 2) {
                        nxt_ma = __ldg(mat + (size_t)a_node * T + (start - 2));
                        nxt_ml = a_node >= 3 ? __ldg(mat + (size_t)(a_node - 1) * T + (start - 2)) : 0.f;
                    }
                }
            }
        }
        __syncthreads();
    }
    if (loss && tid == 0) loss[b] = (n >= 2) ? col[0] : Sb[0];
}

// ---------------------------------------------------------------------------------------
// outside pass
// ---------------------------------------------------------------------------------------
// GRAD: the weights of a step are also the terms of both gradients (pcfg_loss_backward.cu:223-276, 339-382,
// 547-602), so the kernel sums them up as it goes instead of leaving that to a second kernel that would compute
// every weight again.  A pair's weights over the steps give links_grad[a][j][c] (same values, same order as
// grad_kernel: bit-identical).  The emission gradients need the weights of a parent summed over its children,
// per j: that is G[a][s] times the share of j in the parent's inside value, which the free-order inside kernel
// has left in the cells of match_all_grad where the two gradients go (share of j = 0 at [a][s], of j = 1 at
// [a-1][s]); thread 512 + row turns them into gradients step by step.  All other cells of the dense gradients
// are zero-filled first.
template <int NIT, bool GRAD>
__global__ void __launch_bounds__(kBalThreads, 1)
    outside_balanced_kernel(const float *__restrict__ grad_output, const float *__restrict__ S,
                            const float *__restrict__ match_all, const float *__restrict__ links,
                            const int64_t *__restrict__ ol, const int64_t *__restrict__ tl, int L, int T, float *G,
                            float *mg, float *lg, int *status, int Mc, int cs, int P) {
    extern __shared__ float smem[];
    const int b = blockIdx.x;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    float *Gb = G + (size_t)b * Mc * W;
    float *mgb = GRAD ? mg + (size_t)b * L * T : nullptr;
    float *lgb = GRAD ? lg + (size_t)b * L * 2 * L : nullptr;
    for (int i = tid; i < Mc * W; i += nthr) Gb[i] = 0.f;
    // GRAD: links_grad is zero-filled in units of 16 bytes where its size and address allow, else of 4
    const bool lg_vec = GRAD && (((size_t)L * 2 * L) & 3) == 0 && (reinterpret_cast<uintptr_t>(lgb) & 15) == 0;
    const int lg_units = GRAD ? (int)((size_t)L * 2 * L / (lg_vec ? 4 : 1)) : 0;
    auto zero_lg = [&](int lo, int hi, int first, int stride) {
        if (lg_vec)
            for (int i = lo + first; i < hi; i += stride) reinterpret_cast<float4 *>(lgb)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        else
            for (int i = lo + first; i < hi; i += stride) lgb[i] = 0.f;
    };
    if (GRAD) {
        // (slicing this fill over the steps, for the threads that idle in a step's second phase, was slower)
        const bool usable = lengths_ok(m, n, L, T);
        zero_lg(0, lg_units, tid, nthr);
        // emission gradients: every cell that does not hold a share (for an unusable sentence: every cell)
        const int live_rows = usable ? 2 * main_nodes_below(m) : 0;
        for (int row = tid / T, t = tid - row * T; row < L; ) {
            const bool share = row >= 1 && row < live_rows && t < n - 1;
            if (!share) mgb[(size_t)row * T + t] = 0.f;
            t += nthr;
            while (t >= T) {
                t -= T;
                row++;
            }
        }
    }
    if (!lengths_ok(m, n, L, T)) {
        if (tid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const int Mb = main_nodes_below(m);
    float *gcol = smem;           // [3][cs] rolling G columns
    float *ga = gcol + 3 * cs;    // [cs] G[a][s] where usable, else 0
    float *q0 = ga + cs;          // [cs] match[a][s] - S[a][s]
    float *q1 = q0 + cs;          // [cs] match[a-1][s] + match[a][s+1] - S[a][s]
    float *sc1 = q1 + cs;         // [cs] S[c][s+1]
    float *sc2 = sc1 + cs;        // [cs] S[c][s+2]
    float *lt0 = sc2 + cs;        // [P] lower triangle packed by column: (c, a < c) at c(c-1)/2 + a
    float *lt1 = lt0 + P;
    float *W0 = lt1 + P;
    float *W1 = W0 + P;
    float *D0 = W1 + P;           // GRAD only: the pair's weights summed over the steps
    float *D1 = D0 + P;

    // strict triangle: column c = 1..Mb-1 has c parents; fold column r+1 with column Mb-1-r
    const int tri = Mb - 1;
    const int fold_len = Mb, fold_rows = (tri + 1) / 2;
    auto decode = [&](const FoldIter &f, int &ai, int &ci) -> bool {
        if (f.r >= fold_rows) return false;
        if (f.j < f.r + 1) {
            ci = f.r + 1;
            ai = f.j;
            return true;
        }
        if (2 * f.r == tri - 1) return false;
        ci = Mb - 1 - f.r;
        ai = f.j - (f.r + 1);
        return true;
    };
    auto colstart = [&](int ci) { return (ci * (ci - 1)) / 2; };

    // GRAD: a pair's weights summed over the steps, in registers when the pairs per thread are few
    constexpr int kRegAcc = 4;
    float d0[kRegAcc] = {0.f, 0.f, 0.f, 0.f}, d1[kRegAcc] = {0.f, 0.f, 0.f, 0.f};
    int pk[NIT];  // this thread's (parent, child) pairs, the same at every step: a-slot | c-slot << 8, or -1
    {
        FoldIter f(tid, nthr, fold_len);
#pragma unroll
        for (int it = 0; it < NIT; it++, f.next()) {
            int ai = 0, ci = 0;
            const bool valid = decode(f, ai, ci);
            pk[it] = valid ? (ai | (ci << 8)) : -1;
            if (valid) {
                const int p = colstart(ci) + ai;
                const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L + (2 * ci + 1);
                lt0[p] = __ldg(row);
                lt1[p] = __ldg(row + L);
                if (GRAD) {
                    D0[p] = 0.f;
                    D1[p] = 0.f;
                }
            }
        }
    }
    for (int i = tid; i < 3 * cs; i += nthr) gcol[i] = 0.f;

    // thread (x, row) = (tid & 3, tid >> 2); x == 0 owns the row's scalars
    const int x = tid & 3, my_row = tid >> 2;
    const bool p2_warp = tid < ((4 * Mb + 31) / 32) * 32;
    const bool row_live = my_row < Mb;
    const bool owner = row_live && x == 0;
    // GRAD: thread 512 + a finishes the emission gradients of parent a
    const int h_row = tid - kBalThreads / 2;
    const bool h_live = h_row >= 0 && h_row < Mb;
    const int h_a = 2 * h_row + 1;
    float sh0 = 0.f, sh1 = 0.f;  // shares of the j = 0 and of the j = 1 terms in S[h_row][s]
    if (GRAD && h_live && n >= 2) {
        sh0 = mgb[(size_t)h_a * T];
        if (h_a >= 3) sh1 = mgb[(size_t)(h_a - 1) * T];
    }
    const int a_node = 2 * my_row + 1;
    const float *Srow = Sb + (size_t)my_row * W;
    const float *Mrow = mat + (size_t)a_node * T;
    const float *Lrow = mat + (size_t)(a_node - 1) * T;
    // owner state for step s: s_cur = S[row][s], s_n1 = S[row][s+1], s_n2 = S[row][s+2], m_n1 = match[a][s+1]
    float s_cur = 0.f, s_n1 = 0.f, s_n2 = 0.f, m_n1 = 0.f;
    float pf_s = 0.f, pf_m = 0.f, pf_l = 0.f;  // prefetched: S[row][s+3], match[a][s+2], match[a-1][s+1]
    float carry = 0.f, g_col = 0.f;            // GRAD: row h_row's j = 1 weight of the step before; G[my_row][s]
    __syncthreads();
    if (owner) {
        const float go = grad_output ? grad_output[b] : 1.f;
        s_cur = __ldg(Srow + 0);
        s_n1 = __ldg(Srow + 1);
        s_n2 = __ldg(Srow + 2);  // W = T + 2 >= 3
        const float m0 = __ldg(Mrow + 0);
        m_n1 = n >= 2 ? __ldg(Mrow + 1) : 0.f;
        const bool on = my_row == 0 && go != 0.f && !isinf(s_cur);
        ga[my_row] = on ? go : 0.f;
        q0[my_row] = on ? m0 - s_cur : 0.f;
        q1[my_row] = neg_inf();  // node 1 has no leaf; other rows carry no weight at s = 0
        sc1[my_row] = s_n1;
        sc2[my_row] = s_n2;
        if (my_row == 0) {
            gcol[0] = go;  // S_grad[0][0] = grad_output (pcfg_loss_backward.cu:78)
            Gb[0] = go;
            g_col = go;
        }
        pf_s = 3 < W ? __ldg(Srow + 3) : neg_inf();
        pf_m = 2 < n ? __ldg(Mrow + 2) : 0.f;
        pf_l = (a_node >= 3 && 1 < n) ? __ldg(Lrow + 1) : 0.f;
    }
    __syncthreads();

    for (int s = 0; s + 1 < n; s++) {
        float *g1 = gcol + ((s + 1) % 3) * cs;
        float *g2 = gcol + ((s + 2) % 3) * cs;
        // ---- P1: weights of every (parent, child) pair ----------------------------------------
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            const int q = pk[it];
            if (q < 0) continue;
            const int ai = q & 0xff, ci = (q >> 8) & 0xff;
            const int p = colstart(ci) + ai;
            const float g = ga[ai];
            float w0 = 0.f, w1 = 0.f;
            if (g != 0.f) {
                const float e0 = fast_exp((lt0[p] + sc1[ci]) + q0[ai]);
                const float e1 = fast_exp((lt1[p] + sc2[ci]) + q1[ai]);
                w0 = g * e0;
                w1 = g * e1;
            }
            W0[p] = w0;
            W1[p] = w1;
            if (GRAD) {
                if (NIT <= kRegAcc) {
                    d0[it < kRegAcc ? it : 0] += w0;
                    d1[it < kRegAcc ? it : 0] += w1;
                } else if (g != 0.f) {  // slot p is this thread's alone
                    D0[p] += w0;
                    D1[p] += w1;
                }
            }
        }
        __syncthreads();
        // ---- P2: column sums, G columns, scalars of the next step -----------------------------
        if (p2_warp) {
            float acc0 = 0.f, acc1 = 0.f;
            if (row_live) {
                const int cs0 = colstart(my_row);
                for (int k = x; k < my_row; k += 16) {
                    float u0[4], u1[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int kk = k + 4 * u;
                        const bool in = kk < my_row;
                        u0[u] = in ? W0[cs0 + kk] : 0.f;
                        u1[u] = in ? W1[cs0 + kk] : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        acc0 += u0[u];
                        acc1 += u1[u];
                    }
                }
            }
            acc0 += __shfl_down_sync(0xffffffffu, acc0, 2, 4);
            acc0 += __shfl_down_sync(0xffffffffu, acc0, 1, 4);
            acc1 += __shfl_down_sync(0xffffffffu, acc1, 2, 4);
            acc1 += __shfl_down_sync(0xffffffffu, acc1, 1, 4);
            if (owner) {
                const float v = g1[my_row] + acc0;  // column s+1 is final now
                g1[my_row] = v;
                Gb[(size_t)my_row * W + s + 1] = v;
                if (GRAD) g_col = v;
                g2[my_row] = acc1;  // first contribution to column s+2
                // this row as parent and as child at step s+1
                const float sa = s_n1;  // S[row][s+1]
                const bool on = v != 0.f && !isinf(sa);
                ga[my_row] = on ? v : 0.f;
                q0[my_row] = on ? m_n1 - sa : 0.f;
                q1[my_row] = (on && a_node >= 3 && s + 2 < n) ? (pf_l + pf_m) - sa : neg_inf();
                sc1[my_row] = s_n2;
                sc2[my_row] = pf_s;
                s_cur = s_n1;
                s_n1 = s_n2;
                s_n2 = pf_s;
                m_n1 = pf_m;
                pf_s = s + 4 < W ? __ldg(Srow + s + 4) : neg_inf();
                pf_m = s + 3 < n ? __ldg(Mrow + s + 3) : 0.f;
                pf_l = (a_node >= 3 && s + 2 < n) ? __ldg(Lrow + s + 2) : 0.f;
            }
        }
        if (GRAD && h_live) {
            // G[h_row][s] is still in its rolling column; a share next to a zero G may be anything
            const float g = gcol[(s % 3) * cs + h_row];
            const float r0 = g != 0.f ? g * sh0 : 0.f, r1 = g != 0.f ? g * sh1 : 0.f;
            // j = 0 weights are match[a][s]'s; j = 1 weights are match[a][s+1]'s and match[a-1][s]'s
            // (pcfg_loss_backward.cu:339-382)
            mgb[(size_t)h_a * T + s] = r0 + carry;
            if (h_a >= 3) mgb[(size_t)(h_a - 1) * T + s] = r1;
            carry = r1;
            if (s + 2 < n) {  // shares of the next step
                sh0 = mgb[(size_t)h_a * T + s + 1];
                if (h_a >= 3) sh1 = mgb[(size_t)(h_a - 1) * T + s + 1];
            }
        }
        __syncthreads();
    }
    if (GRAD) {
        if (h_live) mgb[(size_t)h_a * T + n - 1] = carry;
        __syncthreads();  // the terminal cell below is added to a cell written above
        if (owner) {
            // terminal cell: match_all_grad[m-1][n-1] += S_grad[slot of m-1][n-1] (pcfg_loss_backward.cu:379-382)
            // (the slot's own row holds no j = 1 weight there: the last node has no children)
            if (my_row == (m - 2) / 2) mgb[(size_t)(m - 1) * T + n - 1] = g_col;
        }
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            const int q = pk[it];
            if (q < 0) continue;
            const int ai = q & 0xff, ci = (q >> 8) & 0xff;
            const int p = colstart(ci) + ai;
            float *cell = lgb + (size_t)(2 * ai + 1) * 2 * L + (2 * ci + 1);
            cell[0] = NIT <= kRegAcc ? d0[it < kRegAcc ? it : 0] : D0[p];
            cell[L] = NIT <= kRegAcc ? d1[it < kRegAcc ? it : 0] : D1[p];
        }
    }
}

// trips of 1024 threads over a folded triangle of `rows` combined rows of `len` positions (batch maximum)
int fold_trips(int len, int rows) { return (len * rows + kBalThreads - 1) / kBalThreads; }

size_t balanced_smem_bytes(int Mc, int *cs_out, int *P_out, bool with_grad = false) {
    const int cs = (Mc + 3) / 4 * 4;
    const int P = Mc * (Mc + 1) / 2;
    *cs_out = cs;
    *P_out = P;
    return ((size_t)8 * cs + (size_t)(with_grad ? 6 : 4) * P) * sizeof(float);
}

}  // namespace

// Both return PCFGNAT_ERR_UNSUPPORTED when the shape does not fit (the caller then uses the
// row-per-thread kernels).
int launch_loss_fwd_balanced(const float *match_all, const float *links, const int64_t *ol, const int64_t *tl, int B,
                             int L, int T, float *S, float *C, float *loss, int *status, cudaStream_t st) {
    const int Mc = main_slots(L, 1), Lt = L - Mc;
    int cs, P;
    const size_t bytes = balanced_smem_bytes(Mc, &cs, &P);
    if (bytes > (size_t)kSmemLimit - 1024 || 4 * Mc > kBalThreads) return PCFGNAT_ERR_UNSUPPORTED;
    const int trips = fold_trips(Mc + 1, (Mc + 1) / 2);
#define PCFGNAT_LAUNCH_INSIDE(NIT)                                                                                     \
    do {                                                                                                               \
        if (ensure_dynamic_smem(inside_balanced_kernel<NIT>, bytes) != cudaSuccess) return PCFGNAT_ERR_CUDA;           \
        inside_balanced_kernel<NIT><<<B, kBalThreads, bytes, st>>>(match_all, links, ol, tl, L, T, S, C, loss, status, \
                                                                   Mc, Lt, cs, P);                                     \
    } while (0)
    if (trips <= 4) PCFGNAT_LAUNCH_INSIDE(4);
    else if (trips <= 9) PCFGNAT_LAUNCH_INSIDE(9);
    else if (trips <= 13) PCFGNAT_LAUNCH_INSIDE(13);
    else return PCFGNAT_ERR_UNSUPPORTED;
#undef PCFGNAT_LAUNCH_INSIDE
    return cuda_rc(cudaGetLastError());
}

bool outside_balanced_fits_grad(int L) {
    const int Mc = main_slots(L, 1);
    int cs, P;
    const size_t bytes = balanced_smem_bytes(Mc, &cs, &P, true);
    return bytes <= (size_t)kSmemLimit - 1024 && 8 * Mc <= kBalThreads && fold_trips(Mc, Mc / 2) <= 9;
}

// mg, lg both given: the kernel also writes both gradients from the emission shares the inside pass left in mg
// (only for shapes outside_balanced_fits_grad accepts).
int launch_outside_balanced(const float *grad_output, const float *S, const float *match_all, const float *links,
                            const int64_t *ol, const int64_t *tl, int B, int L, int T, float *G, float *mg, float *lg,
                            int *status, cudaStream_t st) {
    const int Mc = main_slots(L, 1);
    const bool with_grad = mg != nullptr && lg != nullptr;
    int cs, P;
    const size_t bytes = balanced_smem_bytes(Mc, &cs, &P, with_grad);
    if (bytes > (size_t)kSmemLimit - 1024 || 4 * Mc > kBalThreads) return PCFGNAT_ERR_UNSUPPORTED;
    if (with_grad && 8 * Mc > kBalThreads) return PCFGNAT_ERR_UNSUPPORTED;  // second set of (x, row) threads
    const int trips = fold_trips(Mc, Mc / 2);
#define PCFGNAT_LAUNCH_OUTSIDE(NIT, GRAD)                                                                             \
    do {                                                                                                              \
        if (ensure_dynamic_smem(outside_balanced_kernel<NIT, GRAD>, bytes) != cudaSuccess) return PCFGNAT_ERR_CUDA;   \
        outside_balanced_kernel<NIT, GRAD><<<B, kBalThreads, bytes, st>>>(grad_output, S, match_all, links, ol, tl, L, \
                                                                          T, G, mg, lg, status, Mc, cs, P);           \
    } while (0)
    if (with_grad) {
        if (trips <= 4) PCFGNAT_LAUNCH_OUTSIDE(4, true);
        else if (trips <= 9) PCFGNAT_LAUNCH_OUTSIDE(9, true);
        else return PCFGNAT_ERR_UNSUPPORTED;
    } else {
        if (trips <= 4) PCFGNAT_LAUNCH_OUTSIDE(4, false);
        else if (trips <= 9) PCFGNAT_LAUNCH_OUTSIDE(9, false);
        else if (trips <= 13) PCFGNAT_LAUNCH_OUTSIDE(13, false);
        else return PCFGNAT_ERR_UNSUPPORTED;
    }
#undef PCFGNAT_LAUNCH_OUTSIDE
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
