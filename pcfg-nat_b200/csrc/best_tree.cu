// Best-tree extraction for glancing training, max_left == 1.
//
// Replaces calculate_S_trace_kernel / calculate_C_kernel_trace of the reference
// (fs_plugins/custom_ops/pcfg_best_tree.cu:65-197, :240-301).  The reference marks cells
// of two trace tables and runs a block-wide barrier per `start`, although exactly one
// (node, start) cell is live per step: the derivation is a single chain.  Here one block
// per sentence walks that chain top-down: at (a, start) it takes the arg-max over right
// children c and the two live expansions
//     t0 = ((links[a][0][c] + S[c][start+1]) + 0) + match[a][start]            (j = 0, no left child)
//     t1 = ((links[a][1][c] + S[c][start+2]) + match[a-1][start]) + match[a][start+1]   (j = 1, leaf a-1)
// writes tree[a] = start + j (and tree[a-1] = start when the leaf is used) and moves to
// (c, start + j + 1).
//
// Tie-breaking is the reference's: it scans with 4 lanes, lane x taking
// c_id = a_id + 1 + x + 4k in increasing k, t0 before t1, strict '>' inside a lane, then
// combines lanes with shfl_down 2 and 1 under strict '>' — so among equal values lanes
// win in the order 0, 2, 1, 3 and, inside a lane, the smallest c then the smaller j.
// The threads of a block (one block per sentence) each scan a subset of one virtual lane and the
// reduction orders candidates by (value desc, lane rank, c, j), which is the same order.  All loads of a
// step are independent, so a step costs one round trip to L2, a hardware warp reduction and one block barrier.
#include <cstdlib>

#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kTreeWarps = 4;

// Monotone map float -> unsigned (no NaN reaches it); -0 is mapped like +0 so that, as under the reference's
// '>', neither beats the other.
__device__ __forceinline__ unsigned ordered_bits(float v) {
    const unsigned u = __float_as_uint(v == 0.f ? 0.f : v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kTreeWarps * 32)
    best_tree_kernel(const float *__restrict__ S, const float *__restrict__ match_all,
                     const float *__restrict__ links, const int64_t *__restrict__ ol,
                     const int64_t *__restrict__ tl, int B, int L, int T, int64_t *tree, int *status, int Mc) {
    __shared__ unsigned s_ord[2][kTreeWarps];  // per-warp winners of a step, double-buffered by step parity
    __shared__ int s_key[2][kTreeWarps];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    int64_t *tr = tree + (size_t)b * L;
    for (int i = tid; i < L; i += kTreeWarps * 32) tr[i] = -1;
    if (!lengths_ok(m, n, L, T)) {
        if (tid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    __syncthreads();
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    const int Mb = main_nodes_below(m);

    int ai = 0, start = 0;
    // each step consumes at least one target position, so at most n + 1 steps (start = 0 .. n)
    for (int step = 0; step <= n && start <= n; step++) {
        const int a = 2 * ai + 1;
        const int jmax = min(n - start, 2);  // j < n - start && j < max_left + 1
        float best = neg_inf();
        int key = 0x7fffffff;  // (lane rank << 24) | (ci << 1) | j ; smaller wins among equal values
        if (jmax >= 1) {
            const float ma0 = __ldg(mat + (size_t)a * T + start);
            const bool leaf = jmax >= 2 && a >= 3;
            const float ma1 = leaf ? __ldg(mat + (size_t)a * T + start + 1) : 0.f;
            const float ml = leaf ? __ldg(mat + (size_t)(a - 1) * T + start) : 0.f;
            for (int ci = ai + 1 + tid; ci < Mb; ci += kTreeWarps * 32) {
                const int c = 2 * ci + 1;
                // reference thread x = (ci - ai - 1) & 3 scans this child; threads rank 0, 2, 1, 3 in ties
                const int rank_of_lane = (0x3120 >> (4 * ((ci - ai - 1) & 3))) & 0xf;
                const float l0 = __ldg(lkb + ((size_t)a * 2 + 0) * L + c), s1 = __ldg(Sb + (size_t)ci * W + start + 1);
                float l1 = 0.f, s2 = 0.f;
                if (leaf) {
                    l1 = __ldg(lkb + ((size_t)a * 2 + 1) * L + c);
                    s2 = __ldg(Sb + (size_t)ci * W + start + 2);
                }
                const float t0 = ((l0 + s1) + 0.f) + ma0;  // a NaN never wins a '>': the reference's NaN -> -inf
                if (t0 > best) {
                    best = t0;
                    key = (rank_of_lane << 24) | (ci << 1);
                }
                if (leaf) {
                    const float t1 = ((l1 + s2) + ml) + ma1;
                    if (t1 > best) {
                        best = t1;
                        key = (rank_of_lane << 24) | (ci << 1) | 1;
                    }
                }
            }
        }
        // warp: largest value, among equal values the smallest key; then the same over the warps
        unsigned ord = ordered_bits(best);
        const unsigned top = __reduce_max_sync(0xffffffffu, ord);
        const unsigned kmin = __reduce_min_sync(0xffffffffu, ord == top ? (unsigned)key : 0xffffffffu);
        if (lane == 0) {
            s_ord[step & 1][warp] = top;
            s_key[step & 1][warp] = (int)kmin;
        }
        __syncthreads();
        unsigned w_ord = s_ord[step & 1][0];
        int w_key = s_key[step & 1][0];
#pragma unroll
        for (int w = 1; w < kTreeWarps; w++) {
            const unsigned o = s_ord[step & 1][w];
            const int k = s_key[step & 1][w];
            if (o > w_ord || (o == w_ord && (unsigned)k < (unsigned)w_key)) {
                w_ord = o;
                w_key = k;
            }
        }
        const bool found = w_key != 0x7fffffff;  // some term was > -inf
        const int j = found ? (w_key & 1) : 0;
        if (tid == 0) {
            tr[a] = start + j;  // pcfg_best_tree.cu:182
            if (found && j == 1) tr[a - 1] = start;  // leaf visited by the local-tree trace (:293)
        }
        if (!found) break;
        ai = (w_key >> 1) & 0x7fffff;
        start = start + j + 1;
    }
}

// The same walk with everything it reads staged in shared memory first: the triangle links[a][k][c], c > a, of the
// main-chain nodes (packed row after row), the inside table and the emissions.  A step of the walk above is one
// round trip to L2 (about 1 300 cycles with the reduction and the barrier) and there are up to n + 1 of them in a
// row; from shared memory a step is about 250 cycles, and the staging is one coalesced pass with every load of
// the block in flight.  Same arithmetic, same keys: the result is bit for bit the same.
constexpr int kStagedTreeWarps = 32;

__host__ __device__ inline size_t tri_rows_before(int ai, int Mb) {  // pairs (a, c > a) of the rows before ai
    return (size_t)ai * (Mb - 1) - (size_t)ai * (ai - 1) / 2;
}

__global__ void __launch_bounds__(kStagedTreeWarps * 32)
    best_tree_staged_kernel(const float *__restrict__ S, const float *__restrict__ match_all,
                            const float *__restrict__ links, const int64_t *__restrict__ ol,
                            const int64_t *__restrict__ tl, int B, int L, int T, int64_t *tree, int *status, int Mc) {
    extern __shared__ float tree_smem[];
    __shared__ unsigned s_ord[2][kStagedTreeWarps];
    __shared__ int s_key[2][kStagedTreeWarps];
    constexpr int kThreads = kStagedTreeWarps * 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    int64_t *tr = tree + (size_t)b * L;
    for (int i = tid; i < L; i += kThreads) tr[i] = -1;
    if (!lengths_ok(m, n, L, T)) {
        if (tid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    const int Mb = main_nodes_below(m);
    const size_t tri = tri_rows_before(Mb > 0 ? Mb - 1 : 0, Mb);  // pairs in all
    float *tri0 = tree_smem, *tri1 = tri0 + tri;  // [pairs] links[a][0][c], links[a][1][c]
    float *Ss = tri1 + tri;                       // [Mb][W]
    float *ms = Ss + (size_t)Mb * W;              // [m][T]
    // eight elements per thread and trip, all their loads issued before the first store: the staging is a handful
    // of round trips to L2
    constexpr int kBatch = 8;
    for (int i0 = tid; i0 < (Mb - 1) * Mb; i0 += kBatch * kThreads) {  // (ai, ci) over the square; pairs ci > ai only
        float v0[kBatch], v1[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int i = i0 + u * kThreads, ai = i / Mb, ci = i - ai * Mb;
            v0[u] = v1[u] = 0.f;
            if (i < (Mb - 1) * Mb && ci > ai) {
                const float *row = lkb + (size_t)(2 * ai + 1) * 2 * L + 2 * ci + 1;
                v0[u] = __ldg(row);
                v1[u] = __ldg(row + L);
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int i = i0 + u * kThreads, ai = i / Mb, ci = i - ai * Mb;
            if (i < (Mb - 1) * Mb && ci > ai) {
                const size_t at = tri_rows_before(ai, Mb) + (ci - ai - 1);
                tri0[at] = v0[u];
                tri1[at] = v1[u];
            }
        }
    }
    auto stage = [&](float *dst, const float *src, int count) {
        for (int i0 = tid; i0 < count; i0 += kBatch * kThreads) {
            float v[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; u++) v[u] = i0 + u * kThreads < count ? __ldg(src + i0 + u * kThreads) : 0.f;
#pragma unroll
            for (int u = 0; u < kBatch; u++)
                if (i0 + u * kThreads < count) dst[i0 + u * kThreads] = v[u];
        }
    };
    stage(Ss, Sb, Mb * W);
    stage(ms, mat, m * T);
    __syncthreads();
    // the walk needs a thread per right child at most: the other warps are done, the walkers meet on a barrier of
    // their own
    const int walkers = max(1, (Mb - 1 + 31) / 32);
    if (warp >= walkers) return;
    const int walk_threads = walkers * 32;

    int ai = 0, start = 0;
    for (int step = 0; step <= n && start <= n; step++) {
        const int a = 2 * ai + 1;
        const int jmax = min(n - start, 2);
        float best = neg_inf();
        int key = 0x7fffffff;
        if (jmax >= 1) {
            const float ma0 = ms[(size_t)a * T + start];
            const bool leaf = jmax >= 2 && a >= 3;
            const float ma1 = leaf ? ms[(size_t)a * T + start + 1] : 0.f;
            const float ml = leaf ? ms[(size_t)(a - 1) * T + start] : 0.f;
            const size_t off = tri_rows_before(ai, Mb);
            for (int ci = ai + 1 + tid; ci < Mb; ci += walk_threads) {
                const int rank_of_lane = (0x3120 >> (4 * ((ci - ai - 1) & 3))) & 0xf;
                const float l0 = tri0[off + (ci - ai - 1)], s1 = Ss[(size_t)ci * W + start + 1];
                const float t0 = ((l0 + s1) + 0.f) + ma0;
                if (t0 > best) {
                    best = t0;
                    key = (rank_of_lane << 24) | (ci << 1);
                }
                if (leaf) {
                    const float l1 = tri1[off + (ci - ai - 1)], s2 = Ss[(size_t)ci * W + start + 2];
                    const float t1 = ((l1 + s2) + ml) + ma1;
                    if (t1 > best) {
                        best = t1;
                        key = (rank_of_lane << 24) | (ci << 1) | 1;
                    }
                }
            }
        }
        unsigned ord = ordered_bits(best);
        const unsigned top = __reduce_max_sync(0xffffffffu, ord);
        const unsigned kmin = __reduce_min_sync(0xffffffffu, ord == top ? (unsigned)key : 0xffffffffu);
        if (lane == 0) {
            s_ord[step & 1][warp] = top;
            s_key[step & 1][warp] = (int)kmin;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(walk_threads) : "memory");
        // every walking warp reduces the winners of all of them (one per lane) the same way
        static_assert(kStagedTreeWarps <= 32, "one lane per warp's winner");
        const unsigned my_ord = lane < walkers ? s_ord[step & 1][lane] : 0u;
        const int my_key = lane < walkers ? s_key[step & 1][lane] : 0x7fffffff;
        const unsigned w_ord = __reduce_max_sync(0xffffffffu, my_ord);
        const int w_key = (int)__reduce_min_sync(0xffffffffu, my_ord == w_ord ? (unsigned)my_key : 0xffffffffu);
        const bool found = w_key != 0x7fffffff;
        const int j = found ? (w_key & 1) : 0;
        if (tid == 0) {
            tr[a] = start + j;
            if (found && j == 1) tr[a - 1] = start;
        }
        if (!found) break;
        ai = (w_key >> 1) & 0x7fffff;
        start = start + j + 1;
    }
}

}  // namespace

int launch_best_tree(const float *S, const float *match_all, const float *links, const int64_t *ol, const int64_t *tl,
                     int B, int L, int T, int64_t *tree, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    const int Mc = main_slots(L, 1);
    if (Mc >= (1 << 22)) return PCFGNAT_ERR_TOO_LARGE;
    // everything the walk reads in shared memory, where the largest sentence the shapes allow fits
    const size_t staged = (2 * tri_rows_before(Mc > 0 ? Mc - 1 : 0, Mc) + (size_t)Mc * (T + 2) + (size_t)L * T) * sizeof(float);
    const char *env = getenv("PCFGNAT_TREE_STAGED");  // "0": the walk over global memory
    if (staged <= (size_t)kSmemLimit - 1024 && !(env && env[0] == '0')) {
        if (ensure_dynamic_smem(best_tree_staged_kernel, staged) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        best_tree_staged_kernel<<<B, kStagedTreeWarps * 32, staged, st>>>(S, match_all, links, ol, tl, B, L, T, tree, status, Mc);
        return cuda_rc(cudaGetLastError());
    }
    best_tree_kernel<<<B, kTreeWarps * 32, 0, st>>>(S, match_all, links, ol, tl, B, L, T, tree, status, Mc);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
