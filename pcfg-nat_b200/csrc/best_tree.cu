// Best-tree extraction for glancing training, max_left == 1.
//
// Replaces calculate_S_trace_kernel / calculate_C_kernel_trace of the reference
// (fs_plugins/custom_ops/pcfg_best_tree.cu:65-197, :240-301).  The reference marks cells
// of two trace tables and runs a block-wide barrier per `start`, although exactly one
// (node, start) cell is live per step: the derivation is a single chain.  Here one warp
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
// The 32 physical lanes here each scan a subset of one virtual lane and the warp
// reduction orders candidates by (value desc, lane rank, c, j), which is the same order.
#include "common.cuh"

namespace pcfgnat {

namespace {

struct Cand {
    float v;
    int key;  // (lane rank << 24) | (ci << 1) | j ; smaller wins among equal values
};

__device__ __forceinline__ bool better(const Cand &p, const Cand &q) {
    return p.v > q.v || (p.v == q.v && p.key < q.key);
}

constexpr int kTreeWarps = 4;

__global__ void __launch_bounds__(kTreeWarps * 32)
    best_tree_kernel(const float *__restrict__ S, const float *__restrict__ match_all,
                     const float *__restrict__ links, const int64_t *__restrict__ ol,
                     const int64_t *__restrict__ tl, int B, int L, int T, int64_t *tree, int *status, int Mc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x * kTreeWarps + warp;
    if (b >= B) return;
    const int W = T + 2;
    const int m = (int)ol[b], n = (int)tl[b];
    int64_t *tr = tree + (size_t)b * L;
    for (int i = lane; i < L; i += 32) tr[i] = -1;
    if (!lengths_ok(m, n, L, T)) {
        if (lane == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    __syncwarp();
    const float *mat = match_all + (size_t)b * L * T;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *Sb = S + (size_t)b * Mc * W;
    const int Mb = main_nodes_below(m);
    const int rank_of_lane = (0x3120 >> (4 * (lane & 3))) & 0xf;  // virtual lane 0,1,2,3 -> rank 0,2,1,3

    int ai = 0, start = 0;
    // each step consumes at least one target position, so at most n + 1 steps (start = 0 .. n)
    for (int step = 0; step <= n && start <= n; step++) {
        const int a = 2 * ai + 1;
        const int jmax = min(n - start, 2);  // j < n - start && j < max_left + 1
        Cand best{neg_inf(), 0x7fffffff};
        if (jmax >= 1) {
            const float ma0 = __ldg(mat + (size_t)a * T + start);
            const bool leaf = jmax >= 2 && a >= 3;
            const float ma1 = leaf ? __ldg(mat + (size_t)a * T + start + 1) : 0.f;
            const float ml = leaf ? __ldg(mat + (size_t)(a - 1) * T + start) : 0.f;
            for (int ci = ai + 1 + lane; ci < Mb; ci += 32) {
                const int c = 2 * ci + 1;
                float t0 = ((__ldg(lkb + ((size_t)a * 2 + 0) * L + c) + __ldg(Sb + (size_t)ci * W + start + 1)) + 0.f) + ma0;
                if (isnan(t0)) t0 = neg_inf();
                if (t0 > best.v) best = Cand{t0, (rank_of_lane << 24) | (ci << 1)};
                if (leaf) {
                    float t1 = ((__ldg(lkb + ((size_t)a * 2 + 1) * L + c) + __ldg(Sb + (size_t)ci * W + start + 2)) + ml) + ma1;
                    if (isnan(t1)) t1 = neg_inf();
                    if (t1 > best.v) best = Cand{t1, (rank_of_lane << 24) | (ci << 1) | 1};
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Cand other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.key, o)};
            if (better(other, best)) best = other;
        }
        const bool found = best.key != 0x7fffffff;  // some term was > -inf
        const int j = found ? (best.key & 1) : 0;
        if (lane == 0) {
            tr[a] = start + j;  // pcfg_best_tree.cu:182
            if (found && j == 1) tr[a - 1] = start;  // leaf visited by the local-tree trace (:293)
        }
        if (!found) break;
        ai = (best.key >> 1) & 0x7fffff;
        start = start + j + 1;
    }
}

}  // namespace

int launch_best_tree(const float *S, const float *match_all, const float *links, const int64_t *ol, const int64_t *tl,
                     int B, int L, int T, int64_t *tree, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    const int Mc = main_slots(L, 1);
    if (Mc >= (1 << 22)) return PCFGNAT_ERR_TOO_LARGE;
    best_tree_kernel<<<(B + kTreeWarps - 1) / kTreeWarps, kTreeWarps * 32, 0, st>>>(S, match_all, links, ol, tl, B, L, T,
                                                                                  tree, status, Mc);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
