// Viterbi decode tables (max semiring over output lengths, with backpointers) and the
// back-trace, max_left == 1.
//
// viterbi_kernel replaces calculate_C_kernel / calculate_S_kernel of the reference
// (fs_plugins/custom_ops/pcfg_viterbi.cu:178-241, :23-140): one CTA per sentence loops over
// the output length inside the kernel (the reference spins on a global counter between
// lengths).  With max_left == 1 the two live expansions of node a at length len are
//     t0 = ((links[a][0][c] + 0) + S[c][len-1]) + ob[a]                (j = 0, no left child)
//     t1 = ((links[a][1][c] + ob[a-1]) + S[c][len-2]) + ob[a]          (j = 1, leaf a-1)
// The reference gives node id four threads x = 0..3; thread x scans c_id = id + x + 4k in increasing
// k, t0 before t1, under strict '>', and the four are merged with shfl_down 2 then 1 under strict
// '>'.  A maximum is order-free except for ties, so here a whole warp owns the node (lane l scans
// c_id = id + l + 32 i, which is reference thread x = l & 3) and the reference's choice among equal
// values is reproduced by an explicit tie key: thread priority 0 > 2 > 1 > 3, then the smaller c,
// then j = 0 before j = 1.  Values and backpointers are bit-exact.  Tables are indexed by node id;
// R, Lt hold node ids (Lt = 0 for "no left child"), Mt holds j.
//
// viterbi_cluster_kernel spreads the nodes of a sentence over the CTAs of a thread-block cluster
// (one cluster per sentence, sized so that the batch fills the GPU): every CTA keeps the rolling
// columns of the whole chain, a warp that finishes a node stores its value into every CTA's copy
// through distributed shared memory, and the cluster meets at a hardware barrier once per length.
// viterbi_global_kernel (one CTA per sentence, links read from global memory) takes the shapes
// whose links do not fit the cluster's shared memory.
//
// backtrace_kernel replaces the host function viterbi_decoding
// (fs_plugins/custom_ops/pcfg_loss.cpp:12-73): one thread per sentence (a block each, so that the
// walks run on different SMs) does the in-order walk with an explicit stack, skipping pad tokens and
// collapsing repeats.  The three table entries of a node are fetched together when it is stacked.
#include <cooperative_groups.h>

#include <climits>
#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace pcfgnat {

namespace {

constexpr int kVitThreads = 1024;
constexpr int kVitWarps = kVitThreads / 32;

// Monotone map float -> unsigned (no NaN reaches it); -0 is mapped like +0 so that, as under the
// reference's '>', neither beats the other.
__device__ __forceinline__ unsigned ordered_bits(float v) {
    const unsigned u = __float_as_uint(v == 0.f ? 0.f : v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Warp arg-max of (best, key) pairs: the largest value, among equal values the smallest key.
// Every lane returns the winner's value and key (key INT_MAX: nothing finite was seen).
__device__ __forceinline__ void warp_argmax(float &best, int &key, int lane) {
    const unsigned ord = ordered_bits(best);
    const unsigned top = __reduce_max_sync(0xffffffffu, ord);
    const unsigned k = __reduce_min_sync(0xffffffffu, ord == top ? (unsigned)key : 0xffffffffu);
    const unsigned holders = __ballot_sync(0xffffffffu, ord == top && (unsigned)key == k);
    best = __shfl_sync(0xffffffffu, best, holders ? __ffs(holders) - 1 : lane);
    key = (int)k;
}

// One step of node `id` for the lanes of a warp: children ci = id + lane + 32 i.
//   t0 = ((links[a][0][c] + 0) + S[c][len-1]) + ob[a]      (k0[ci] holds links[a][0][c] + 0)
//   t1 = ((links[a][1][c] + ob[a-1]) + S[c][len-2]) + ob[a] (k1[ci] holds links[a][1][c] + ob[a-1];
//        -inf for the first node, which has no leaf, so that t1 never wins there)
// A NaN term never wins a '>' either, which is what the reference's NaN -> -inf cleaning achieves.
template <class K0, class K1>
__device__ __forceinline__ void viterbi_node(int id, int Mb, int lane, int prio, float oa, const float *S1,
                                             const float *S2, K0 k0, K1 k1, float &best, int &key) {
    best = neg_inf();
    key = INT_MAX;  // (prio << 24) | (c_slot << 1) | j of the current best; smaller wins ties
    for (int ci = id + lane; ci < Mb; ci += 32) {
        const int kk = (prio << 24) | (ci << 1);
        const float t0 = (k0(ci) + S1[ci]) + oa;
        if (t0 > best) {
            best = t0;
            key = kk;
        }
        const float t1 = (k1(ci) + S2[ci]) + oa;
        if (t1 > best) {
            best = t1;
            key = kk | 1;
        }
    }
    warp_argmax(best, key, lane);
}

// The same for a group of G lanes (G = 4, 8, 16 or 32, the groups of a warp side by side): lane q of the group scans
// children ci = id + q + G i, so that its reference thread (ci - id) & 3 = q & 3 is still one per lane, and the group
// settles on (largest value, smallest key) with a butterfly of shuffles.  The lanes of a group without a node
// (live = false) go through the shuffles with -inf.
template <class K0, class K1>
__device__ __forceinline__ void viterbi_node_group(bool live, int id, int Mb, int q, int G, float oa, const float *S1,
                                                   const float *S2, K0 k0, K1 k1, float &best, int &key) {
    best = neg_inf();
    key = INT_MAX;
    if (live) {
        const int x = q & 3, prio = ((x & 1) << 1) | (x >> 1);
        for (int ci = id + q; ci < Mb; ci += G) {
            const int kk = (prio << 24) | (ci << 1);
            const float t0 = (k0(ci) + S1[ci]) + oa;
            if (t0 > best) {
                best = t0;
                key = kk;
            }
            const float t1 = (k1(ci) + S2[ci]) + oa;
            if (t1 > best) {
                best = t1;
                key = kk | 1;
            }
        }
    }
    for (int o = G >> 1; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int ok = __shfl_xor_sync(0xffffffffu, key, o);
        if (ov > best || (ov == best && ok < key)) {  // -0 and +0 compare equal, as under the reference's '>'
            best = ov;
            key = ok;
        }
    }
}

__device__ __forceinline__ void viterbi_store(float best, int key, int a, int Q, int len, float *Sb, int64_t *Rb,
                                              int64_t *Lb, int64_t *Mtb) {
    if (isinf(best)) return;  // cell stays at its initial value (pcfg_viterbi.cu:113-121)
    const int bj = key & 1, bc = 2 * ((key >> 1) & 0x7FFFFF) + 1;
    const size_t o = (size_t)a * Q + len;
    Sb[o] = best;
    Lb[o] = bj ? a - 1 : 0;
    Rb[o] = bc;
    Mtb[o] = bj;
}

__global__ void __launch_bounds__(kVitThreads, 1)
    viterbi_cluster_kernel(const float *__restrict__ ob_lprob, const float *__restrict__ links,
                           const int64_t *__restrict__ ol, int L, float *S, int64_t *R, int64_t *Lt, int64_t *Mt,
                           int *status, int Mc, int cs, int rows_cap, int lk_stride, int B, int wide) {
    extern __shared__ float smem[];
    cg::cluster_group cluster = cg::this_cluster();
    int crank = (int)cluster.block_rank();  // below: the rank among the CTAs that work on this sentence
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // wide < 0: every sentence gets the whole cluster.  wide >= 0 (more sentences than half the SMs; clusters of
    // two): the sentences are taken in order of decreasing graph length, the `wide` longest get a cluster each and
    // the others share clusters, one CTA per sentence, so that the grid is one CTA per SM and every sentence
    // starts at once (a second CTA that merely left would not make room for clusters still waiting: a new cluster
    // needs both of its SMs free together).
    int NC = (int)cluster.num_blocks();
    int b = blockIdx.x / NC;
    if (wide >= 0) {
        __shared__ int s_b;
        const int want = b < wide ? b : wide + 2 * (b - wide) + crank;  // the length rank this CTA serves
        if (want >= B) return;  // the odd CTA of the last shared cluster
        if (b >= wide) {
            NC = 1;
            crank = 0;
        }
        for (int i = tid; i < B; i += kVitThreads) {
            const long long mi = ol[i], ci = (mi >= 2 && mi <= L) ? mi : 0;
            int before = 0;
            for (int j = 0; j < B; j++) {
                const long long mj = ol[j], cj = (mj >= 2 && mj <= L) ? mj : 0;
                before += cj > ci || (cj == ci && j < i);
            }
            if (before == want) s_b = i;
        }
        __syncthreads();
        b = s_b;
    }
    const int ctid = crank * kVitThreads + tid, cthreads = NC * kVitThreads;  // thread index inside the cluster
    const int Q = L / 4;
    const int m = (int)ol[b];
    const float *ob = ob_lprob + (size_t)b * L;
    const float *lkb = links + (size_t)b * L * 2 * L;
    float *Sb = S + (size_t)b * L * Q;
    int64_t *Rb = R + (size_t)b * L * Q, *Lb = Lt + (size_t)b * L * Q, *Mtb = Mt + (size_t)b * L * Q;
    for (int i = ctid; i < L * Q; i += cthreads) {
        Sb[i] = neg_inf();
        Rb[i] = 0;
        Lb[i] = 0;
        Mtb[i] = 0;
    }
    if (m < 2 || m > L) {  // uniform over the cluster: nobody reaches a cluster barrier
        if (ctid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const int Mb = main_nodes_below(m);
    const int my_rows = Mb > crank ? (Mb - crank + NC - 1) / NC : 0;  // nodes id = crank + NC * r
    float *col = smem;                // [4][cs] rolling S columns of the whole chain (replicated per CTA)
    float *lk0 = col + 4 * cs;        // [rows_cap][lk_stride] links[a][0][c] + 0 of this CTA's nodes, by child slot
    float *lk1 = lk0 + (size_t)rows_cap * lk_stride;  // links[a][1][c] + ob[a-1]
    // results of this CTA's nodes, flushed to global memory after the last length: a global store inside
    // the loop would make every cluster barrier (a release) wait for it to reach L2
    float *own_v = lk1 + (size_t)rows_cap * lk_stride;       // [rows_cap][Q]
    int *own_k = reinterpret_cast<int *>(own_v + (size_t)rows_cap * Q);  // [rows_cap][Q]

    for (int r = warp; r < my_rows; r += kVitWarps) {
        const int id = crank + NC * r;
        const float *row = lkb + (size_t)(2 * id + 1) * 2 * L;
        const float olf = id >= 1 ? __ldg(ob + 2 * id) : neg_inf();  // C[a-1][1] = ob[a-1] (pcfg_viterbi.cu:203-205)
        for (int ci = id + lane; ci < Mb; ci += 32) {
            lk0[r * lk_stride + ci] = __ldg(row + 2 * ci + 1) + 0.f;
            lk1[r * lk_stride + ci] = __ldg(row + L + 2 * ci + 1) + olf;
        }
    }
    __shared__ __align__(8) uint64_t col_bar[2];
    __shared__ int s_timeout;
    for (int i = tid; i < 4 * cs; i += kVitThreads) col[i] = neg_inf();  // lengths 0 and 1; slots >= Mb for good
    if (tid == 0) {
        s_timeout = 0;
        for (int i = 0; i < 2; i++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dsm_smem_u32(&col_bar[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // S[m-1][1] = ob[m-1] (pcfg_viterbi.cu:58); it feeds the recurrence only if m-1 is a main-chain node
    if (tid == 0 && ((m - 1) & 1)) col[1 * cs + (m - 2) / 2] = __ldg(ob + (m - 1));  // every CTA fills its own copy
    // all copies initialised before anybody stores into a neighbour's; also orders the initial fill of the
    // global tables (done by threads of any CTA of the cluster) before the cells written below
    if (NC > 1) cluster.sync(); else __syncthreads();
    if (ctid == 0) Sb[(size_t)(m - 1) * Q + 1] = __ldg(ob + (m - 1));

    // G lanes share a node, as few as still let the warps take all of this CTA's nodes in one pass (a second pass
    // costs a step more than the longer scan per lane does); lane q < NC of a group also sends the result to CTA q
    int G = 32;
    while ((32 / G) * kVitWarps < my_rows && (G >> 1) >= 4 && (G >> 1) >= NC) G >>= 1;
    const int RW = 32 / G, q = lane % G, sub = lane / G;  // RW nodes per warp
    const uint32_t rcol = NC > 1 && q < NC ? dsm_map_to_cta(dsm_smem_u32(col), q) : 0;  // this CTA's columns as CTA q maps them
    const uint32_t rbar0 = NC > 1 && q < NC ? dsm_map_to_cta(dsm_smem_u32(&col_bar[0]), q) : 0;
    const uint32_t rbar1 = NC > 1 && q < NC ? dsm_map_to_cta(dsm_smem_u32(&col_bar[1]), q) : 0;
    const int n_len = m / 4;
    for (int len = 2; len < n_len; len++) {
        const float *S1 = col + ((len - 1) & 3) * cs;
        const float *S2 = col + ((len - 2) & 3) * cs;
        float *S0 = col + (len & 3) * cs;
        const uint32_t bar = dsm_smem_u32(&col_bar[len & 1]);
        if (NC > 1 && tid == 0)  // this CTA expects the whole column of this length: one value per node of the chain
            asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(4 * Mb)
                         : "memory");
        for (int r0w = warp * RW; r0w < my_rows; r0w += kVitWarps * RW) {
            const int r = r0w + sub;
            const bool live = r < my_rows;
            const int rr = live ? r : 0, id = crank + NC * rr;
            const float *r0 = lk0 + rr * lk_stride, *r1 = lk1 + rr * lk_stride;
            float best;
            int key;
            viterbi_node_group(live, id, Mb, q, G, __ldg(ob + 2 * id + 1), S1, S2, [&](int ci) { return r0[ci]; },
                               [&](int ci) { return r1[ci]; }, best, key);
            if (live) {
                if (NC > 1) {  // into every CTA's column, counted on that CTA's barrier of this length
                    if (q < NC) dsm_store_async(rcol + 4u * ((len & 3) * cs + id), best, (len & 1) ? rbar1 : rbar0);
                } else if (q == 0) {
                    S0[id] = best;
                }
                if (q == 0) {
                    own_v[r * Q + len] = best;
                    own_k[r * Q + len] = key;
                }
            }
        }
        // one warp waits for the column on the byte-counting barrier, the block barrier releases the others: 32 warps
        // polling the same barrier get in each other's way
        if (NC > 1 && warp == kVitWarps - 1 && !dsm_wait_column(bar, ((len - 2) >> 1) & 1)) s_timeout = 1;
        __syncthreads();
    }
    if (s_timeout && tid == 0) flag(status, PCFGNAT_STATUS_TIMEOUT);
    // no CTA leaves (its shared memory with it) while a peer may still send to it: the last column has arrived
    // everywhere once every CTA has passed its last wait
    if (NC > 1) cluster.sync();
    for (int i = tid; i < my_rows * (n_len - 2); i += kVitThreads) {  // computed cells: lengths 2 .. n_len-1
        const int r = i / (n_len - 2), len = 2 + i - r * (n_len - 2);
        viterbi_store(own_v[r * Q + len], own_k[r * Q + len], 2 * (crank + NC * r) + 1, Q, len, Sb, Rb, Lb, Mtb);
    }
}

__global__ void __launch_bounds__(kVitThreads)
    viterbi_global_kernel(const float *__restrict__ ob_lprob, const float *__restrict__ links,
                          const int64_t *__restrict__ ol, int L, float *S, int64_t *R, int64_t *Lt, int64_t *Mt,
                          int *status, int Mc, int cs) {
    extern __shared__ float smem[];
    const int b = blockIdx.x;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int warp = tid >> 5, lane = tid & 31, n_warps = nthr >> 5;
    const int Q = L / 4;
    const int m = (int)ol[b];
    const float *ob = ob_lprob + (size_t)b * L;
    const float *lkb = links + (size_t)b * L * 2 * L;
    float *Sb = S + (size_t)b * L * Q;
    int64_t *Rb = R + (size_t)b * L * Q, *Lb = Lt + (size_t)b * L * Q, *Mtb = Mt + (size_t)b * L * Q;
    for (int i = tid; i < L * Q; i += nthr) {
        Sb[i] = neg_inf();
        Rb[i] = 0;
        Lb[i] = 0;
        Mtb[i] = 0;
    }
    if (m < 2 || m > L) {
        if (tid == 0) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        return;
    }
    const int Mb = main_nodes_below(m);
    float *col = smem;  // 3 rolling columns of S over main-chain slots
    for (int i = tid; i < 3 * cs; i += nthr) col[i] = neg_inf();
    __syncthreads();  // also orders the initial fill of the tables before the cells written below
    if (tid == 0) {
        const float v = __ldg(ob + (m - 1));
        Sb[(size_t)(m - 1) * Q + 1] = v;
        if ((m - 1) & 1) col[1 * cs + (m - 2) / 2] = v;
    }
    __syncthreads();
    const int x = lane & 3;
    const int prio = ((x & 1) << 1) | (x >> 1);
    for (int len = 2; len < m / 4; len++) {
        const float *S1 = col + ((len - 1) % 3) * cs;
        const float *S2 = col + ((len - 2) % 3) * cs;
        float *S0 = col + (len % 3) * cs;
        for (int id = warp; id < Mb; id += n_warps) {
            const int a = 2 * id + 1;
            const float *row = lkb + (size_t)a * 2 * L;
            const float olf = id >= 1 ? __ldg(ob + 2 * id) : neg_inf();
            float best;
            int key;
            viterbi_node(id, Mb, lane, prio, __ldg(ob + a), S1, S2, [&](int ci) { return __ldg(row + 2 * ci + 1) + 0.f; },
                         [&](int ci) { return __ldg(row + L + 2 * ci + 1) + olf; }, best, key);
            if (lane == 0) {
                S0[id] = best;
                viterbi_store(best, key, a, Q, len, Sb, Rb, Lb, Mtb);
            }
        }
        __syncthreads();
    }
}

// With S and penalty given, the output length is chosen here first, as the model does it
// (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:488-492): scores = S[b][1][len] /
// penalty[len] with NaN -> -inf, first maximum over len = 1 .. Q-1; it is written to pred_out.
__global__ void backtrace_kernel(const float *__restrict__ S, const float *__restrict__ penalty, int64_t *pred_out,
                                 const int64_t *__restrict__ pred, const int64_t *__restrict__ ol,
                                 const int64_t *__restrict__ Lt, const int64_t *__restrict__ R,
                                 const int64_t *__restrict__ Mt, const int64_t *__restrict__ tokens,
                                 const int64_t *__restrict__ mask, int mask_dim, int64_t pad, int B, int L, int Q,
                                 int cap, int64_t *out, int64_t *cnt, int *status) {
    const int i = blockIdx.x;
    if (i >= B) return;
    int chosen = 0;
    if (S) {
        const int lane = threadIdx.x;
        const float *row = S + ((size_t)i * L + 1) * Q;
        float best = neg_inf();
        int key = INT_MAX;
        for (int len = 1 + lane; len < Q; len += 32) {
            float v = row[len] / penalty[len];
            if (isnan(v)) v = neg_inf();
            if (v > best || key == INT_MAX) {  // the first entry counts even at -inf: an all -inf row picks len = 1
                best = v;
                key = len;
            }
        }
        warp_argmax(best, key, lane);
        chosen = key == INT_MAX ? 1 : key;
        if (lane == 0) pred_out[i] = chosen;
    }
    if (threadIdx.x != 0) return;
    constexpr int kStack = 32;  // the walk only stacks a node and its left spine: depth <= left_tree_layer + 2
    int stk_node[kStack], stk_len[kStack], stk_right[kStack], stk_mt[kStack];
    int sp = 0, count = 0;
    int node = 1, len = S ? chosen : (int)pred[i];
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
            const size_t at = base + (size_t)node * Q + len;
            int left = (int)Lt[at];
            const int mt = (int)Mt[at];
            stk_node[sp] = node;
            stk_len[sp] = len;
            stk_right[sp] = (int)R[at];
            stk_mt[sp] = mt;
            sp++;
            if (left == node) left = 0;
            if (left < 0 || left >= mask_dim || node >= mask_dim) {
                bad = true;
                break;
            }
            if (mask[(size_t)node * mask_dim + left]) break;
            node = left;
            len = mt;
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
        len = len - stk_mt[sp] - 1;
        node = stk_right[sp];
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
    const int Mc = main_slots(L, 1), Q = L / 4;
    const int cs = (Mc + 3) / 4 * 4;
    const int lk_stride = (Mc + 31) / 32 * 32 + 1;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // Cluster size: as many CTAs per sentence (up to 8) as still lets all sentences run at once; more when
    // a CTA's share of the links would not fit shared memory.  PCFGNAT_DP_KERNEL=rows forces the
    // single-CTA kernel (A/B runs and tests), PCFGNAT_DP_CLUSTER_SIZE a cluster size.
    int nc = 1;
    while (nc < 8 && (long long)B * nc * 2 <= sms && Mc > 8 * nc) nc *= 2;
    if (const char *v = getenv("PCFGNAT_DP_CLUSTER_SIZE")) {
        const int want = atoi(v);
        if (want == 1 || want == 2 || want == 4 || want == 8 || want == 16) nc = want;
    }
    // more sentences than half the SMs but fewer than SMs: clusters of two, which the longest sentences have to
    // themselves and the others share (see the kernel); `wide` = the SMs left over once every sentence has one
    int wide = -1;
    if (nc == 1 && B * 2 > sms && B < sms && B <= 256 && Mc > 16 && !getenv("PCFGNAT_DP_CLUSTER_SIZE")) wide = sms - B;
    if (dp_kernel_choice() == kDpRows) nc = 32;  // skips the loop below
    for (; nc <= 16; nc *= 2) {
        const int rows_cap = (Mc + nc - 1) / nc;  // also right for mixed widths: nc is 1 there, every CTA may hold a chain
        const size_t smem = ((size_t)4 * cs + (size_t)2 * rows_cap * lk_stride + (size_t)2 * rows_cap * Q) * sizeof(float);
        if (smem > (size_t)kSmemLimit - 1024) continue;
        if (ensure_dynamic_smem(viterbi_cluster_kernel, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        if (nc > 8 && cudaFuncSetAttribute(viterbi_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
                          cudaSuccess) {
            cudaGetLastError();
            break;
        }
        cudaLaunchConfig_t cfg = {};
        // mixed widths only while one CTA holds a chain; a grid larger than the GPU takes the sentences by
        // decreasing length (wide = B), so that the clusters that wait for a place get the shortest
        const bool mixed = wide >= 0 && nc == 1;
        const int order = mixed ? wide : ((long long)B * nc > sms && B <= 256 ? B : -1);
        const int launch_nc = mixed ? 2 : nc;
        cfg.gridDim = dim3((unsigned)((mixed ? wide + (B - wide + 1) / 2 : B) * launch_nc));
        cfg.blockDim = dim3(kVitThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)launch_nc;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int max_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&max_clusters, viterbi_cluster_kernel, &cfg) != cudaSuccess || max_clusters < 1) {
            cudaGetLastError();
            continue;  // this cluster size cannot be scheduled here: try the next one
        }
        return cuda_rc(cudaLaunchKernelEx(&cfg, viterbi_cluster_kernel, ob, links, ol, L, S, R, Lt, Mt, status, Mc, cs,
                                          rows_cap, lk_stride, B, order));
    }
    const size_t smem_cols = (size_t)3 * cs * sizeof(float);
    if (smem_cols > (size_t)kSmemLimit - 1024) return PCFGNAT_ERR_TOO_LARGE;
    if (ensure_dynamic_smem(viterbi_global_kernel, smem_cols) != cudaSuccess) return PCFGNAT_ERR_CUDA;
    const int warps = Mc < 4 ? 4 : (Mc > kVitWarps ? kVitWarps : Mc);
    viterbi_global_kernel<<<B, 32 * warps, smem_cols, st>>>(ob, links, ol, L, S, R, Lt, Mt, status, Mc, cs);
    return cuda_rc(cudaGetLastError());
}

int launch_backtrace(const int64_t *pred, const int64_t *ol, const int64_t *Lt, const int64_t *R, const int64_t *Mt,
                     const int64_t *tokens, const int64_t *mask, int mask_dim, int64_t pad, int B, int L, int Q,
                     int cap, int64_t *out, int64_t *cnt, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    backtrace_kernel<<<B, 32, 0, st>>>(nullptr, nullptr, nullptr, pred, ol, Lt, R, Mt, tokens, mask, mask_dim, pad, B, L, Q,
                                       cap, out, cnt, status);
    return cuda_rc(cudaGetLastError());
}

int launch_viterbi_decode(const float *S, const float *penalty, const int64_t *ol, const int64_t *Lt, const int64_t *R,
                          const int64_t *Mt, const int64_t *tokens, const int64_t *mask, int mask_dim, int64_t pad, int B,
                          int L, int Q, int cap, int64_t *pred_out, int64_t *out, int64_t *cnt, int *status,
                          cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    backtrace_kernel<<<B, 32, 0, st>>>(S, penalty, pred_out, nullptr, ol, Lt, R, Mt, tokens, mask, mask_dim, pad, B, L, Q,
                                       cap, out, cnt, status);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
