// Lookahead and greedy decoding (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:419-482) on the
// device, one launch: the reference forms links_lookahead [B, L, 2, L] with torch operators, takes its arg-max per
// node, copies the indices to the host (.cpu().tolist()) and walks the tree in a Python loop per sentence.
//
// Per node a the choice is the first maximum over (k, c), k-major (index k * L + c), of
//     lookahead:  (links[a][k][c] + ob[c] * beta) + ob[left(a, k)] * beta,   left(a, 0) = 0, left(a, k) = max(a - k, 0)
//     greedy:      links[a][k][c]
// in float32 with the reference's association (models/...pcfg.py:422-428, :431).  The walk is the reference's
// in-order traversal (:435-478): from node 1 descend to the chosen left child (k == 0: node 0; else a - k) unless
// left_tree_mask forbids it, emit the node's token unless it is padding (consecutive equal tokens are NOT merged
// here, unlike the Viterbi back-trace), continue with the chosen right child; node 0 or a node at or beyond the
// sentence's length ends a branch.
//
// The reference's lookahead term for the left child is gathered from unreduced_logits.unsqueeze(1).repeat(bsz,
// prelen, 1) with an index of batch extent 1 (:425), which for bsz > 1 hands every sentence the log-probabilities of
// sentence 0; its published lookahead decoding runs with batch size 1, where that is the sentence's own.  Here every
// sentence uses its own log-probabilities.
#include <climits>

#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kLookThreads = 256;

__global__ void __launch_bounds__(kLookThreads)
    lookahead_decode_kernel(const float *__restrict__ links, const float *__restrict__ ob, const int64_t *__restrict__ tokens,
                            const int64_t *__restrict__ ol, const int64_t *__restrict__ mask, int mask_dim, float beta,
                            int lookahead, int64_t pad, int L, int cap, int64_t *out, int64_t *cnt, int *status) {
    extern __shared__ int s_idx[];  // [L] chosen (k * L + c) of every node, then [L] the walk's stack
    int *stack = s_idx + L;
    const int b = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *lkb = links + (size_t)b * L * 2 * L;
    const float *obb = ob + (size_t)b * L;
    for (int a = warp; a < L; a += kLookThreads / 32) {
        const float *row = lkb + (size_t)a * 2 * L;
        float best = neg_inf();
        int key = INT_MAX;
        for (int i = lane; i < 2 * L; i += 32) {  // a lane sees its candidates in increasing index order
            const int k = i >= L, c = i - k * L;
            float v = row[i];
            if (lookahead) {
                const int left = k == 0 ? 0 : (a - 1 < 0 ? 0 : a - 1);
                v = (v + obb[c] * beta) + obb[left] * beta;
            }
            if (v > best || (key == INT_MAX && !isnan(v))) {  // strict: the first maximum stays; -inf counts as a value
                best = v;
                key = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int ok = __shfl_xor_sync(0xffffffffu, key, o);
            if (ok != INT_MAX && (key == INT_MAX || ov > best || (ov == best && ok < key))) {
                best = ov;
                key = ok;
            }
        }
        if (lane == 0) s_idx[a] = key == INT_MAX ? 0 : key;
    }
    __syncthreads();
    if (tid != 0) return;
    const int length = (int)ol[b];
    int64_t *o = out + (size_t)b * cap;
    int sp = 0, count = 0, now = 1;
    bool bad = length < 0 || length > L;
    long guard = 0;
    while (!bad && ((now < length && now != 0) || sp > 0)) {
        while (now < length && now != 0) {
            if (now < 0 || now >= L || sp >= L || ++guard > 4L * L + 16) {
                bad = true;
                break;
            }
            stack[sp++] = now;
            const int k = s_idx[now] / L;
            const int left = k == 0 ? 0 : now - k;
            if (left < 0 || now >= mask_dim || left >= mask_dim) {
                bad = true;
                break;
            }
            if (mask[(size_t)now * mask_dim + left]) break;
            now = left;
        }
        if (bad || sp == 0) break;
        now = stack[--sp];
        const int64_t tok = tokens[(size_t)b * L + now];
        if (tok != pad) {
            if (count < cap) o[count] = tok;
            count++;
        }
        now = s_idx[now] % L;
    }
    if (bad) flag(status, PCFGNAT_STATUS_BAD_TRACE);
    const int kept = count < cap ? count : cap;
    for (int i = kept; i < cap; i++) o[i] = pad;
    cnt[b] = kept;
}

}  // namespace

int launch_lookahead_decode(const float *links, const float *ob, const int64_t *tokens, const int64_t *ol,
                            const int64_t *mask, int mask_dim, float beta, int lookahead, int64_t pad, int B, int L,
                            int cap, int64_t *out, int64_t *cnt, int *status, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    const size_t smem = (size_t)2 * L * sizeof(int);
    if (smem > 48 * 1024 && ensure_dynamic_smem(lookahead_decode_kernel, smem) != cudaSuccess) return PCFGNAT_ERR_TOO_LARGE;
    lookahead_decode_kernel<<<B, kLookThreads, smem, st>>>(links, ob, tokens, ol, mask, mask_dim, beta, lookahead, pad, L, cap,
                                                           out, cnt, status);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
