// Transition log-probabilities ("links") of the PCFG-NAT decoder from the projected link features,
// max_left == 1: extract_links() of the reference model after its three link projections
// (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:163-199) in three launches, and its
// gradient with respect to the link features and the gate logits in two more.
//
// The reference forms, per sentence b, node a, head h (chunk of the decoder dimension):
//     ab[a][k][h]    = q[a][h] . kl[left(a,k)][h] / sqrt(D)     left(a,0) = 0 (no left child), left(a,1) = a - 1
//     bc[a][k][c][h] = kl[left(a,k)][h] . kr[c][h] / sqrt(D)
//     ac[a][c][h]    = q[a][h] . kr[c][h] / sqrt(D)
// masks ab where left(a,k) is padding or outside a's left subtree and ac where c is padding, outside a's right
// subtree or not a main-chain node, normalises (ab + bc) + ac jointly over (k, c) per head (log-softmax), mixes
// the heads with log-softmax(gate logits) by log-sum-exp, and sets the whole row to -inf when a has no admissible
// left or no admissible right child.  That is ~30 element-wise / gather / roll / softmax launches over
// [B, L, 2, L, heads] tensors.  Only main-chain nodes have right children and only main-chain nodes are right
// children, so here
//   links_gather_kernel        packs the features of the M main-chain nodes (and of their left options) as the
//                              float32 operands of the GEMMs:  qm, krm [B][H][M][D], klm [B][H][M+1][D];
//   links_scores_kernel        ac [B][H][M][M] = qm krm^T,  bc [B][H][M+1][M] = klm krm^T, unscaled (small batched
//                              float32 products, one block per sentence, head and 64 x 64 tile);
//   links_from_scores_kernel   one block per (sentence, node) does the rest.
// Backward (training): links_grad [B][L][2][L] ->
//   links_scores_grad_kernel   one block per (sentence, node): the row's forward quantities once more, then the
//                              gradient of every logit (k, c, head) as X0, X1 [B][H][M][M] (left option 0 / 1,
//                              scaled), their row sums (gradient of ab) and the gradient of the gate logits;
//   links_features_grad_kernel one block per (sentence, head): the five small products that turn X0, X1 into the
//                              gradients of q, kl, kr at the main-chain nodes and their left options (operands in
//                              shared memory, 4 x 4 outputs per thread; a plain version for odd shapes).
#include <cuda_fp16.h>

#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kLinkThreads = 128;
constexpr int kMaxHeads = 32;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float feat(const void *p, bool half, size_t i) {
    return half ? __half2float(static_cast<const __half *>(p)[i]) : static_cast<const float *>(p)[i];
}

// q, kl, kr [B][L][H][D] (f16 or f32); nodes [M] = ids of the main-chain nodes, ascending.
//   qm = q[nodes], krm = kr[nodes]; klm row 0 = kl[0] (no left child), row 1 + s = kl[nodes[s] - 1].
__global__ void links_gather_kernel(const void *__restrict__ q, const void *__restrict__ kl, const void *__restrict__ kr,
                                    int is_half, const int *__restrict__ nodes, int M, int L, int H, int D, float *qm,
                                    float *klm, float *krm) {
    const int b = blockIdx.y, r = blockIdx.x;  // r = 0 .. M: row of klm; rows 1 .. M are also rows r - 1 of qm, krm
    const int HD = H * D;
    const int left = r == 0 ? 0 : max(nodes[r - 1] - 1, 0);
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
        const int h = i / D, d = i - h * D;
        klm[(((size_t)b * H + h) * (M + 1) + r) * D + d] = feat(kl, is_half, ((size_t)b * L + left) * HD + i);
        if (r > 0) {
            const size_t src = ((size_t)b * L + nodes[r - 1]) * HD + i;
            const size_t dst = (((size_t)b * H + h) * M + (r - 1)) * D + d;
            qm[dst] = feat(q, is_half, src);
            krm[dst] = feat(kr, is_half, src);
        }
    }
}

// HT: number of heads known at compile time (the terms of a cell stay in registers between the two reductions
// over the heads), or 0 for any number up to kMaxHeads.
// gates [B][L][H] f32 (logits); nonpad [B][L] u8; left_mask, right_mask [L][L] u8 (1 = not allowed); main_chain [L]
// u8; slot_of [L] = index of a node among the main-chain nodes or -1; nodes [M] its inverse.
template <int HT>
__global__ void __launch_bounds__(kLinkThreads)
    links_from_scores_kernel(const float *__restrict__ ac, const float *__restrict__ bc, const float *__restrict__ qm,
                             const float *__restrict__ klm, const float *__restrict__ gates,
                             const uint8_t *__restrict__ nonpad, const uint8_t *__restrict__ left_mask,
                             const uint8_t *__restrict__ right_mask, const uint8_t *__restrict__ main_chain,
                             const int *__restrict__ slot_of, const int *__restrict__ nodes, int M, int L, int H, int D,
                             float scale, float *__restrict__ links) {
    extern __shared__ uint8_t s_right_ok[];  // [M] right child nodes[s] admissible for this node
    __shared__ float s_ab[2][kMaxHeads], s_lse[kMaxHeads], s_lg[kMaxHeads];
    const int a = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = kLinkThreads / 32;
    const uint8_t *np = nonpad + (size_t)b * L;
    float *out = links + ((size_t)b * L + a) * 2 * L;
    for (int i = tid; i < 2 * L; i += kLinkThreads) out[i] = neg_inf();  // admissible cells are overwritten below
    const int sa = slot_of[a];
    if (sa < 0) return;  // not on the main chain: no right child at max_left == 1
    // admissible children of a at all?  (the reference's link_left_nouse_mask / link_right_nouse_mask)
    int any_left = 0, any_right = 0;
    for (int j = tid; j < L; j += kLinkThreads) any_left |= np[j] && !left_mask[(size_t)a * L + j];
    for (int s = tid; s < M; s += kLinkThreads) {
        const int c = nodes[s];
        const bool r_ok = np[c] && !right_mask[(size_t)a * L + c] && main_chain[c];
        s_right_ok[s] = r_ok;
        any_right |= r_ok;
    }
    any_left = __syncthreads_or(any_left);
    any_right = __syncthreads_or(any_right);  // also: s_right_ok is written, and so is the -inf fill of this row
    if (!any_left || !any_right) return;
    const int left1 = a >= 1 ? a - 1 : 0;  // the reference's _max_left_index[a][1]
    const bool ok_left0 = np[0] && !left_mask[(size_t)a * L + 0];
    const bool ok_left1 = np[left1] && !left_mask[(size_t)a * L + left1];
    // ab[k][h]: one warp per head at a time, lanes over the chunk dimension
    for (int h = warp; h < H; h += n_warps) {
        const float *qa = qm + (((size_t)b * H + h) * M + sa) * D;
        const float *k0 = klm + (((size_t)b * H + h) * (M + 1) + 0) * D;
        const float *k1 = klm + (((size_t)b * H + h) * (M + 1) + 1 + sa) * D;
        float d0 = 0.f, d1 = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float x = qa[d];
            d0 = fmaf(x, k0[d], d0);
            d1 = fmaf(x, k1[d], d1);
        }
        d0 = warp_sum_f(d0);
        d1 = warp_sum_f(d1);
        if (lane == 0) {
            s_ab[0][h] = ok_left0 ? d0 * scale : neg_inf();
            s_ab[1][h] = ok_left1 ? d1 * scale : neg_inf();
        }
    }
    if (warp == n_warps - 1) {  // log-softmax of the gate logits over the heads
        const float gt = lane < H ? gates[((size_t)b * L + a) * H + lane] : neg_inf();
        const float mx = warp_max_f(gt);
        const float sum = warp_sum_f(lane < H ? expf(gt - mx) : 0.f);
        if (lane < H) s_lg[lane] = gt - (mx + logf(sum));
    }
    __syncthreads();
    // logit of (left option k, right child slot s) for head h: (ab + bc) + ac
    auto logit = [&](int h, int k, int s) {
        const float vac = ac[(((size_t)b * H + h) * M + sa) * M + s] * scale;
        const float vbc = bc[(((size_t)b * H + h) * (M + 1) + (k ? 1 + sa : 0)) * M + s] * scale;
        return (s_ab[k][h] + vbc) + vac;
    };
    // pass 1: log-sum-exp over (k, c) per head
    for (int h = warp; h < H; h += n_warps) {
        float mx = neg_inf(), sum = 0.f;
        for (int s = lane; s < M; s += 32) {
            if (!s_right_ok[s]) continue;
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float v = logit(h, k, s);
                if (v > mx) {
                    sum = sum * expf(mx - v) + 1.f;  // exp(-inf - v) = 0 on the first finite value
                    mx = v;
                } else if (v > neg_inf()) {
                    sum += expf(v - mx);
                }
            }
        }
        const float top = warp_max_f(mx);
        sum = isinf(mx) ? 0.f : sum * expf(mx - top);
        sum = warp_sum_f(sum);
        if (lane == 0) s_lse[h] = isinf(top) ? top : top + logf(sum);
    }
    __syncthreads();
    // pass 2: mix the heads
    for (int i = tid; i < 2 * M; i += kLinkThreads) {
        const int k = i / M, s = i - k * M;
        if (!s_right_ok[s]) continue;
        float res = neg_inf();
        if (HT > 0) {
            float term[HT > 0 ? HT : 1];
            float mx = neg_inf();
#pragma unroll
            for (int h = 0; h < HT; h++) {
                term[h] = (logit(h, k, s) - s_lse[h]) + s_lg[h];
                mx = fmaxf(mx, term[h]);  // fmaxf drops NaN
            }
            if (!isinf(mx)) {
                float sum = 0.f;
#pragma unroll
                for (int h = 0; h < HT; h++)
                    if (term[h] > neg_inf()) sum += expf(term[h] - mx);
                res = mx + logf(sum);
            }
        } else {
            float mx = neg_inf();
            for (int h = 0; h < H; h++) mx = fmaxf(mx, (logit(h, k, s) - s_lse[h]) + s_lg[h]);
            if (!isinf(mx)) {
                float sum = 0.f;
                for (int h = 0; h < H; h++) {
                    const float t = (logit(h, k, s) - s_lse[h]) + s_lg[h];
                    if (t > neg_inf()) sum += expf(t - mx);
                }
                res = mx + logf(sum);
            }
        }
        out[(size_t)k * L + nodes[s]] = res;
    }
}

// C[b][h] = A[b][h] krm[b][h]^T for the rows of A = qm (M rows -> ac) and A = klm (M + 1 rows -> bc): float32, 64 x 64
// output tiles, the D axis walked in chunks of 16 through shared memory.
constexpr int kScoreTile = 64, kScoreK = 16;
__global__ void __launch_bounds__(256)
    links_scores_kernel(const float *__restrict__ qm, const float *__restrict__ klm, const float *__restrict__ krm, int M,
                        int D, float *__restrict__ ac, float *__restrict__ bc) {
    __shared__ float sa[kScoreK][kScoreTile + 1], sb[kScoreK][kScoreTile + 1];
    const int bh = blockIdx.z;
    const int tiles_m = (M + kScoreTile - 1) / kScoreTile, tiles_r = (2 * M + 1 + kScoreTile - 1) / kScoreTile;
    const int tr = blockIdx.y, tc = blockIdx.x;  // row tile over the 2 M + 1 stacked rows (qm then klm), column tile over M
    if (tr >= tiles_r || tc >= tiles_m) return;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4] = {};
    const float *qb = qm + (size_t)bh * M * D, *klb = klm + (size_t)bh * (M + 1) * D, *krb = krm + (size_t)bh * M * D;
    for (int k0 = 0; k0 < D; k0 += kScoreK) {
        for (int i = threadIdx.x; i < kScoreTile * kScoreK; i += 256) {
            const int r = i / kScoreK, k = i - r * kScoreK;
            const int row = tr * kScoreTile + r, col = tc * kScoreTile + r;
            float va = 0.f, vb = 0.f;
            if (k0 + k < D) {
                if (row < M) va = qb[(size_t)row * D + k0 + k];
                else if (row < 2 * M + 1) va = klb[(size_t)(row - M) * D + k0 + k];
                if (col < M) vb = krb[(size_t)col * D + k0 + k];
            }
            sa[k][r] = va;
            sb[k][r] = vb;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kScoreK; k++) {
            float a4[4], b4[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a4[i] = sa[k][ty * 4 + i];
                b4[i] = sb[k][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = tr * kScoreTile + ty * 4 + i;
        if (row >= 2 * M + 1) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int col = tc * kScoreTile + tx * 4 + j;
            if (col >= M) continue;
            if (row < M) ac[((size_t)bh * M + row) * M + col] = acc[i][j];
            else bc[((size_t)bh * (M + 1) + (row - M)) * M + col] = acc[i][j];
        }
    }
}

// Gradient of the logits of one (sentence, node) row.  With G = links_grad[a][k][c], res = links[a][k][c],
//   term[h] = logit[h] - lse[h] + lg[h],  w[h] = exp(term[h] - res)             (share of head h in the mixture)
//   d lp[k][c][h] = G w[h],   Gs[h] = sum_{k,c} d lp[k][c][h]  (= d lg[h]),
//   d logit[k][c][h] = d lp[k][c][h] - exp(logit[k][c][h] - lse[h]) Gs[h]
// written scaled by 1/sqrt(D) (the logits are scaled dot products) as X0 (k = 0) and X1 (k = 1) [B][H][M][M] at row
// slot(a); dab [B][H][M][2] = their row sums; dgates[a][h] = Gs[h] - softmax(gates)[h] sum_h' Gs[h'].  Rows of nodes
// that are not on the main chain, or have no admissible child, are zero (X rows) / zero (dgates).
__global__ void __launch_bounds__(kLinkThreads)
    links_scores_grad_kernel(const float *__restrict__ links_grad, const float *__restrict__ ac, const float *__restrict__ bc,
                             const float *__restrict__ qm, const float *__restrict__ klm, const float *__restrict__ gates,
                             const uint8_t *__restrict__ nonpad, const uint8_t *__restrict__ left_mask,
                             const uint8_t *__restrict__ right_mask, const uint8_t *__restrict__ main_chain,
                             const int *__restrict__ slot_of, const int *__restrict__ nodes, int M, int L, int H, int D,
                             float scale, float *__restrict__ X0, float *__restrict__ X1, float *__restrict__ dab,
                             float *__restrict__ dgates) {
    extern __shared__ uint8_t s_right_ok[];
    __shared__ float s_ab[2][kMaxHeads], s_lse[kMaxHeads], s_lg[kMaxHeads], s_gs[kMaxHeads], s_red[kMaxHeads][4];
    const int a = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = kLinkThreads / 32;
    const uint8_t *np = nonpad + (size_t)b * L;
    float *dg = dgates + ((size_t)b * L + a) * H;
    for (int h = tid; h < H; h += kLinkThreads) dg[h] = 0.f;
    const int sa = slot_of[a];
    if (sa < 0) return;
    // this node's rows of X0, X1 and dab start at zero
    for (int i = tid; i < H * M; i += kLinkThreads) {
        const int h = i / M, s = i - h * M;
        X0[(((size_t)b * H + h) * M + sa) * M + s] = 0.f;
        X1[(((size_t)b * H + h) * M + sa) * M + s] = 0.f;
    }
    for (int i = tid; i < 2 * H; i += kLinkThreads) dab[(((size_t)b * H + i / 2) * M + sa) * 2 + (i & 1)] = 0.f;
    int any_left = 0, any_right = 0;
    for (int j = tid; j < L; j += kLinkThreads) any_left |= np[j] && !left_mask[(size_t)a * L + j];
    for (int s = tid; s < M; s += kLinkThreads) {
        const int c = nodes[s];
        const bool r_ok = np[c] && !right_mask[(size_t)a * L + c] && main_chain[c];
        s_right_ok[s] = r_ok;
        any_right |= r_ok;
    }
    any_left = __syncthreads_or(any_left);
    any_right = __syncthreads_or(any_right);
    if (!any_left || !any_right) return;
    const int left1 = a >= 1 ? a - 1 : 0;
    const bool ok_left0 = np[0] && !left_mask[(size_t)a * L + 0];
    const bool ok_left1 = np[left1] && !left_mask[(size_t)a * L + left1];
    for (int h = warp; h < H; h += n_warps) {
        const float *qa = qm + (((size_t)b * H + h) * M + sa) * D;
        const float *k0 = klm + (((size_t)b * H + h) * (M + 1) + 0) * D;
        const float *k1 = klm + (((size_t)b * H + h) * (M + 1) + 1 + sa) * D;
        float d0 = 0.f, d1 = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float x = qa[d];
            d0 = fmaf(x, k0[d], d0);
            d1 = fmaf(x, k1[d], d1);
        }
        d0 = warp_sum_f(d0);
        d1 = warp_sum_f(d1);
        if (lane == 0) {
            s_ab[0][h] = ok_left0 ? d0 * scale : neg_inf();
            s_ab[1][h] = ok_left1 ? d1 * scale : neg_inf();
        }
    }
    float gate_p = 0.f;  // softmax(gates)[lane] in the last warp
    if (warp == n_warps - 1) {
        const float gt = lane < H ? gates[((size_t)b * L + a) * H + lane] : neg_inf();
        const float mx = warp_max_f(gt);
        const float sum = warp_sum_f(lane < H ? expf(gt - mx) : 0.f);
        if (lane < H) {
            s_lg[lane] = gt - (mx + logf(sum));
            gate_p = expf(s_lg[lane]);
        }
    }
    __syncthreads();
    auto logit = [&](int h, int k, int s) {
        const float vac = ac[(((size_t)b * H + h) * M + sa) * M + s] * scale;
        const float vbc = bc[(((size_t)b * H + h) * (M + 1) + (k ? 1 + sa : 0)) * M + s] * scale;
        return (s_ab[k][h] + vbc) + vac;
    };
    for (int h = warp; h < H; h += n_warps) {
        float mx = neg_inf(), sum = 0.f;
        for (int s = lane; s < M; s += 32) {
            if (!s_right_ok[s]) continue;
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float v = logit(h, k, s);
                if (v > mx) {
                    sum = sum * expf(mx - v) + 1.f;
                    mx = v;
                } else if (v > neg_inf()) {
                    sum += expf(v - mx);
                }
            }
        }
        const float top = warp_max_f(mx);
        sum = isinf(mx) ? 0.f : sum * expf(mx - top);
        sum = warp_sum_f(sum);
        if (lane == 0) s_lse[h] = isinf(top) ? top : top + logf(sum);
    }
    for (int i = tid; i < kMaxHeads * 4; i += kLinkThreads) s_red[i / 4][i & 3] = 0.f;
    __syncthreads();
    // pass A: Gs[h] = sum over the row's cells of G w[h]; every thread walks its cells, heads in registers
    const float *grow = links_grad + ((size_t)b * L + a) * 2 * L;
    float gs_part[kMaxHeads];
    for (int h = 0; h < H; h++) gs_part[h] = 0.f;
    for (int i = tid; i < 2 * M; i += kLinkThreads) {
        const int k = i / M, s = i - k * M;
        if (!s_right_ok[s]) continue;
        const float G = grow[(size_t)k * L + nodes[s]];
        if (G == 0.f) continue;
        float mx = neg_inf();
        for (int h = 0; h < H; h++) mx = fmaxf(mx, (logit(h, k, s) - s_lse[h]) + s_lg[h]);
        if (isinf(mx)) continue;  // the cell is -inf: no gradient
        float sum = 0.f;
        for (int h = 0; h < H; h++) {
            const float t = (logit(h, k, s) - s_lse[h]) + s_lg[h];
            if (t > neg_inf()) sum += expf(t - mx);
        }
        const float inv = G / sum;
        for (int h = 0; h < H; h++) {
            const float t = (logit(h, k, s) - s_lse[h]) + s_lg[h];
            if (t > neg_inf()) gs_part[h] += expf(t - mx) * inv;
        }
    }
    for (int h = 0; h < H; h++) {
        const float v = warp_sum_f(gs_part[h]);
        if (lane == 0) s_red[h][warp] = v;
    }
    __syncthreads();
    if (tid < H) s_gs[tid] = (s_red[tid][0] + s_red[tid][1]) + (s_red[tid][2] + s_red[tid][3]);
    __syncthreads();
    if (warp == n_warps - 1) {  // gate logits: d lg - softmax(gates) sum d lg
        const float tot = warp_sum_f(lane < H ? s_gs[lane] : 0.f);
        if (lane < H) dg[lane] = s_gs[lane] - gate_p * tot;
    }
    // pass B: d logit of every cell and head, and the row sums per left option
    float ab_part[2][kMaxHeads];
    for (int h = 0; h < H; h++) ab_part[0][h] = ab_part[1][h] = 0.f;
    for (int i = tid; i < 2 * M; i += kLinkThreads) {
        const int k = i / M, s = i - k * M;
        if (!s_right_ok[s]) continue;
        const float G = grow[(size_t)k * L + nodes[s]];
        float mx = neg_inf(), sum = 0.f;
        for (int h = 0; h < H; h++) mx = fmaxf(mx, (logit(h, k, s) - s_lse[h]) + s_lg[h]);
        if (!isinf(mx))
            for (int h = 0; h < H; h++) {
                const float t = (logit(h, k, s) - s_lse[h]) + s_lg[h];
                if (t > neg_inf()) sum += expf(t - mx);
            }
        float *X = k ? X1 : X0;
        for (int h = 0; h < H; h++) {
            const float lgt = logit(h, k, s);
            float d = 0.f;
            if (lgt > neg_inf()) {
                const float t = (lgt - s_lse[h]) + s_lg[h];
                const float dlp = (G != 0.f && !isinf(mx)) ? G * expf(t - mx) / sum : 0.f;
                d = (dlp - expf(lgt - s_lse[h]) * s_gs[h]) * scale;
            }
            X[(((size_t)b * H + h) * M + sa) * M + s] = d;
            ab_part[k][h] += d;
        }
    }
    __syncthreads();  // s_red is reused
    for (int k = 0; k < 2; k++) {
        for (int h = 0; h < H; h++) {
            const float v = warp_sum_f(ab_part[k][h]);
            if (lane == 0) s_red[h][warp] = v;
        }
        __syncthreads();
        if (tid < H) dab[(((size_t)b * H + tid) * M + sa) * 2 + k] = (s_red[tid][0] + s_red[tid][1]) + (s_red[tid][2] + s_red[tid][3]);
        __syncthreads();
    }
}

// Gradients of the packed features from X0, X1 and dab, one block per (sentence, head):
//   dqm[a]      = dab[a][0] klm[0] + dab[a][1] klm[1 + a] + sum_s (X0 + X1)[a][s] krm[s]
//   dklm[1 + a] = dab[a][1] qm[a] + sum_s X1[a][s] krm[s]
//   dklm[0]     = sum_a ( dab[a][0] qm[a] + sum_s X0[a][s] krm[s] )
//   dkrm[s]     = sum_a ( (X0 + X1)[a][s] qm[a] + X0[a][s] klm[0] + X1[a][s] klm[1 + a] )
// and scattered to the nodes: dq[nodes[a]], dkr[nodes[s]], dkl[nodes[a] - 1] and dkl[0] (which also takes row 1 of the
// first main-chain node, whose left option 1 is node 0 again).  dq, dkl, dkr [B][L][H][D] f32 were zero-filled.
__global__ void __launch_bounds__(256)
    links_features_grad_simple_kernel(const float *__restrict__ X0, const float *__restrict__ X1, const float *__restrict__ dab,
                               const float *__restrict__ qm, const float *__restrict__ klm, const float *__restrict__ krm,
                               const int *__restrict__ nodes, int M, int L, int H, int D, float *__restrict__ dq,
                               float *__restrict__ dkl, float *__restrict__ dkr) {
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t bh = (size_t)b * H + h;
    const float *x0 = X0 + bh * M * M, *x1 = X1 + bh * M * M, *da = dab + bh * M * 2;
    const float *q = qm + bh * M * D, *kl = klm + bh * (M + 1) * D, *kr = krm + bh * M * D;
    const int HD = H * D;
    // outputs indexed (row, d): one thread each, sums over the other node index
    for (int i = threadIdx.x; i < M * D; i += blockDim.x) {
        const int r = i / D, d = i - r * D;
        // row r as a parent a
        float s0 = 0.f, s1 = 0.f;  // sum_s X0[a][s] krm[s][d], sum_s X1[a][s] krm[s][d]
        for (int s = 0; s < M; s++) {
            const float k = kr[(size_t)s * D + d];
            s0 = fmaf(x0[(size_t)r * M + s], k, s0);
            s1 = fmaf(x1[(size_t)r * M + s], k, s1);
        }
        const float d0 = da[r * 2 + 0], d1 = da[r * 2 + 1];
        const float qv = q[(size_t)r * D + d];
        const float g_q = d0 * kl[d] + d1 * kl[(size_t)(1 + r) * D + d] + (s0 + s1);
        const float g_kl1 = d1 * qv + s1;      // left option 1 of node r
        const float g_kl0 = d0 * qv + s0;      // this node's part of the "no left child" row
        // row r as a child s
        float t = 0.f;
        for (int a = 0; a < M; a++) {
            const float v0 = x0[(size_t)a * M + r], v1 = x1[(size_t)a * M + r];
            t = fmaf(v0 + v1, q[(size_t)a * D + d], t);
            t = fmaf(v0, kl[d], t);
            t = fmaf(v1, kl[(size_t)(1 + a) * D + d], t);
        }
        const int node = nodes[r];
        const size_t at = ((size_t)b * L + node) * HD + (size_t)h * D + d;
        dq[at] = g_q;
        dkr[at] = t;
        const int left = node - 1 > 0 ? node - 1 : 0;
        atomicAdd(dkl + ((size_t)b * L + left) * HD + (size_t)h * D + d, g_kl1);
        atomicAdd(dkl + ((size_t)b * L + 0) * HD + (size_t)h * D + d, g_kl0);
    }
}

// The same with every operand staged in shared memory once and 4 x 4 outputs per thread (D a multiple of 4): the five
// products are small matrix products, M x M x D each, and a thread that computes one output from global memory
// re-reads every operand M or D times.  The contributions to the "no left child" row of kl are summed in shared
// memory and leave as one atomic per column (all M parents share that row).  xs = row pitch of X0 / X1 in shared
// memory, M rounded up to a multiple of 4 with the padding zero.
constexpr int kFeatThreads = 320;
__global__ void __launch_bounds__(kFeatThreads)
    links_features_grad_kernel(const float *__restrict__ X0, const float *__restrict__ X1, const float *__restrict__ dab,
                               const float *__restrict__ qm, const float *__restrict__ klm, const float *__restrict__ krm,
                               const int *__restrict__ nodes, int M, int L, int H, int D, int xs, float *__restrict__ dq,
                               float *__restrict__ dkl, float *__restrict__ dkr) {
    extern __shared__ __align__(16) float s_feat[];
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const size_t bh = (size_t)b * H + h;
    const float *da = dab + bh * M * 2;
    const int HD = H * D;
    float *sx0 = s_feat, *sx1 = sx0 + (size_t)M * xs, *sq = sx1 + (size_t)M * xs, *skr = sq + (size_t)M * D;
    float *skl = skr + (size_t)M * D, *skl0 = skl + (size_t)(M + 1) * D;  // skl0 [D]: sum for row 0 of kl
    {
        const float *x0 = X0 + bh * M * M, *x1 = X1 + bh * M * M;
        for (int i = tid; i < M * xs; i += kFeatThreads) {
            const int r = i / xs, c = i - r * xs;
            sx0[i] = c < M ? x0[(size_t)r * M + c] : 0.f;
            sx1[i] = c < M ? x1[(size_t)r * M + c] : 0.f;
        }
        const float *q = qm + bh * M * D, *kr = krm + bh * M * D, *kl = klm + bh * (M + 1) * D;
        for (int i = tid; i < M * D; i += kFeatThreads) sq[i] = q[i], skr[i] = kr[i];
        for (int i = tid; i < (M + 1) * D; i += kFeatThreads) skl[i] = kl[i];
        for (int i = tid; i < D; i += kFeatThreads) skl0[i] = 0.f;
    }
    __syncthreads();
    const int CG = D / 4, micro = ((M + 3) / 4) * CG;
    for (int mt = tid; mt < micro; mt += kFeatThreads) {
        const int r0 = (mt / CG) * 4, d0 = (mt % CG) * 4;
        int rr[4];  // rows of this tile, clamped: a row past the end repeats the last one and is not written
#pragma unroll
        for (int i = 0; i < 4; i++) rr[i] = r0 + i < M ? r0 + i : M - 1;
        // rows as parents a: s0 = sum_s X0[a][s] krm[s], s1 = sum_s X1[a][s] krm[s]
        float a0[4][4], a1[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) a0[i][c] = a1[i][c] = 0.f;
        for (int s = 0; s < xs; s += 4) {
            float4 x0v[4], x1v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                x0v[i] = *reinterpret_cast<const float4 *>(sx0 + (size_t)rr[i] * xs + s);
                x1v[i] = *reinterpret_cast<const float4 *>(sx1 + (size_t)rr[i] * xs + s);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int sr = s + j < M ? s + j : M - 1;  // padding columns of X are zero
                const float4 kv = *reinterpret_cast<const float4 *>(skr + (size_t)sr * D + d0);
                const float kc[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float v0 = j == 0 ? x0v[i].x : j == 1 ? x0v[i].y : j == 2 ? x0v[i].z : x0v[i].w;
                    const float v1 = j == 0 ? x1v[i].x : j == 1 ? x1v[i].y : j == 2 ? x1v[i].z : x1v[i].w;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        a0[i][c] = fmaf(v0, kc[c], a0[i][c]);
                        a1[i][c] = fmaf(v1, kc[c], a1[i][c]);
                    }
                }
            }
        }
        float kl0_part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = r0 + i;
            if (r >= M) continue;
            const float w0 = da[r * 2 + 0], w1 = da[r * 2 + 1];
            const int node = nodes[r];
            const size_t at = ((size_t)b * L + node) * HD + (size_t)h * D + d0;
            const int left = node - 1 > 0 ? node - 1 : 0;
            float *dkl_row = dkl + ((size_t)b * L + left) * HD + (size_t)h * D + d0;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float qv = sq[(size_t)r * D + d0 + c];
                dq[at + c] = w0 * skl[d0 + c] + w1 * skl[(size_t)(1 + r) * D + d0 + c] + (a0[i][c] + a1[i][c]);
                atomicAdd(dkl_row + c, w1 * qv + a1[i][c]);  // left option 1 of node r
                kl0_part[c] += w0 * qv + a0[i][c];         // this node's part of the "no left child" row
            }
        }
#pragma unroll
        for (int c = 0; c < 4; c++) atomicAdd(skl0 + d0 + c, kl0_part[c]);
        // rows as children s: sum_a ( (X0 + X1)[a][s] qm[a] + X0[a][s] klm[0] + X1[a][s] klm[1 + a] )
        float t[4][4], x0sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) t[i][c] = 0.f;
        for (int a = 0; a < M; a++) {
            const float4 xa0 = *reinterpret_cast<const float4 *>(sx0 + (size_t)a * xs + r0);
            const float4 xa1 = *reinterpret_cast<const float4 *>(sx1 + (size_t)a * xs + r0);
            const float4 qv = *reinterpret_cast<const float4 *>(sq + (size_t)a * D + d0);
            const float4 k1 = *reinterpret_cast<const float4 *>(skl + (size_t)(1 + a) * D + d0);
            const float v0[4] = {xa0.x, xa0.y, xa0.z, xa0.w}, v1[4] = {xa1.x, xa1.y, xa1.z, xa1.w};
            const float qc[4] = {qv.x, qv.y, qv.z, qv.w}, kc[4] = {k1.x, k1.y, k1.z, k1.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                x0sum[i] += v0[i];
#pragma unroll
                for (int c = 0; c < 4; c++) t[i][c] = fmaf(v1[i], kc[c], fmaf(v0[i] + v1[i], qc[c], t[i][c]));
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = r0 + i;
            if (r >= M) continue;
            const size_t at = ((size_t)b * L + nodes[r]) * HD + (size_t)h * D + d0;
#pragma unroll
            for (int c = 0; c < 4; c++) dkr[at + c] = fmaf(x0sum[i], skl[d0 + c], t[i][c]);
        }
    }
    __syncthreads();
    for (int d = tid; d < D; d += kFeatThreads) atomicAdd(dkl + ((size_t)b * L + 0) * HD + (size_t)h * D + d, skl0[d]);
}

}  // namespace

int launch_links_scores(const float *qm, const float *klm, const float *krm, int M, int B, int H, int D, float *ac,
                        float *bc, cudaStream_t st) {
    if (B == 0 || M == 0) return PCFGNAT_OK;
    const dim3 grid((M + kScoreTile - 1) / kScoreTile, (2 * M + 1 + kScoreTile - 1) / kScoreTile, B * H);
    links_scores_kernel<<<grid, 256, 0, st>>>(qm, klm, krm, M, D, ac, bc);
    return cuda_rc(cudaGetLastError());
}

int launch_links_backward(const float *links_grad, const float *ac, const float *bc, const float *qm, const float *klm,
                          const float *krm, const float *gates, const uint8_t *nonpad, const uint8_t *left_mask,
                          const uint8_t *right_mask, const uint8_t *main_chain, const int *slot_of, const int *nodes, int M,
                          int B, int L, int H, int D, float *X0, float *X1, float *dab, float *dq, float *dkl, float *dkr,
                          float *dgates, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    if (H > kMaxHeads) return PCFGNAT_ERR_TOO_LARGE;
    const float scale = 1.f / sqrtf((float)D);
    const size_t smem = (size_t)(M + 16) / 16 * 16;
    if (smem > 40 * 1024) return PCFGNAT_ERR_TOO_LARGE;
    links_scores_grad_kernel<<<dim3(L, B), kLinkThreads, smem, st>>>(links_grad, ac, bc, qm, klm, gates, nonpad, left_mask,
                                                                     right_mask, main_chain, slot_of, nodes, M, L, H, D, scale,
                                                                     X0, X1, dab, dgates);
    if (cudaGetLastError() != cudaSuccess) return PCFGNAT_ERR_CUDA;
    if (M == 0) return PCFGNAT_OK;
    // operands in shared memory and 4 x 4 outputs per thread where D allows it and they fit (M = 80, D = 64: 113 KB)
    const int xs = (M + 3) / 4 * 4;
    const size_t feat_smem = ((size_t)2 * M * xs + (size_t)(3 * M + 1) * D + D) * sizeof(float);
    if (D % 4 == 0 && feat_smem <= (size_t)kSmemLimit - 1024 &&
        ensure_dynamic_smem(links_features_grad_kernel, feat_smem) == cudaSuccess)
        links_features_grad_kernel<<<dim3(H, B), kFeatThreads, feat_smem, st>>>(X0, X1, dab, qm, klm, krm, nodes, M, L, H, D,
                                                                              xs, dq, dkl, dkr);
    else
        links_features_grad_simple_kernel<<<dim3(H, B), 256, 0, st>>>(X0, X1, dab, qm, klm, krm, nodes, M, L, H, D, dq, dkl,
                                                                      dkr);
    return cuda_rc(cudaGetLastError());
}

int launch_links_gather(const void *q, const void *kl, const void *kr, int is_half, const int *nodes, int M, int B, int L,
                        int H, int D, float *qm, float *klm, float *krm, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    links_gather_kernel<<<dim3(M + 1, B), 256, 0, st>>>(q, kl, kr, is_half, nodes, M, L, H, D, qm, klm, krm);
    return cuda_rc(cudaGetLastError());
}

int launch_links_from_scores(const float *ac, const float *bc, const float *qm, const float *klm, const float *gates,
                             const uint8_t *nonpad, const uint8_t *left_mask, const uint8_t *right_mask,
                             const uint8_t *main_chain, const int *slot_of, const int *nodes, int M, int B, int L, int H,
                             int D, float *links, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    if (H > kMaxHeads) return PCFGNAT_ERR_TOO_LARGE;
    const float scale = 1.f / sqrtf((float)D);
    const size_t smem = (size_t)(M + 16) / 16 * 16;
    if (smem > 40 * 1024) return PCFGNAT_ERR_TOO_LARGE;
    if (H == 8)
        links_from_scores_kernel<8><<<dim3(L, B), kLinkThreads, smem, st>>>(ac, bc, qm, klm, gates, nonpad, left_mask, right_mask,
                                                                          main_chain, slot_of, nodes, M, L, H, D, scale, links);
    else
        links_from_scores_kernel<0><<<dim3(L, B), kLinkThreads, smem, st>>>(ac, bc, qm, klm, gates, nonpad, left_mask, right_mask,
                                                                          main_chain, slot_of, nodes, M, L, H, D, scale, links);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
