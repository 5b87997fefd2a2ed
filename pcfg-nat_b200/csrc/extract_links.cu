// Transition log-probabilities ("links") of the PCFG-NAT decoder from the projected link features,
// max_left == 1: extract_links() of the reference model after its three link projections
// (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:163-199) in two launches around two
// library batched GEMMs.
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
//   (library)                  ac [B][H][M][M] = qm krm^T,  bc [B][H][M+1][M] = klm krm^T, unscaled;
//   links_from_scores_kernel   one block per (sentence, node) does the rest.
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

}  // namespace

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
