// Transition log-probabilities ("links") of the PCFG-NAT decoder from per-head attention scores,
// max_left == 1: the tail of extract_links() of the reference model
// (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:140-201) in one launch.
//
// The reference forms, per sentence b, node a, head h (chunk of the decoder dimension):
//     ab[a][k][h]    = q[a][h] . kl[left(a,k)][h] / sqrt(D)     left(a,0) = 0 (no left child), left(a,1) = a - 1
//     bc[a][k][c][h] = kl[left(a,k)][h] . kr[c][h] / sqrt(D)
//     ac[a][c][h]    = q[a][h] . kr[c][h] / sqrt(D)
// masks ab where left(a,k) is padding or outside a's left subtree and ac where c is padding, outside a's right
// subtree or not a main-chain node, normalises (ab + bc) + ac jointly over (k, c) per head (log-softmax), mixes
// the heads with log-softmax(gate logits) by log-sum-exp, and sets the whole row to -inf when a has no admissible
// left or no admissible right child.  That is ~30 element-wise / gather / roll / softmax launches over
// [B, L, 2, L, heads] tensors; here the two L x L score matrices per head come from library batched GEMMs
// (ac = q kr^T, bc = kl kr^T, unscaled) and one block per (sentence, node) does the rest.
#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kLinkThreads = 256;
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

// Only main-chain nodes have right children and only main-chain nodes are right children, so the score matrices
// are compact: with M main-chain nodes and slot_of[node] = index among them (or -1),
//   ac [B][H][M][M]      ac[b][h][slot(a)][slot(c)] = q[a] . kr[c]
//   bc [B][H][M + 1][M]  row 0 = kl[0] . kr[c] (no left child), row 1 + slot(a) = kl[a - 1] . kr[c]
// both unscaled.  q, kl: [B][L][H][D] f32; gates [B][L][H] f32 (logits); nonpad [B][L] u8; left_mask, right_mask
// [L][L] u8 (1 = not allowed), main_chain [L] u8.  A node that is not on the main chain gets a -inf row.
// HT: number of heads known at compile time (terms of a cell stay in registers between the two reductions over
// the heads), or 0 for any number up to kMaxHeads.
template <int HT>
__global__ void __launch_bounds__(kLinkThreads)
    links_from_scores_kernel(const float *__restrict__ ac, const float *__restrict__ bc, const float *__restrict__ q,
                             const float *__restrict__ kl, const float *__restrict__ gates,
                             const uint8_t *__restrict__ nonpad, const uint8_t *__restrict__ left_mask,
                             const uint8_t *__restrict__ right_mask, const uint8_t *__restrict__ main_chain,
                             const int *__restrict__ slot_of, int M, int L, int H, int D, float scale,
                             float *__restrict__ links) {
    extern __shared__ uint8_t s_right_ok[];  // [L] right child c admissible for this node
    __shared__ float s_ab[2][kMaxHeads], s_lse[kMaxHeads], s_lg[kMaxHeads];
    const int a = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = kLinkThreads / 32;
    const uint8_t *np = nonpad + (size_t)b * L;
    float *out = links + ((size_t)b * L + a) * 2 * L;
    // admissible children of a at all?  (the reference's link_left_nouse_mask / link_right_nouse_mask)
    int any_left = 0, any_right = 0;
    for (int j = tid; j < L; j += kLinkThreads) {
        const bool there = np[j] != 0;
        any_left |= there && !left_mask[(size_t)a * L + j];
        const bool r_ok = there && !right_mask[(size_t)a * L + j] && main_chain[j];
        s_right_ok[j] = r_ok;
        any_right |= r_ok;
    }
    any_left = __syncthreads_or(any_left);
    any_right = __syncthreads_or(any_right);
    const int sa = slot_of[a];
    if (!any_left || !any_right || sa < 0) {
        for (int i = tid; i < 2 * L; i += kLinkThreads) out[i] = neg_inf();
        return;
    }
    const int left1 = a >= 1 ? a - 1 : 0;  // the reference's _max_left_index[a][1]
    const bool ok_left0 = np[0] && !left_mask[(size_t)a * L + 0];
    const bool ok_left1 = np[left1] && !left_mask[(size_t)a * L + left1];
    // ab[k][h]: one warp per head at a time, lanes over the chunk dimension
    for (int h = warp; h < H; h += n_warps) {
        const float *qa = q + (((size_t)b * L + a) * H + h) * D;
        const float *k0 = kl + (((size_t)b * L + 0) * H + h) * D;
        const float *k1 = kl + (((size_t)b * L + left1) * H + h) * D;
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
    if (tid == 0) {  // log-softmax of the gate logits over the heads
        const float *gt = gates + ((size_t)b * L + a) * H;
        float mx = neg_inf();
        for (int h = 0; h < H; h++) mx = fmaxf(mx, gt[h]);
        float sum = 0.f;
        for (int h = 0; h < H; h++) sum += expf(gt[h] - mx);
        const float lse = mx + logf(sum);
        for (int h = 0; h < H; h++) s_lg[h] = gt[h] - lse;
    }
    __syncthreads();
    // logit of (k, c) for head h: (ab + bc) + ac, -inf where the right child is not admissible
    auto logit = [&](int h, int k, int c, bool right_ok) {
        if (!right_ok) return neg_inf();
        const int sc = slot_of[c];  // >= 0: an admissible right child is a main-chain node
        const float vac = ac[(((size_t)b * H + h) * M + sa) * M + sc] * scale;
        const float vbc = bc[(((size_t)b * H + h) * (M + 1) + (k ? 1 + sa : 0)) * M + sc] * scale;
        return (s_ab[k][h] + vbc) + vac;
    };
    // pass 1: log-sum-exp over (k, c) per head
    for (int h = warp; h < H; h += n_warps) {
        float mx = neg_inf(), sum = 0.f;
        for (int c = lane; c < L; c += 32) {
            const bool right_ok = s_right_ok[c];
            if (!right_ok) continue;
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const float v = logit(h, k, c, right_ok);
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
    for (int i = tid; i < 2 * L; i += kLinkThreads) {
        const int k = i / L, c = i - k * L;
        float res = neg_inf();
        if (s_right_ok[c]) {
            if (HT > 0) {
                float term[HT > 0 ? HT : 1];
                float mx = neg_inf();
#pragma unroll
                for (int h = 0; h < HT; h++) {
                    term[h] = (logit(h, k, c, true) - s_lse[h]) + s_lg[h];
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
                for (int h = 0; h < H; h++) mx = fmaxf(mx, (logit(h, k, c, true) - s_lse[h]) + s_lg[h]);
                if (!isinf(mx)) {
                    float sum = 0.f;
                    for (int h = 0; h < H; h++) {
                        const float t = (logit(h, k, c, true) - s_lse[h]) + s_lg[h];
                        if (t > neg_inf()) sum += expf(t - mx);
                    }
                    res = mx + logf(sum);
                }
            }
        }
        out[i] = res;
    }
}

}  // namespace

int launch_links_from_scores(const float *ac, const float *bc, const float *q, const float *kl, const float *gates,
                             const uint8_t *nonpad, const uint8_t *left_mask, const uint8_t *right_mask,
                             const uint8_t *main_chain, const int *slot_of, int M, int B, int L, int H, int D,
                             float *links, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    if (H > kMaxHeads) return PCFGNAT_ERR_TOO_LARGE;
    const float scale = 1.f / sqrtf((float)D);
    const size_t smem = (size_t)(L + 15) / 16 * 16;
    if (smem > 40 * 1024) return PCFGNAT_ERR_TOO_LARGE;
    if (H == 8)
        links_from_scores_kernel<8><<<dim3(L, B), kLinkThreads, smem, st>>>(ac, bc, q, kl, gates, nonpad, left_mask, right_mask,
                                                                          main_chain, slot_of, M, L, H, D, scale, links);
    else
        links_from_scores_kernel<0><<<dim3(L, B), kLinkThreads, smem, st>>>(ac, bc, q, kl, gates, nonpad, left_mask, right_mask,
                                                                          main_chain, slot_of, M, L, H, D, scale, links);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
