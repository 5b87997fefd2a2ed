// The small reductions and selections the criterion does around the DP operators, one launch each
// instead of a dozen element-wise torch kernels:
//
//  * loss_stats_kernel — the three numbers the scalar loss is formed from
//    (fs_plugins/criterions/nat_pcfg_loss.py:117-135: invalid sentences zeroed, per-sentence loss divided by
//    its target length, batch mean; the division by the sentence count is left to the caller so that the
//    three numbers can be summed over ranks first);
//  * loss_stats_exchange_kernel — the same three numbers summed over the GPUs of a sentence-sharded job, in the
//    same launch: every rank stores its partial into every peer's exchange buffer over NVLink (plain peer
//    stores, no multimem) and adds up what the peers stored into its own.  It replaces the 12-byte NCCL
//    all-reduce that otherwise follows the kernel, whose launch latency is several percent of a step;
//  * glance_select_kernel — the glancing sampler between the two decoder passes
//    (nat_pcfg_loss.py:216-267, all three strategies): alignment -> match mask, oracle tokens, number of
//    already-correct predictions, the kept positions (the glance_nums ones with the largest noise, or an
//    independent draw per node), and the decoder input with the oracle tokens revealed at those positions;
//  * force_emit_kernel / force_emit_grad_kernel — the force-emit mask of the training pass
//    (nat_pcfg_loss.py:116-121): a node whose token was revealed may only emit the target position it is
//    aligned to, and carries no gradient.
#include "common.cuh"

namespace pcfgnat {

namespace {

__device__ __forceinline__ float block_sum(float v, float *scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < n_warps; i++) t += scratch[i];  // same order in every thread: deterministic
    return t;
}

// stats[0] = sum over valid sentences of loss_b / max(n_b, 1); stats[1] = B; stats[2] = invalid sentences
// (loss_b infinite or NaN).
__global__ void loss_stats_kernel(const float *__restrict__ loss, const int64_t *__restrict__ tl, int B, float *stats) {
    __shared__ float scratch[32];
    chain_begin();
    float s = 0.f, bad = 0.f;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const float v = loss[b];
        if (isinf(v) || isnan(v)) {
            bad += 1.f;
        } else {
            const int64_t n = tl[b];
            s += v / (float)(n < 1 ? 1 : n);
        }
    }
    s = block_sum(s, scratch);
    bad = block_sum(bad, scratch);
    if (threadIdx.x == 0) {
        stats[0] = s;
        stats[1] = (float)B;
        stats[2] = bad;
    }
}

// Exchange buffer of a rank (PCFGNAT_EXCHANGE_BYTES(world) bytes, zeroed once, mapped into every peer):
//   [0]            uint32 epoch: calls made so far (only this rank's kernel touches it)
//   [64 + 32 * (parity * world + src)]  slot written by rank src: float data[3], uint32 flag = epoch of the call
// Two parities: a rank can be at most one call ahead of a peer (it needs the peer's slot of the current call to
// finish it), so the slots of call e are not overwritten before call e + 2, when every rank has read them.
__global__ void loss_stats_exchange_kernel(const float *__restrict__ loss, const int64_t *__restrict__ tl, int B,
                                           const uint64_t *__restrict__ peer_bufs, int rank, int world, float *stats,
                                           int *status) {
    __shared__ float scratch[32];
    __shared__ float part[PCFGNAT_EXCHANGE_MAX_WORLD][3];
    __shared__ unsigned epoch_s;
    chain_begin();
    float s = 0.f, bad = 0.f;
    bool arrived = true;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const float v = loss[b];
        if (isinf(v) || isnan(v)) {
            bad += 1.f;
        } else {
            const int64_t n = tl[b];
            s += v / (float)(n < 1 ? 1 : n);
        }
    }
    s = block_sum(s, scratch);
    bad = block_sum(bad, scratch);
    char *mine = reinterpret_cast<char *>(peer_bufs[rank]);
    if (threadIdx.x == 0) epoch_s = ++*reinterpret_cast<unsigned *>(mine);
    __syncthreads();
    const unsigned epoch = epoch_s;
    const size_t slot0 = 64 + (size_t)32 * ((epoch & 1u) * world);
    if ((int)threadIdx.x < world) {
        // this rank's partial into peer threadIdx.x's buffer (its own included), data before flag
        char *dst = reinterpret_cast<char *>(peer_bufs[threadIdx.x]) + slot0 + (size_t)32 * rank;
        volatile float *d = reinterpret_cast<volatile float *>(dst);
        d[0] = s;
        d[1] = (float)B;
        d[2] = bad;
        __threadfence_system();
        *reinterpret_cast<volatile unsigned *>(dst + 16) = epoch;
        // the partial peer threadIdx.x stored here; bounded wait: 2^21 polls 200 ns apart, about half a second
        const char *src = mine + slot0 + (size_t)32 * threadIdx.x;
        bool there = false;
        for (unsigned it = 0; it < (1u << 21) && !there; ++it) {
            there = *reinterpret_cast<const volatile unsigned *>(src + 16) == epoch;
            if (!there) __nanosleep(200);
        }
        __threadfence_system();
        const volatile float *q = reinterpret_cast<const volatile float *>(src);
        part[threadIdx.x][0] = there ? q[0] : 0.f;
        part[threadIdx.x][1] = there ? q[1] : 0.f;
        part[threadIdx.x][2] = there ? q[2] : 0.f;
        arrived = there;
        if (!there) flag(status, PCFGNAT_STATUS_TIMEOUT);
    }
    const int missing = __syncthreads_count((int)threadIdx.x < world && !arrived);
    if (threadIdx.x == 0) {
        float t0 = 0.f, t1 = 0.f, t2 = 0.f;
        for (int r = 0; r < world; r++) {  // rank order on every rank: the same sum everywhere
            t0 += part[r][0];
            t1 += part[r][1];
            t2 += part[r][2];
        }
        // a short sum must not pass for a loss: with a peer missing all three numbers are NaN, so that the
        // host sees it in the value it reads anyway (the status word carries PCFGNAT_STATUS_TIMEOUT as well)
        const float poison = missing ? CUDART_NAN_F : 0.f;
        stats[0] = t0 + poison;
        stats[1] = t1 + poison;
        stats[2] = t2 + poison;
    }
}

// One block per sentence.  path[l] = aligned target position of graph node l, or < 0.
//   aligned[l]   = path[l] >= 0                                   (taken before the range check below)
//   p            = path[l] if 0 <= path[l] < T else -1
//   matchmask[b][t][l] = (p == t)
//   oracle[l]    = tgt[b][max(p, 0)]
//   same         = #{l : pred[l] == oracle[l] and aligned[l]}
// strategy PCFGNAT_GLANCE_NUMBER_RANDOM (nat_pcfg_loss.py:232-238):
//   k            = (long)((n_b - same) * context_p + 0.5)          (float32 arithmetic, as torch does it)
//   keep[l]      = noise'[l] >= (k-th largest of noise')           noise' = noise, -100 where not aligned
//                = fewer than k entries of noise' are strictly larger than noise'[l];   nothing if k == 0,
//                  and k < 0 (never the case for a real alignment) acts as k = 1
// strategy PCFGNAT_GLANCE_CMLM (:240-246): the same with k = (long)(n_b * uniform[b] + 0.5), uniform [B]
// strategy PCFGNAT_GLANCE_FRACTION (glance_strategy None, :229-230):
//   keep[l]      = aligned[l] and uniform[b][l] < ((n_b - same) / n_b) * context_p,  uniform [B][L];
//   glance_num   = number of kept nodes
//   glat_prev[l] = keep[l] ? oracle[l] : prev[l]
// For the two counting strategies the reference then draws rand < keep_prob with keep_prob in {0, 1}: the same
// mask, so no second draw.
__global__ void glance_select_kernel(const int64_t *__restrict__ path, const int64_t *__restrict__ pred,
                                     const int64_t *__restrict__ tgt, const int64_t *__restrict__ prev,
                                     const int64_t *__restrict__ tl, const float *__restrict__ noise,
                                     const float *__restrict__ uniform, int strategy, float context_p, int L, int T,
                                     uint8_t *matchmask, int64_t *oracle, int64_t *same_num, int64_t *glance_num,
                                     uint8_t *keep, int64_t *glat_prev) {
    extern __shared__ float sm_noise[];  // [L]
    __shared__ float scratch[32];
    const int b = blockIdx.x;
    const int64_t *pb = path + (size_t)b * L;
    float same = 0.f;
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
        const int64_t raw = pb[l];
        const bool aligned = raw >= 0;
        const int p = (raw >= 0 && raw < T) ? (int)raw : -1;
        const int64_t o = tgt[(size_t)b * T + (p < 0 ? 0 : p)];
        oracle[(size_t)b * L + l] = o;
        if (aligned && pred[(size_t)b * L + l] == o) same += 1.f;
        if (strategy == PCFGNAT_GLANCE_FRACTION) sm_noise[l] = aligned ? 1.f : 0.f;
        else sm_noise[l] = aligned ? noise[(size_t)b * L + l] : -100.f;
    }
    for (int i = threadIdx.x; i < T * L; i += blockDim.x) {
        const int t = i / L, l = i - t * L;
        matchmask[(size_t)b * T * L + i] = pb[l] == t;
    }
    same = block_sum(same, scratch);  // exact: a count below 2^24; its barriers also publish sm_noise
    const int64_t n = tl[b];
    const int64_t same_i = (int64_t)same;
    if (strategy == PCFGNAT_GLANCE_FRACTION) {
        const float kp = ((float)(n - same_i) / (float)n) * context_p;
        float kept = 0.f;
        for (int l = threadIdx.x; l < L; l += blockDim.x) {
            const bool k_l = uniform[(size_t)b * L + l] < kp * sm_noise[l];
            keep[(size_t)b * L + l] = k_l;
            glat_prev[(size_t)b * L + l] = k_l ? oracle[(size_t)b * L + l] : prev[(size_t)b * L + l];
            kept += k_l ? 1.f : 0.f;
        }
        kept = block_sum(kept, scratch);
        if (threadIdx.x == 0) {
            same_num[b] = same_i;
            glance_num[b] = (int64_t)kept;
        }
        return;
    }
    const int64_t k = strategy == PCFGNAT_GLANCE_CMLM ? (int64_t)((float)n * uniform[b] + 0.5f)
                                                      : (int64_t)((float)(n - same_i) * context_p + 0.5f);
    if (threadIdx.x == 0) {
        same_num[b] = same_i;
        glance_num[b] = k;
    }
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
        const float mine = sm_noise[l];
        int larger = 0;
        for (int j = 0; j < L; j++) larger += sm_noise[j] > mine;
        const bool kp = k != 0 && larger < (k < 1 ? 1 : k);  // a negative k indexes the sorted list at 0, as torch's clip does
        keep[(size_t)b * L + l] = kp;
        glat_prev[(size_t)b * L + l] = kp ? oracle[(size_t)b * L + l] : prev[(size_t)b * L + l];
    }
}

// out[b][l][t] = keep[b][l] && !matchmask[b][t][l] ? -inf : match[b][l][t]   (out may be match itself)
__global__ void force_emit_kernel(const float *match, const uint8_t *__restrict__ matchmask,
                                  const uint8_t *__restrict__ keep, int L, int T, size_t total, float *out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / T;  // b * L + l
        const int t = (int)(i - row * T);
        const size_t b = row / L;
        const int l = (int)(row - b * L);
        float v = match[i];
        if (keep[row] && !matchmask[(b * T + t) * L + l]) v = neg_inf();
        out[i] = v;
    }
}

// out[b][l][t] = keep[b][l] ? 0 : grad[b][l][t]   (out may be grad itself)
__global__ void force_emit_grad_kernel(const float *grad, const uint8_t *__restrict__ keep, int T, size_t total,
                                       float *out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = keep[i / T] ? 0.f : grad[i];
}

}  // namespace

int launch_loss_stats(const float *loss, const int64_t *tl, int B, float *stats, cudaStream_t st) {
    launch_chain(loss_stats_kernel, dim3(1), dim3(256), 0, st, loss, tl, B, stats);
    return cuda_rc(cudaGetLastError());
}

int launch_loss_stats_exchange(const float *loss, const int64_t *tl, int B, const uint64_t *peer_bufs, int rank, int world,
                               float *stats, int *status, cudaStream_t st) {
    launch_chain(loss_stats_exchange_kernel, dim3(1), dim3(256), 0, st, loss, tl, B, peer_bufs, rank, world, stats, status);
    return cuda_rc(cudaGetLastError());
}

int launch_glance_select(const int64_t *path, const int64_t *pred, const int64_t *tgt, const int64_t *prev,
                         const int64_t *tl, const float *noise, const float *uniform, int strategy, float context_p,
                         int B, int L, int T, uint8_t *matchmask, int64_t *oracle, int64_t *same_num,
                         int64_t *glance_num, uint8_t *keep, int64_t *glat_prev, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    const size_t smem = (size_t)L * sizeof(float);
    if (smem > 48 * 1024 && ensure_dynamic_smem(glance_select_kernel, smem) != cudaSuccess) return PCFGNAT_ERR_TOO_LARGE;
    glance_select_kernel<<<B, 256, smem, st>>>(path, pred, tgt, prev, tl, noise, uniform, strategy, context_p, L, T,
                                               matchmask, oracle, same_num, glance_num, keep, glat_prev);
    return cuda_rc(cudaGetLastError());
}

int launch_force_emit(const float *match, const uint8_t *matchmask, const uint8_t *keep, int B, int L, int T, float *out,
                      cudaStream_t st) {
    const size_t total = (size_t)B * L * T;
    if (total == 0) return PCFGNAT_OK;
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    force_emit_kernel<<<blocks, 256, 0, st>>>(match, matchmask, keep, L, T, total, out);
    return cuda_rc(cudaGetLastError());
}

int launch_force_emit_grad(const float *grad, const uint8_t *keep, int B, int L, int T, float *out, cudaStream_t st) {
    const size_t total = (size_t)B * L * T;
    if (total == 0) return PCFGNAT_OK;
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    force_emit_grad_kernel<<<blocks, 256, 0, st>>>(grad, keep, T, total, out);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
