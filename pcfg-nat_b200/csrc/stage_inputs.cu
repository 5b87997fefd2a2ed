// Host plumbing for callers that stage batches from pinned host memory: one kernel that fetches exactly what the
// kernels of this library read — the decoder states of the real graph nodes and, of the transition matrix, the
// entries links[a][k][c] with a on the main chain and a < c < m_b — straight from the host buffers over PCIe
// (mapped pinned memory; no intermediate copy), and defines the rest of the main-chain rows as -inf on the device.
// For a training batch of ~90 sentences that is 14 MB over the bus instead of 33 MB for the padded tensors
// (24 MB when only the main-chain rows of the transitions are copied).  The reference has no counterpart: its
// inputs are produced on the device by the model.
#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kStageThreads = 512;

// hidden [B][L][row16 * 16 bytes] -> rows l < m_b copied; links [B][L][2][L] f32 -> for odd a < m_b and k = 0, 1:
// c in (a, m_b) copied, c <= a and c >= m_b set to -inf; odd rows a >= m_b set to -inf entirely.  Even rows are
// left as they are (the caller filled the buffer with -inf once; no kernel reads them).
__global__ void __launch_bounds__(kStageThreads)
    stage_inputs_kernel(const uint4 *__restrict__ hidden_src, uint4 *__restrict__ hidden_dst, int row16,
                        const float *__restrict__ links_src, float *__restrict__ links_dst,
                        const int64_t *__restrict__ ol, int B, int L) {
    const int warp = (blockIdx.x * kStageThreads + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int n_warps = (gridDim.x * kStageThreads) >> 5;
    // decoder states: one warp per row, 16 bytes per lane and trip
    if (hidden_src) {
        for (long long row = warp; row < (long long)B * L; row += n_warps) {
            const int b = (int)(row / L), l = (int)(row - (long long)b * L);
            long long m = ol[b];
            if (m > L) m = L;
            if (l >= m) continue;
            const uint4 *s = hidden_src + row * row16;
            uint4 *d = hidden_dst + row * row16;
            for (int i = lane; i < row16; i += 32) d[i] = s[i];
        }
    }
    // transitions: one warp per (sentence, main-chain node, left option)
    if (links_src) {
        const int Mc = L / 2;  // odd nodes below L
        for (long long seg = warp; seg < (long long)B * Mc * 2; seg += n_warps) {
            const int k = (int)(seg & 1);
            const long long r = seg >> 1;
            const int b = (int)(r / Mc), a = 2 * (int)(r - (long long)b * Mc) + 1;
            long long m = ol[b];
            if (m > L) m = L;
            const size_t at = (((size_t)b * L + a) * 2 + k) * L;
            const float *s = links_src + at;
            float *d = links_dst + at;
            const int lo = a < m ? a + 1 : L, hi = a < m ? (int)m : L;  // copied range [lo, hi)
            for (int c = lane; c < L; c += 32) d[c] = (c >= lo && c < hi) ? s[c] : neg_inf();
        }
    }
}

}  // namespace

int launch_stage_inputs(const void *hidden_src, void *hidden_dst, int row_bytes, const float *links_src, float *links_dst,
                        const int64_t *ol, int B, int L, cudaStream_t st) {
    if (B == 0) return PCFGNAT_OK;
    // few CTAs: the kernel waits on the bus, not on the SMs, and shares them with whatever else runs
    stage_inputs_kernel<<<48, kStageThreads, 0, st>>>(static_cast<const uint4 *>(hidden_src), static_cast<uint4 *>(hidden_dst),
                                                      row_bytes / 16, links_src, links_dst, ol, B, L);
    return cuda_rc(cudaGetLastError());
}

}  // namespace pcfgnat
