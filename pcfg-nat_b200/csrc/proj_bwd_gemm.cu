// The two matrix products that finish the backward of the output projection, on the tcgen05 tensor cores:
//     d rows   [n][H] = dlogits [n][V] . W [V][H]            (K = V)
//     d weight [V][H] = dlogits^T [V][n] . rows [n][H]       (K = n)
// with dlogits bf16 as proj_kernel's gradient mode writes it (compact: the n real graph nodes), W and the rows of
// the decoder states as bf16, float32 accumulation.  They stand in for autograd's two GEMMs of nn.Linear behind
// DagLogsoftmaxGatherFunc.backward (fs_plugins/custom_ops/pcfg_loss.py:168-180, models/...pcfg.py:237).
//
// One kernel, C [M][N] += A . B with either operand K-major ([rows][K] in memory) or MN-major ([K][rows]), so that
// neither product needs a transposed copy of the 0.9 GB dlogits: the first reads dlogits K-major and W MN-major,
// the second reads dlogits and the rows both MN-major.  Tiles of 256 x 256 per CTA in K steps of 32 (32 KB of
// operands per 4.2 MFLOP; a 128-row tile moves half as much again per FLOP), both operands brought in by TMA (this
// CTA only) through a ring of six 32 KB stages; warp 0 issues the loads, warp 1 two tcgen05.mma 128 x 256 x 16 per
// 16 K (rows 0-127 and 128-255 of the tile, each into its own 256-column accumulator: all 512 columns of tensor
// memory), eight warps drain the accumulators with tcgen05.ld and add them to C with float4 reductions.  The work is
// a list of (tile, K step) pairs cut into equal contiguous ranges, one per SM (a tile cut by a range boundary is
// summed up in C by the reductions), so every SM runs the same number of K steps whatever the shape; a range is
// hundreds of K steps long, so the one accumulator set (no second one to overlap the drain with) costs a few
// microseconds per range.  The SMs form one group per column tile, and the members of equal rank walk the same
// (row tile, K step) list side by side, so that dlogits comes from HBM once and from L2 for the other group.
// Every wait on an mbarrier is bounded; on expiry the CTA records PCFGNAT_STATUS_TIMEOUT, stops issuing work and
// still frees its tensor memory.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace pcfgnat {

namespace {

using namespace tc;

constexpr int GBM = 256, GBN = 256, GBK = 32, GUK = 16;
constexpr int G_HALF = 128;  // rows per tcgen05.mma (tensor-memory lanes)
constexpr int G_STAGES = 6;  // 32 KB each: three 64 KB stages (K = 64) left the tensor pipe waiting for loads
constexpr int G_A_BYTES = GBM * GBK * 2;  // 16 KB
constexpr int G_B_BYTES = GBN * GBK * 2;  // 16 KB
constexpr int G_STAGE_BYTES = G_A_BYTES + G_B_BYTES;
constexpr int G_BLOCK_BYTES = 64 * GBK * 2;  // an MN-major tile comes as blocks of 64 indices x 32 K: 4 KB each
constexpr int G_EPI_WARPS = 8;               // two per tensor-memory sub-partition
constexpr int G_THREADS = 32 * (2 + G_EPI_WARPS);
constexpr int G_TMEM_COLS = (GBM / G_HALF) * GBN;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(G_THREADS, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float *C, int M,
                     int N, int ldc, int k_steps, int m_tiles, int n_tiles, int groups, int *status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * G_STAGES + 2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_full = smem_u32(&bars[0]);                  // [G_STAGES] stage landed
    const uint32_t bar_empty = smem_u32(&bars[G_STAGES]);          // [G_STAGES] stage consumed
    const uint32_t bar_tfull = smem_u32(&bars[2 * G_STAGES]);      // accumulators ready
    const uint32_t bar_tempty = smem_u32(&bars[2 * G_STAGES + 1]); // accumulators drained
    volatile int *abort_flag = &abort_flag_s;
    if (threadIdx.x == 0) {
        for (int i = 0; i < G_STAGES; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, G_EPI_WARPS);
        abort_flag_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_base_slot), G_TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // This CTA's contiguous range of a list of (tile, K step) pairs; every role walks it segment by segment.
    // groups == n_tiles: the CTAs form one group per column tile, and the members of equal rank of all groups walk
    // the same (row tile, K step) list side by side, so that the A tiles one of them brings in from HBM are still in
    // L2 when the others ask for them (with one list over all tiles, the column tiles of a row tile ran hundreds
    // of K steps apart and A was read from HBM once per column tile).  groups == 1: one list, column tile fastest.
    const int per_group = gridDim.x / groups, group = blockIdx.x / per_group, member = blockIdx.x % per_group;
    const long long total = (long long)m_tiles * (groups == 1 ? n_tiles : 1) * k_steps;
    const long long beg = total * member / per_group, end = total * (member + 1) / per_group;
    auto tile_origin = [&](long long pos, int &m0, int &n0) {
        const int tile = (int)(pos / k_steps);
        m0 = (groups == 1 ? tile / n_tiles : tile) * GBM;
        n0 = (groups == 1 ? tile % n_tiles : group) * GBN;
    };
    constexpr uint32_t idesc = idesc_f16(G_HALF, GBN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        uint32_t st = 0, ph = 0;
        bool ok = true;
        for (long long pos = beg; pos < end && ok;) {
            const int ks0 = (int)(pos % k_steps);
            const int n = (int)min((long long)(k_steps - ks0), end - pos);
            int m0, n0;
            tile_origin(pos, m0, n0);
            for (int ks = ks0; ks < ks0 + n; ks++) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * st, ph ^ 1, abort_flag));
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t full = bar_full + 8 * st;
                    const uint32_t a_dst = smem_base + st * G_STAGE_BYTES, b_dst = a_dst + G_A_BYTES;
                    mbar_expect_tx(full, G_STAGE_BYTES);
                    if (A_MN) {
#pragma unroll
                        for (int j = 0; j < GBM / 64; j++) tma_load_2d(a_dst + j * G_BLOCK_BYTES, &map_a, full, m0 + 64 * j, ks * GBK);
                    } else {
                        tma_load_2d(a_dst, &map_a, full, ks * GBK, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < GBN / 64; j++) tma_load_2d(b_dst + j * G_BLOCK_BYTES, &map_b, full, n0 + 64 * j, ks * GBK);
                    } else {
                        tma_load_2d(b_dst, &map_b, full, ks * GBK, n0);
                    }
                }
                if (++st == G_STAGES) st = 0, ph ^= 1;
            }
            pos += n;
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        uint32_t st = 0, ph = 0, seg = 0;
        bool ok = true;
        for (long long pos = beg; pos < end && ok; seg++) {
            const int ks0 = (int)(pos % k_steps);
            const int n = (int)min((long long)(k_steps - ks0), end - pos);
            ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty, (seg & 1) ^ 1, abort_flag));
            if (!ok) break;
            fence_after();
            for (int ks = 0; ks < n; ks++) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * st, ph, abort_flag));
                if (!ok) break;
                fence_after();
                const uint32_t a_src = smem_base + st * G_STAGE_BYTES, b_src = a_src + G_A_BYTES;
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < GBK / GUK; k++) {
                        const uint64_t db = B_MN ? desc_mn_major(b_src + k * GUK * 128, G_BLOCK_BYTES) : desc_k_major_sw64(b_src) + 2 * k;
#pragma unroll
                        for (int h = 0; h < GBM / G_HALF; h++) {  // rows 128 h .. of the tile: 128 rows x 128 B, or two blocks
                            const uint32_t a_half = a_src + h * (G_HALF * GBK * 2);
                            const uint64_t da = A_MN ? desc_mn_major(a_half + k * GUK * 128, G_BLOCK_BYTES) : desc_k_major_sw64(a_half) + 2 * k;
                            umma_f16(tmem_base + h * GBN, da, db, idesc, (ks | k) != 0);
                        }
                    }
                    umma_commit(bar_empty + 8 * st);  // frees the stage when these MMAs have read it
                }
                if (++st == G_STAGES) st = 0, ph ^= 1;
            }
            if (ok && elect_one()) umma_commit(bar_tfull);
            pos += n;
        }
    } else {
        // ------------------------------ epilogue: one row and one 128-column half per thread ------------------
        const int ew = warp - 2;
        const int sub = warp & 3;  // tensor-memory sub-partition (lanes 32 * sub ..) this warp may read
        const int half = ew >> 2;  // which 128 columns of the 256-wide tile
        uint32_t seg = 0;
        bool ok = true;
        for (long long pos = beg; pos < end && ok; seg++) {
            const int ks0 = (int)(pos % k_steps);
            const int n = (int)min((long long)(k_steps - ks0), end - pos);
            int m0, n0;
            tile_origin(pos, m0, n0);
            if (!mbar_wait(bar_tfull, seg & 1, abort_flag)) break;
            fence_after();
#pragma unroll 1
            for (int h = 0; h < GBM / G_HALF; h++) {
                const int row = m0 + h * G_HALF + sub * 32 + lane;
                float *crow = C + (size_t)row * ldc;
#pragma unroll 1
                for (int c = 0; c < GBN / 2 / 32; c++) {
                    uint32_t r[32];
                    const int col0 = n0 + half * (GBN / 2) + c * 32;
                    tmem_ld32_issue(tmem_base + ((uint32_t)(sub * 32) << 16) + h * GBN + half * (GBN / 2) + c * 32, r);
                    tmem_ld_wait(r);
                    if (row < M) {
#pragma unroll
                        for (int q = 0; q < 8; q++)
                            if (col0 + 4 * q < N)  // N is a multiple of 4
                                atomicAdd(reinterpret_cast<float4 *>(crow + col0 + 4 * q),
                                          make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                      __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty);
            pos += n;
        }
    }
    if (*abort_flag && threadIdx.x == 0) flag(status, PCFGNAT_STATUS_TIMEOUT);
    fence_before();
    __syncthreads();
    if (warp == 0) {
        fence_after();
        tmem_dealloc(tmem_base, G_TMEM_COLS);
    }
}

// bf16 matrix [outer][inner] row-major with a row pitch of ld elements; tiles of box_outer rows x box_inner elements
// (64: 128-byte swizzle, 32: 64-byte swizzle), zeros outside.
bool gemm_map(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
              uint32_t box_outer) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// C [M][N] (float32, pitch N) += A . B.  A: [M][K] (a_mn = false) or [K][M]; B: [N][K] (b_mn = false) or [K][N];
// lda / ldb are their row pitches in elements.  Only the two operand layouts the projection backward needs exist.
int launch_gemm(const void *A, bool a_mn, int lda, const void *B, bool b_mn, int ldb, float *C, int M, int N, int K,
                int *status, cudaStream_t st) {
    if (M == 0 || N == 0 || K == 0) return PCFGNAT_OK;
    if (!b_mn) return PCFGNAT_ERR_UNSUPPORTED;
    CUtensorMap map_a, map_b;
    static_assert(GBK == 32, "K-major tiles are described with the 64-byte swizzle");
    const bool ok_a = a_mn ? gemm_map(&map_a, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, GBK)
                           : gemm_map(&map_a, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, GBK, GBM);  // 256 rows: the largest box
    const bool ok_b = gemm_map(&map_b, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, GBK);
    if (!ok_a || !ok_b) return PCFGNAT_ERR_CUDA;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int m_tiles = (M + GBM - 1) / GBM, n_tiles = (N + GBN - 1) / GBN, k_steps = (K + GBK - 1) / GBK;
    const long long total = (long long)m_tiles * n_tiles * k_steps;
    int grid = (int)(total < sms ? total : sms);
    int groups = 1;  // one group of CTAs per column tile where they divide evenly and every CTA still gets work
    if (n_tiles > 1 && grid >= n_tiles && (long long)m_tiles * k_steps >= grid / n_tiles) {
        groups = n_tiles;
        grid -= grid % n_tiles;
    }
    const size_t smem = (size_t)G_STAGES * G_STAGE_BYTES + 1024;
    if (a_mn) {
        auto k = gemm_bf16_kernel<true, true>;
        if (ensure_dynamic_smem(k, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        k<<<grid, G_THREADS, smem, st>>>(map_a, map_b, C, M, N, N, k_steps, m_tiles, n_tiles, groups, status);
    } else {
        auto k = gemm_bf16_kernel<false, true>;
        if (ensure_dynamic_smem(k, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        k<<<grid, G_THREADS, smem, st>>>(map_a, map_b, C, M, N, N, k_steps, m_tiles, n_tiles, groups, status);
    }
    return cuda_rc(cudaGetLastError());
}

}  // namespace

int launch_proj_backward_gemms(const void *dlogits, const void *weight_bf16, const void *rows_bf16, int n, int V, int H,
                               float *d_rows, float *d_weight, int *status, cudaStream_t st) {
    if (V % 8 || H % 8) return PCFGNAT_ERR_UNSUPPORTED;  // row pitches of 16-byte multiples for the tensor maps
    if ((reinterpret_cast<uintptr_t>(dlogits) | reinterpret_cast<uintptr_t>(weight_bf16) |
         reinterpret_cast<uintptr_t>(rows_bf16) | reinterpret_cast<uintptr_t>(d_rows) |
         reinterpret_cast<uintptr_t>(d_weight)) % 16)
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (d_rows) {
        if (cudaMemsetAsync(d_rows, 0, (size_t)n * H * sizeof(float), st) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        const int rc = launch_gemm(dlogits, false, V, weight_bf16, true, H, d_rows, n, H, V, status, st);
        if (rc != PCFGNAT_OK) return rc;
    }
    if (d_weight) {
        if (cudaMemsetAsync(d_weight, 0, (size_t)V * H * sizeof(float), st) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        const int rc = launch_gemm(dlogits, true, V, rows_bf16, true, H, d_weight, V, H, n, status, st);
        if (rc != PCFGNAT_OK) return rc;
    }
    return PCFGNAT_OK;
}

}  // namespace pcfgnat
