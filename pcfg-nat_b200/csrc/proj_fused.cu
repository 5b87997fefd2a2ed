// Fused output projection + log-softmax + target gather / row max (the only dense contraction
// of the path, so the only tensor-core kernel).
//
// Replaces, without ever writing the [rows, V] logits to HBM:
//   logits = output_projection(features)                (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:237)
//   match  = logsoftmax_gather(logits, targets)         (fs_plugins/custom_ops/logsoftmax_gather.cu:240-292)
//   lprob, token = logits.log_softmax(-1).max(-1)       (models/...pcfg.py:414-415)
//
// Shape of the kernel (sm_100a only: tcgen05 tensor cores, TMEM accumulators, TMA):
//   * rows are compacted first: when the graph lengths are known, only the rows of real nodes
//     (l < m_b) are projected; a small kernel builds the list of source rows.  Padded rows get
//     zeros in every output;
//   * the work is the grid of (128 compact rows) x (256-wide vocabulary tile) units, flattened
//     row-tile-major and cut into one contiguous range per CTA, one CTA per SM, so that every SM
//     gets the same number of units whatever the number of rows.  A range crosses at most a few
//     row tiles ("segments"); per segment the 128 x H fp16 state tile is gathered once into shared
//     memory (128-byte-swizzled, the layout TMA would produce; H <= 512: 128 KB) and stays resident
//     while the projection matrix streams through a 3-stage TMA ring of 256 x 64 fp16 tiles;
//   * warp 0 drives TMA (cp.async.bulk.tensor into this CTA only, 128-byte swizzle), warp 1 issues
//     tcgen05.mma 128x256x16 (fp16 in, fp32 accumulate) into one of two 256-column TMEM
//     accumulators, warps 2-9 load the state tile and are the epilogue: two warps per TMEM
//     sub-partition, each thread owns one row and one 128-column half of the tile, reads it with
//     tcgen05.ld and keeps an online (max, sum-exp), the running arg-max and the raw logits of this
//     row's targets, while the MMA warp already fills the other accumulator;
//   * a last, tiny kernel merges the per-segment partials: lse, match = logit - lse (with the
//     criterion's EOS masking fused if lengths are given), max log-prob and arg-max.
// Every wait on an mbarrier is bounded; on expiry the CTA records PCFGNAT_STATUS_TIMEOUT, stops
// issuing work, and still frees its tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace pcfgnat {

namespace {

using tc::elect_one;
using tc::kSpinLimit;
using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_u32;
using tc::tma_load_2d;
using tc::tmem_ld32_issue;
using tc::tmem_ld_wait;
using tc::umma_commit;

constexpr int BM = 128;        // rows per CTA (TMEM lanes)
constexpr int BN = 256;        // vocabulary columns per MMA tile (TMEM columns per accumulator)
constexpr int BK = 64;         // K elements per smem tile row: 64 fp16 = 128 B = one swizzle span
constexpr int UK = 16;         // K per tcgen05.mma for 16-bit inputs
constexpr int WK = 64;         // K extent of one W ring stage: 64 (128-byte swizzle) or 32 (64-byte swizzle; six
                               // 16 KB stages were measured slower, 0.40 vs 0.33 ms: the issuing warp's per-stage cost)
constexpr int NSTAGE = 3;      // W ring depth (one CTA per tile)
constexpr int NSTAGE_PAIR = 6; // W ring depth when two CTAs share each W tile: every CTA holds half of it per stage
constexpr int KC_MAX = 8;      // H <= 512
constexpr int A_CHUNK_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * WK * 2;  // 32 KB at WK = 64
constexpr int B_STAGE_BYTES_PAIR = B_STAGE_BYTES / 2;
constexpr int EPI_WARPS = 8;                // two per TMEM sub-partition
constexpr int PROJ_THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_BUF_COLS = 256;         // column pitch of the two accumulators (512 columns allocated)
constexpr int HALF_COLS = BN / 2;           // columns of a tile owned by one epilogue thread
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// tcgen05 instruction descriptor, kind::f16: D = F32 (bits 4-5 = 1), A = B = F16 (0), both K-major (0),
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
// the same for a CTA pair (cta_group::2): M = 256, 128 rows in each CTA's tensor memory
constexpr uint32_t kIdescPair = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);

struct Partial {  // per (CTA, segment, column half, row)
    float m, s, best;
    int best_idx;
};

// Flattened schedule: unit u = row_tile * n_tiles + vocab_tile; CTA g owns [begin(g), begin(g + 1)).
// Built on the device from the compact row count, so the host never needs to know it.
struct Plan {
    int n_tiles, ctas, max_seg;
    long long units, q, rem;  // the first `rem` CTAs own q + 1 units, the others q
    // pair: two CTAs share every unit, each with its own row tile, so a unit covers two row tiles
    __host__ __device__ static Plan make(int rows, int V, int ctas, int max_seg, bool pair = false) {
        Plan p;
        p.n_tiles = (V + BN - 1) / BN;
        p.ctas = ctas;
        p.max_seg = max_seg;
        const int row_tiles = (rows + BM - 1) / BM;
        p.units = (long long)(pair ? (row_tiles + 1) / 2 : row_tiles) * p.n_tiles;
        p.q = p.units / ctas;
        p.rem = p.units % ctas;
        return p;
    }
    __host__ __device__ long long begin(int g) const { return (long long)g * q + (g < rem ? g : rem); }
    __host__ __device__ int cta_of(long long u) const {
        const long long big = rem * (q + 1);
        return u < big ? (int)(u / (q + 1)) : (int)(rem + (u - big) / q);
    }
};

// ---- CTA pair (cluster of 2) variants: barriers that live in the pair's first CTA, loads that signal them ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded wait on a barrier that CTAs of the cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.b32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (it > 32) __nanosleep(128);
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// TMA load into this CTA's shared memory that reports its bytes to a barrier of the pair's first CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t cluster_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

// K-major, 128-byte-swizzled operand tile: rows at 128 B pitch, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) /* leading byte offset (unused with swizzle) */
           | (64ull << 32)                                   /* stride byte offset 1024 B >> 4 */
           | (1ull << 46)                                    /* descriptor version of sm_100 */
           | (2ull << 61);                                   /* SWIZZLE_128B */
}

// The W stage: 128-byte swizzle when its rows are 128 B (WK = 64), else 64-byte swizzle with 64 B rows
// (8-row groups 512 B apart).
__device__ __forceinline__ uint64_t umma_desc_w(uint32_t saddr) {
    if (WK == 64) return umma_desc(saddr);
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (32ull << 32) /* 512 B >> 4 */ | (1ull << 46) |
           (4ull << 61) /* SWIZZLE_64B */;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
// The pair's MMA: 256 x BN x 16, rows 0-127 from this CTA's state tile into its tensor memory, rows 128-255 from
// the second CTA's into that CTA's; each CTA supplies BN / 2 rows of the W tile at the same shared-memory offset.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(kIdescPair), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair when the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { tc::fence_before(); }
__device__ __forceinline__ void tc_fence_after() { tc::fence_after(); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------------------------------
// preparation: compact row list, target lists sorted by token id
// ---------------------------------------------------------------------------------------
// One block per sentence b.
//  * prefix[b] = compact index of its first row = sum of the lengths before it (every block reduces
//    the lengths itself, so no block waits for another); row_src[prefix[b] + l] = padded row b * L + l
//    for every real node (l < m_b; every l when no lengths are given); the last block also writes
//    prefix[B] and *n_rows.
//  * with targets: the sentence's target ids sorted ascending (stable rank sort) into stok, with
//    their original positions in sslot; ids outside [0, V) sort last as INT_MAX and raise a status bit.
__global__ void proj_prepare_kernel(const int64_t *__restrict__ ol, const int64_t *__restrict__ targets, int B, int L,
                                    int T, int V, int *prefix, int *row_src, int *n_rows, int *stok, int *sslot,
                                    int *status) {
    __shared__ int warp_sum[32];
    __shared__ int before_s;
    chain_begin();
    const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto length = [&](int i) {
        int m = ol ? (int)ol[i] : L;
        return m < 0 ? 0 : (m > L ? L : m);
    };
    int acc = 0;
    for (int i = threadIdx.x; i < b; i += blockDim.x) acc += length(i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) warp_sum[warp] = acc;
    __syncthreads();
    if (warp == 0) {
        int v = lane < (int)(blockDim.x >> 5) ? warp_sum[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) before_s = v;
    }
    __syncthreads();
    const int before = before_s, mine = length(b);
    if (threadIdx.x == 0) {
        if (ol && (ol[b] < 0 || ol[b] > L)) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
        prefix[b] = before;
        if (b == B - 1) {
            prefix[B] = before + mine;
            *n_rows = before + mine;
        }
    }
    for (int l = threadIdx.x; l < mine; l += blockDim.x) row_src[before + l] = b * L + l;
    if (!targets) return;
    const int64_t *tg = targets + (size_t)b * T;
    for (int s = threadIdx.x; s < T; s += blockDim.x) {
        int64_t key = tg[s];
        if (key < 0 || key >= V) {
            flag(status, PCFGNAT_STATUS_BAD_INDEX);
            key = INT_MAX;
        }
        int rank = 0;
        for (int j = 0; j < T; j++) {
            int64_t o = tg[j];
            if (o < 0 || o >= V) o = INT_MAX;
            rank += (o < key) || (o == key && j < s);
        }
        stok[(size_t)b * T + rank] = (int)key;
        sslot[(size_t)b * T + rank] = s;
    }
}

// ---------------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------------
// MODE: kForward / kForwardArgmax as described above; kGradLogits recomputes the logits tile the same way and,
// instead of reducing it, writes d loss / d logits = scatter_t(g[row][t] at target t) - softmax(row) * sum_t g[row][t]
// for every projected row as bf16 into dlogits [B*L][V] (rows in padded order), from the row's saved
// log-sum-exp and the gradient g of the emissions (entries the forward masked as EOS carry no gradient).
enum ProjMode { kForward = 0, kForwardArgmax = 1, kGradLogits = 2 };

struct GradArgs {  // kGradLogits only
    const float *lse;        // [B*L] from the forward
    const float *gmatch;     // [B*L][T] gradient of the emissions
    const int64_t *ol, *tl;  // lengths (EOS masking), or null
    __nv_bfloat16 *dlogits;  // [B*L][V], or [capacity][V] when compact
    int compact;             // rows in compact order (row i = the i-th real node of the batch) instead of padded order
    int capacity;            // compact: rows the buffer holds; a batch with more real nodes is flagged, not written
    int tma_store;           // compact and V % 8 == 0: tiles leave through shared memory and TMA stores (map_dl)
};

// PAIR: launched as clusters of two CTAs that share every W tile (tcgen05 cta_group::2).  A unit is then two
// row tiles (one per CTA) x one vocabulary tile; each CTA loads half of the W tile per stage, which halves the
// traffic per SM and lets the same shared memory hold a ring twice as deep; the first CTA issues the MMAs for both.
template <int MODE, bool PAIR>
__global__ void __launch_bounds__(PROJ_THREADS, 1)
    proj_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_dl,
                const __half *__restrict__ hidden,
                const int *__restrict__ row_src, const int *__restrict__ n_rows_ptr, int max_seg, int V, int KC, int L,
                int T, const int *__restrict__ stok, const int *__restrict__ sslot, float *match, Partial *partials,
                GradArgs ga, int *status) {
    constexpr bool WANT_ARGMAX = MODE == kForwardArgmax;
    extern __shared__ uint8_t smem_raw[];
    // the gradient mode gives 32 KB of the W ring to the staging buffers of its TMA stores
    constexpr bool GRAD = MODE == kGradLogits;
    constexpr int NST = PAIR ? (GRAD ? NSTAGE_PAIR - 2 : NSTAGE_PAIR) : (GRAD ? NSTAGE - 1 : NSTAGE);
    constexpr int STAGE_BYTES = PAIR ? B_STAGE_BYTES_PAIR : B_STAGE_BYTES;
    __shared__ __align__(8) uint64_t bars[2 * NST + 2 + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag_s;

    chain_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = blockIdx.x;  // owner of a partial slot
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;  // 0: the CTA that owns the pair's barriers and issues its MMAs
    const int sched = PAIR ? blockIdx.x / 2 : blockIdx.x;
    const int n_rows = *n_rows_ptr;
    const Plan plan = Plan::make(n_rows, V, PAIR ? gridDim.x / 2 : gridDim.x, max_seg, PAIR);
    const long long u_begin = plan.begin(sched), u_end = plan.begin(sched + 1);
    const int NT = plan.n_tiles;

    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_a = smem_u32(smem);
    const uint32_t smem_b = smem_a + KC_MAX * A_CHUNK_BYTES;
    const uint32_t smem_store = smem_b + NST * STAGE_BYTES;  // GRAD: two 2 KB buffers per epilogue warp
    // In a pair, `full`, `a` and `tempty` are used in the first CTA only (both CTAs report to them); `empty`,
    // `a_free` and `tfull` exist in both and are signalled in both by the first CTA's commits.
    const uint32_t bar_full = smem_u32(&bars[0]);              // [NST] W stage landed
    const uint32_t bar_empty = smem_u32(&bars[NST]);           // [NST] W stage consumed
    const uint32_t bar_a = smem_u32(&bars[2 * NST]);           // state tile(s) written (one arrival per CTA)
    const uint32_t bar_a_free = smem_u32(&bars[2 * NST + 1]);  // all MMAs of the segment have read it
    const uint32_t bar_tfull = smem_u32(&bars[2 * NST + 2]);   // [2] accumulator ready
    const uint32_t bar_tempty = smem_u32(&bars[2 * NST + 4]);  // [2] accumulator drained
    volatile int *abort_flag = &abort_flag_s;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NST; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        mbar_init(bar_a, PAIR ? 2 : 1);  // one arrival per CTA, after its loader threads have met
        mbar_init(bar_a_free, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, (PAIR ? 2 : 1) * EPI_WARPS);  // one arrival per epilogue warp
        }
        abort_flag_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                         "r"(2 * TMEM_BUF_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                         "r"(2 * TMEM_BUF_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    if (PAIR) cluster_sync_all();  // both CTAs' barriers are initialised before either reports to the other's
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // The two issuing warps run their loops with all 32 lanes (every lane waits on the barriers, the
    // outcome is made warp-uniform) and elect one lane for the asynchronous instructions, so that loop
    // state, descriptors and addresses stay warp-uniform values.
    if (warp == 0) {
        // ------------------------------ TMA producer: streams W, segment after segment ------------
        uint32_t st = 0, ph = 0;
        bool ok = true;
        int t = (int)(u_begin % NT);
        for (long long u = u_begin; u < u_end && ok; u++) {
            for (int kw = 0; kw < KC * (BK / WK); kw++) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * st, ph ^ 1, abort_flag));
                if (!ok) break;
                if (elect_one()) {
                    if (PAIR) {  // this CTA's half of the tile; the bytes of both halves are counted in the first CTA
                        if (rank == 0) mbar_expect_tx(bar_full + 8 * st, 2 * STAGE_BYTES);
                        tma_load_2d_pair(smem_b + st * STAGE_BYTES, &map_w, map_to_cta(bar_full + 8 * st, 0), kw * WK,
                                         t * BN + (int)rank * (BN / 2));
                    } else {
                        mbar_expect_tx(bar_full + 8 * st, STAGE_BYTES);
                        tma_load_2d(smem_b + st * STAGE_BYTES, &map_w, bar_full + 8 * st, kw * WK, t * BN);
                    }
                }
                if (++st == NST) st = 0, ph ^= 1;
            }
            if (++t == NT) t = 0;
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (of the pair: in its first CTA only) ------------------------
        uint32_t st = 0, ph = 0, seg = 0, tile = 0;
        bool ok = true;
        long long u = rank == 0 ? u_begin : u_end;
        while (u < u_end && ok) {
            const int rt = (int)(u / NT);
            const long long seg_end = min(u_end, (long long)(rt + 1) * NT);
            ok = __all_sync(0xffffffffu, PAIR ? mbar_wait_cluster(bar_a, seg & 1, abort_flag) : mbar_wait(bar_a, seg & 1, abort_flag));
            if (!ok) break;
            for (; u < seg_end && ok; u++, tile++) {
                const uint32_t buf = tile & 1, use = tile >> 1;
                ok = __all_sync(0xffffffffu, PAIR ? mbar_wait_cluster(bar_tempty + 8 * buf, (use & 1) ^ 1, abort_flag)
                                                  : mbar_wait(bar_tempty + 8 * buf, (use & 1) ^ 1, abort_flag));
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * TMEM_BUF_COLS;
                for (int kw = 0; kw < KC * (BK / WK); kw++) {
                    ok = __all_sync(0xffffffffu, PAIR ? mbar_wait_cluster(bar_full + 8 * st, ph, abort_flag)
                                                      : mbar_wait(bar_full + 8 * st, ph, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    // the state tile is in 64-wide chunks; this stage covers WK of them starting at kw * WK
                    const int kc = kw / (BK / WK), sub = kw % (BK / WK);
                    const uint64_t da = umma_desc(smem_a + kc * A_CHUNK_BYTES) + 2 * sub * (WK / UK);
                    const uint64_t db = umma_desc_w(smem_b + st * STAGE_BYTES);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < WK / UK; k++) {  // +32 B along K inside the swizzle span = +2 in the address field
                            if (PAIR) umma_f16_pair(d, da + 2 * k, db + 2 * k, (kw | k) != 0);
                            else umma_f16(d, da + 2 * k, db + 2 * k, (kw | k) != 0);
                        }
                        // frees the W stage (in both CTAs of a pair) when these MMAs have read it
                        if (PAIR) umma_commit_pair(bar_empty + 8 * st);
                        else umma_commit(bar_empty + 8 * st);
                    }
                    if (++st == NST) st = 0, ph ^= 1;
                }
                if (ok && elect_one()) {
                    if (PAIR) umma_commit_pair(bar_tfull + 8 * buf);
                    else umma_commit(bar_tfull + 8 * buf);
                }
            }
            if (ok && elect_one()) {
                if (PAIR) umma_commit_pair(bar_a_free);
                else umma_commit(bar_a_free);
            }
            seg++;
        }
    } else {
        // -------- state-tile loader + epilogue: one row and one 128-column half per thread --------
        const int ew = warp - 2;
        const int et = ew * 32 + lane;  // 0 .. 255
        const int sub = warp & 3;       // TMEM sub-partition (lanes 32*sub ..) this warp may read
        const int half = ew >> 2;       // which 128 columns of each 256-wide tile
        uint32_t tile = 0, seg = 0;
        uint32_t store_buf = 0;  // GRAD: which of the warp's two staging buffers the next TMA store uses
        bool ok = true;
        long long u = u_begin;
        while (u < u_end && ok) {
            const int ut = (int)(u / NT);  // row tile (or pair of row tiles) of this segment
            const int rt = PAIR ? 2 * ut + (int)rank : ut;
            const long long seg_end = min(u_end, (long long)(ut + 1) * NT);
            // ---- gather the 128 x H state tile into the swizzled layout tcgen05.mma reads ----
            if (seg > 0 && !mbar_wait(bar_a_free, (seg - 1) & 1, abort_flag)) break;
            {
                const int chunks_per_row = KC * 8;  // 16-byte chunks
                const int total = BM * chunks_per_row;
                constexpr int STEP = EPI_WARPS * 32, DEPTH = 8;  // DEPTH independent loads in flight per thread
                for (int q0 = et; q0 < total; q0 += STEP * DEPTH) {
                    int src[DEPTH];
                    uint4 val[DEPTH];
#pragma unroll
                    for (int j = 0; j < DEPTH; j++) {
                        const int q = q0 + j * STEP, cr = rt * BM + q / chunks_per_row;
                        src[j] = (q < total && cr < n_rows) ? __ldg(row_src + cr) : -1;
                    }
#pragma unroll
                    for (int j = 0; j < DEPTH; j++) {
                        const int q = q0 + j * STEP, cc = q % chunks_per_row;
                        val[j] = make_uint4(0u, 0u, 0u, 0u);
                        if (src[j] >= 0)
                            val[j] = __ldg(reinterpret_cast<const uint4 *>(hidden + (size_t)src[j] * (KC * BK)) + cc);
                    }
#pragma unroll
                    for (int j = 0; j < DEPTH; j++) {
                        const int q = q0 + j * STEP;
                        if (q < total) {
                            const int r = q / chunks_per_row, cc = q - r * chunks_per_row;
                            const int kc = cc >> 3, c = cc & 7;
                            uint8_t *dst =
                                smem + kc * A_CHUNK_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4);
                            *reinterpret_cast<uint4 *>(dst) = val[j];
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
                asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");  // the loader threads of this CTA
                if (et == 0) {
                    if (PAIR) mbar_arrive_cluster(map_to_cta(bar_a, 0));
                    else mbar_arrive(bar_a);
                }
            }
            const int cr = rt * BM + sub * 32 + lane;
            const bool row_ok = cr < n_rows;
            const int row = row_ok ? __ldg(row_src + cr) : 0;  // padded row index b * L + l
            const int sent = row / L;
            const int *my_tok = stok ? stok + (size_t)sent * T : nullptr;
            const int *my_slot = stok ? sslot + (size_t)sent * T : nullptr;
            float *my_out = match ? match + (size_t)row * T : nullptr;
            int p = 0;
            if (my_tok) {  // first target at or after this segment's first column
                const int c_first = (int)(u - (long long)ut * NT) * BN;
                int lo = 0, hi = T;
                while (lo < hi) {
                    int mid = (lo + hi) >> 1;
                    if (__ldg(my_tok + mid) < c_first) lo = mid + 1; else hi = mid;
                }
                p = lo;
            }
            int next_tok = (my_tok && p < T) ? __ldg(my_tok + p) : INT_MAX;  // next target of this row's sentence
            float m = -CUDART_INF_F, s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            float best = -CUDART_INF_F;
            int best_idx = 0;
            // kGradLogits: this row's log-sum-exp, the sum of its emission gradients, and which target slot the
            // forward masked (the EOS column of every node but the last, criterions/nat_pcfg_loss.py:112-115)
            float row_nlse = 0.f, row_gsum = 0.f;
            int masked_slot = -1;
            const float *my_g = nullptr;
            if (MODE == kGradLogits && row_ok) {
                row_nlse = -ga.lse[row] * kLog2e;
                my_g = ga.gmatch + (size_t)row * T;
                if (ga.ol && ga.tl && row - sent * L != (int)ga.ol[sent] - 1) masked_slot = (int)ga.tl[sent] - 1;
                for (int q = 0; q < T; q++) {
                    if (__ldg(my_tok + q) == INT_MAX) break;  // ids out of range sort last: never gathered, no gradient
                    const int slot = __ldg(my_slot + q);
                    if (slot != masked_slot) row_gsum += my_g[slot];
                }
            }
            for (; u < seg_end && ok; u++, tile++) {
                const uint32_t buf = tile & 1, use = tile >> 1;
                if (!mbar_wait(bar_tfull + 8 * buf, use & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const int tile_col0 = (int)(u - (long long)ut * NT) * BN + half * HALF_COLS;
                const uint32_t tsrc = tmem_base + ((uint32_t)(sub * 32) << 16) + buf * TMEM_BUF_COLS + half * HALF_COLS;
                // One 32-column chunk of this thread's row: online max / sum-exp, arg-max, target logits.
                auto process = [&](const uint32_t *r, const int col0) {
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
                    if (col0 + 32 > V) {
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (col0 + i >= V) v[i] = -CUDART_INF_F;
                    }
                    if (MODE == kGradLogits) {
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = -row_gsum * ex2(fmaf(v[i], kLog2e, row_nlse));
                        while (next_tok < col0 + 32) {
                            const int idx = next_tok - col0;
                            if (idx >= 0 && row_ok) {
                                const int slot = __ldg(my_slot + p);
                                const float g = slot == masked_slot ? 0.f : my_g[slot];
#pragma unroll
                                for (int i = 0; i < 32; i++) v[i] += (idx == i) ? g : 0.f;
                            }
                            p++;
                            next_tok = p < T ? __ldg(my_tok + p) : INT_MAX;
                        }
                        if (ga.tma_store) {
                            // the warp's 32 rows x 32 columns as bf16 into its staging buffer (rows of 64 B in the
                            // 64-byte swizzle: no bank conflicts), then one TMA store: whole 64-byte row segments
                            // instead of 32 scattered 16-byte stores per instruction.  Rows past the batch's real
                            // nodes hold zeros here and the store clips at the buffer's rows and at column V.
                            uint32_t pk[16];
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                const __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                                pk[i] = *reinterpret_cast<const uint32_t *>(&two);
                            }
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");  // this buffer's last store has read it
                            __syncwarp();
                            const uint32_t sbuf = smem_store + (uint32_t)ew * 4096u + store_buf * 2048u;
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sbuf + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4)),
                                             "r"(pk[4 * i]), "r"(pk[4 * i + 1]), "r"(pk[4 * i + 2]), "r"(pk[4 * i + 3])
                                             : "memory");
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if (lane == 0) {
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                                 reinterpret_cast<uint64_t>(&map_dl)),
                                             "r"(sbuf), "r"(col0), "r"(cr - lane)
                                             : "memory");
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            }
                            store_buf ^= 1u;
                        } else if (row_ok && (!ga.compact || cr < ga.capacity)) {
                            __nv_bfloat16 *dst = ga.dlogits + (size_t)(ga.compact ? cr : row) * V + col0;
                            if (col0 + 32 <= V && (V & 7) == 0) {
                                uint32_t pk[16];
#pragma unroll
                                for (int i = 0; i < 16; i++) {
                                    const __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                                    pk[i] = *reinterpret_cast<const uint32_t *>(&two);
                                }
#pragma unroll
                                for (int i = 0; i < 4; i++)
                                    reinterpret_cast<uint4 *>(dst)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; i++)
                                    if (col0 + i < V) dst[i] = __float2bfloat16_rn(v[i]);
                            }
                        }
                        return;
                    }
                    float w16[16];  // tree max
#pragma unroll
                    for (int i = 0; i < 16; i++) w16[i] = fmaxf(v[i], v[i + 16]);
#pragma unroll
                    for (int i = 0; i < 8; i++) w16[i] = fmaxf(w16[i], w16[i + 8]);
#pragma unroll
                    for (int i = 0; i < 4; i++) w16[i] = fmaxf(w16[i], w16[i + 4]);
                    const float cmax = fmaxf(fmaxf(w16[0], w16[2]), fmaxf(w16[1], w16[3]));
                    if (cmax > m) {
                        const float f = ex2((m - cmax) * kLog2e);  // 0 on the first chunk (m = -inf)
                        s0 *= f, s1 *= f, s2 *= f, s3 *= f;
                        m = cmax;
                    }
                    if (WANT_ARGMAX && cmax > best) {
                        best = cmax;
                        int idx = 31;
#pragma unroll
                        for (int i = 30; i >= 0; i--) idx = (v[i] == cmax) ? i : idx;
                        best_idx = col0 + idx;
                    }
                    if (m > -CUDART_INF_F) {
                        const float nm = -m * kLog2e;
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            s0 += ex2(fmaf(v[i], kLog2e, nm));
                            s1 += ex2(fmaf(v[i + 1], kLog2e, nm));
                            s2 += ex2(fmaf(v[i + 2], kLog2e, nm));
                            s3 += ex2(fmaf(v[i + 3], kLog2e, nm));
                        }
                    }
                    while (next_tok < col0 + 32) {  // targets are sorted; those below col0 belong to the other half
                        const int idx = next_tok - col0;
                        if (idx >= 0 && row_ok) {
                            float val = v[0];
#pragma unroll
                            for (int i = 1; i < 32; i++) val = (idx == i) ? v[i] : val;
                            my_out[__ldg(my_slot + p)] = val;  // raw logit; the merge kernel subtracts lse
                        }
                        p++;
                        next_tok = p < T ? __ldg(my_tok + p) : INT_MAX;
                    }
                };
                // the load of chunk c+1 is in flight while chunk c is processed
                uint32_t regs[2][32];
                __syncwarp();  // the target loop may leave the lanes diverged; tcgen05.ld is warp-collective
                tmem_ld32_issue(tsrc, regs[0]);
                tmem_ld_wait(regs[0]);
#pragma unroll
                for (int c = 0; c < HALF_COLS / 32; c++) {
                    if (c + 1 < HALF_COLS / 32) {
                        __syncwarp();
                        tmem_ld32_issue(tsrc + (c + 1) * 32, regs[(c + 1) & 1]);
                    }
                    process(regs[c & 1], tile_col0 + c * 32);
                    if (c + 1 < HALF_COLS / 32) tmem_ld_wait(regs[(c + 1) & 1]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * buf, 0));
                    else mbar_arrive(bar_tempty + 8 * buf);
                }
            }
            if (ok && MODE != kGradLogits) {
                Partial pr;
                pr.m = m;
                pr.s = (s0 + s1) + (s2 + s3);
                pr.best = best;
                pr.best_idx = best_idx;
                partials[(((size_t)g * max_seg + seg) * 2 + half) * BM + sub * 32 + lane] = pr;
            }
            seg++;
        }
        // the staging buffers are read by stores still in flight: they are done before the CTA gives up its memory
        if (GRAD && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    if (*abort_flag && threadIdx.x == 0) flag(status, PCFGNAT_STATUS_TIMEOUT);
    tc_fence_before();
    if (PAIR) cluster_sync_all();  // neither CTA frees tensor memory the pair's MMAs may still write
    else __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TMEM_BUF_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TMEM_BUF_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// merge of the per-segment partials.  Blocks [0, 8 * row_tiles) take 16 rows of one tile of 128 compact
// rows each (the schedule is looked up once per block, one warp per row); the B blocks after them fill
// the padding rows of one sentence each.
// ---------------------------------------------------------------------------------------
constexpr int kMergeSplit = 8, kMergeThreads = 32 * (BM / kMergeSplit);
__global__ void proj_merge_kernel(const Partial *__restrict__ partials, const int *__restrict__ prefix,
                                  const int *__restrict__ row_src, const int *__restrict__ n_rows_ptr, int ctas,
                                  int max_seg, int row_tiles, int pair, int V, int L, int T, const int64_t *__restrict__ ol,
                                  const int64_t *__restrict__ tl, const int64_t *__restrict__ targets, float *match,
                                  float *max_lprob, int64_t *argmax, float *lse_out) {
    chain_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    if ((int)blockIdx.x >= kMergeSplit * row_tiles) {  // padding rows of sentence b: not projected
        const int b = blockIdx.x - kMergeSplit * row_tiles;
        const int len_b = prefix[b + 1] - prefix[b];
        for (int l = len_b + warp; l < L; l += n_warps) {
            const int row = b * L + l;
            if (lane == 0) {
                if (lse_out) lse_out[row] = 0.f;
                if (max_lprob) max_lprob[row] = 0.f;
                if (argmax) argmax[row] = 0;
            }
            if (match)
                for (int t = lane; t < T; t += 32) {
                    const int64_t tok = targets[(size_t)b * T + t];
                    match[(size_t)row * T + t] = (tok < 0 || tok >= V) ? CUDART_NAN_F : 0.f;
                }
        }
        return;
    }
    const int rt = blockIdx.x / kMergeSplit, part = blockIdx.x % kMergeSplit, n_rows = *n_rows_ptr;
    if (rt * BM + part * (BM / kMergeSplit) >= n_rows) return;
    __shared__ int s_glo, s_ghi, s_seg_lo;
    if (threadIdx.x == 0) {
        // `ctas` counts schedule owners: CTAs, or CTA pairs (then a unit is two row tiles and the partials of
        // row tile rt are in CTA 2 * owner + (rt & 1))
        const Plan plan = Plan::make(n_rows, V, ctas, max_seg, pair != 0);
        const int ut = pair ? rt >> 1 : rt;
        const long long u0 = (long long)ut * plan.n_tiles, u1 = u0 + plan.n_tiles - 1;
        s_glo = plan.cta_of(u0);
        s_ghi = plan.cta_of(u1);
        // only the first owner of the tile can have begun in an earlier row tile; the others start inside
        // this one, where it is their segment 0
        s_seg_lo = ut - (int)(plan.begin(s_glo) / plan.n_tiles);
    }
    __syncthreads();
    const int g_lo = s_glo, seg_lo = s_seg_lo, n_part = (s_ghi - g_lo + 1) * 2;
    for (int r_in = part * (BM / kMergeSplit) + warp; r_in < (part + 1) * (BM / kMergeSplit); r_in += n_warps) {
        const int cr = rt * BM + r_in;
        if (cr >= n_rows) break;
        const int row = row_src[cr], b = row / L, l = row - b * L;
        // lane i merges partials i, i + 32, ...; then the lanes are combined
        float m = -CUDART_INF_F, s = 0.f, best = -CUDART_INF_F;
        int best_idx = INT_MAX;
        for (int i = lane; i < n_part; i += 32) {
            const int owner = g_lo + (i >> 1), h = i & 1, seg = (i >> 1) == 0 ? seg_lo : 0;
            const int g = pair ? 2 * owner + (rt & 1) : owner;
            const Partial p = partials[(((size_t)g * max_seg + seg) * 2 + h) * BM + r_in];
            if (p.s > 0.f) {  // then p.m is finite
                const float nm = fmaxf(m, p.m);
                s = (s > 0.f ? s * exp2f((m - nm) * kLog2e) : 0.f) + p.s * exp2f((p.m - nm) * kLog2e);
                m = nm;
            }
            // first maximum in column order: equal values are resolved by the recorded column
            if (p.best > best || (p.best == best && p.best_idx < best_idx)) {
                best = p.best;
                best_idx = p.best_idx;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
            const float nm = fmaxf(m, om);
            s = (s > 0.f ? s * exp2f((m - nm) * kLog2e) : 0.f) + (os > 0.f ? os * exp2f((om - nm) * kLog2e) : 0.f);
            m = nm;
            if (ob > best || (ob == best && oi < best_idx)) {
                best = ob;
                best_idx = oi;
            }
        }
        if (best_idx == INT_MAX) best_idx = 0;
        const float lse = m + log2f(s) * kLn2;
        if (lane == 0) {
            if (lse_out) lse_out[row] = lse;
            if (max_lprob) max_lprob[row] = best - lse;
            if (argmax) argmax[row] = best_idx;
        }
        if (match) {
            int eos_col = -1;
            bool keep_eos = true;
            if (ol && tl) {  // criterion's EOS masking (criterions/nat_pcfg_loss.py:112-115)
                eos_col = (int)tl[b] - 1;
                keep_eos = l == (int)ol[b] - 1;
            }
            float *out = match + (size_t)row * T;
            for (int t = lane; t < T; t += 32) {
                const int64_t tok = targets[(size_t)b * T + t];
                float v = out[t] - lse;
                if (t == eos_col && !keep_eos) v = -CUDART_INF_F;
                if (tok < 0 || tok >= V) v = CUDART_NAN_F;  // never gathered
                out[t] = v;
            }
        }
    }
}

// [rows][K] fp16 row-major, box = 64 (K) x box_rows, 128-byte swizzle, out-of-bounds reads give zeros.
bool make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    tc::EncodeTiledFn fn = tc::encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K * 2};
    cuuint32_t box[2] = {WK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, WK == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// d-logits [rows][V] bf16 row-major for the gradient mode's stores: boxes of 32 rows x 32 columns (64 B per row,
// 64-byte swizzle in shared memory); a store clips at the tensor's bounds.
bool make_store_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t V) {
    tc::EncodeTiledFn fn = tc::encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {V, rows};
    cuuint64_t strides[1] = {V * 2};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Launch geometry from the PADDED row count (an upper bound of the compact one, which only the
// device knows): number of CTAs and the most segments a CTA's range can touch.
struct Geometry {
    int ctas, max_seg;
    bool pair;   // CTA pairs (clusters of 2) share every W tile
    int owners;  // schedule owners: ctas, or ctas / 2 pairs
};

// PCFGNAT_PROJ_PAIR=1 selects CTA pairs (A/B runs and tests).  Measured on 10 804 rows x 40 000 x 512: 0.347 ms
// per call with pairs against 0.325 ms with single CTAs, so single CTAs are the default: the deeper ring and
// the halved L2 traffic of a pair do not pay for its cross-CTA barrier hops.
bool want_pairs(int row_tiles) {
    (void)row_tiles;
    if (const char *v = getenv("PCFGNAT_PROJ_PAIR")) return v[0] == '1';
    return false;
}

Geometry make_geometry(int N, int V) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 148;
    const int n_tiles = (V + BN - 1) / BN;
    const int row_tiles = (N + BM - 1) / BM;
    Geometry g;
    g.pair = want_pairs(row_tiles) && sms >= 2;
    const long long units = (long long)(g.pair ? (row_tiles + 1) / 2 : row_tiles) * n_tiles;
    const int slots = g.pair ? sms / 2 : sms;
    g.owners = (int)(units < slots ? units : slots);
    g.ctas = g.pair ? 2 * g.owners : g.owners;
    const long long per_owner = (units + g.owners - 1) / g.owners;
    g.max_seg = (int)((per_owner + n_tiles - 1) / n_tiles) + 1;
    return g;
}

// Launches proj_kernel<MODE, PAIR>: plain launch, or clusters of two CTAs.
template <int MODE>
int launch_proj_kernel(const Geometry &geo, size_t smem, cudaStream_t st, const CUtensorMap &map_w,
                       const CUtensorMap &map_dl, const __half *hidden,
                       const int *row_src, const int *n_rows, int V, int KC, int L, int T, const int *stok,
                       const int *sslot, float *match, Partial *partials, GradArgs ga, int *status) {
    if (!geo.pair) {
        auto k = proj_kernel<MODE, false>;
        if (ensure_dynamic_smem(k, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
        return cuda_rc(launch_chain(k, dim3(geo.ctas), dim3(PROJ_THREADS), smem, st, map_w, map_dl, hidden, row_src, n_rows,
                                    geo.max_seg, V, KC, L, T, stok, sslot, match, partials, ga, status));
    }
    auto k = proj_kernel<MODE, true>;
    if (ensure_dynamic_smem(k, smem) != cudaSuccess) return PCFGNAT_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)geo.ctas);
    cfg.blockDim = dim3(PROJ_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_rc(cudaLaunchKernelEx(&cfg, k, map_w, map_dl, hidden, row_src, n_rows, geo.max_seg, V, KC, L, T, stok, sslot,
                                      match, partials, ga, status));
}

struct Workspace {
    int *stok, *sslot, *prefix, *row_src, *n_rows;
    Partial *partials;
    size_t bytes;
};

Workspace carve(void *base, int B, int L, int T, int V) {
    const int N = B * L;
    const Geometry g = make_geometry(N > 0 ? N : 1, V > 0 ? V : 1);
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    char *p = static_cast<char *>(base);
    size_t off = 0;
    Workspace w;
    w.stok = reinterpret_cast<int *>(p + off);
    off += up((size_t)B * (T > 0 ? T : 0) * sizeof(int));
    w.sslot = reinterpret_cast<int *>(p + off);
    off += up((size_t)B * (T > 0 ? T : 0) * sizeof(int));
    w.prefix = reinterpret_cast<int *>(p + off);
    off += up((size_t)(B + 1) * sizeof(int));
    w.row_src = reinterpret_cast<int *>(p + off);
    off += up((size_t)N * sizeof(int));
    w.n_rows = reinterpret_cast<int *>(p + off);
    off += 256;
    w.partials = reinterpret_cast<Partial *>(p + off);
    off += up((size_t)g.ctas * g.max_seg * 2 * BM * sizeof(Partial));
    w.bytes = off;
    return w;
}

}  // namespace

size_t proj_workspace_bytes(int B, int L, int T, int V) { return carve(nullptr, B, L, T, V).bytes; }

int launch_proj(const void *hidden, const void *weight, const int64_t *targets, const int64_t *ol, const int64_t *tl,
                int B, int L, int T, int V, int H, float *match, float *max_lprob, int64_t *argmax, float *lse,
                void *workspace, size_t ws_bytes, int *status, cudaStream_t st) {
    const int N = B * L;
    if (N == 0) return PCFGNAT_OK;
    if (H % BK != 0 || H > KC_MAX * BK) return PCFGNAT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(weight)) % 16) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (ws_bytes < proj_workspace_bytes(B, L, T, V) || reinterpret_cast<uintptr_t>(workspace) % 16)
        return PCFGNAT_ERR_WORKSPACE;
    const bool gather = match != nullptr && targets != nullptr && T > 0;
    const Geometry geo = make_geometry(N, V);
    const Workspace w = carve(workspace, B, L, T, V);

    CUtensorMap map_w;
    if (!make_map(&map_w, weight, (uint64_t)V, (uint64_t)H, geo.pair ? BN / 2 : BN)) return PCFGNAT_ERR_CUDA;
    if (launch_chain(proj_prepare_kernel, dim3(B), dim3(128), 0, st, ol, gather ? targets : nullptr, B, L, T, V, w.prefix,
                     w.row_src, w.n_rows, w.stok, w.sslot, status) != cudaSuccess)
        return PCFGNAT_ERR_CUDA;
    const size_t smem = (size_t)KC_MAX * A_CHUNK_BYTES + (size_t)NSTAGE * B_STAGE_BYTES + 1024;
    const bool want_arg = max_lprob != nullptr || argmax != nullptr;
    const __half *hid = static_cast<const __half *>(hidden);
    const GradArgs none = {nullptr, nullptr, nullptr, nullptr, nullptr};
    const int rc = want_arg ? launch_proj_kernel<kForwardArgmax>(geo, smem, st, map_w, map_w, hid, w.row_src, w.n_rows, V, H / BK, L, T,
                                                                 gather ? w.stok : nullptr, gather ? w.sslot : nullptr,
                                                                 gather ? match : nullptr, w.partials, none, status)
                            : launch_proj_kernel<kForward>(geo, smem, st, map_w, map_w, hid, w.row_src, w.n_rows, V, H / BK, L, T,
                                                           gather ? w.stok : nullptr, gather ? w.sslot : nullptr,
                                                           gather ? match : nullptr, w.partials, none, status);
    if (rc != PCFGNAT_OK) return rc;
    const int row_tiles = (N + BM - 1) / BM;
    return cuda_rc(launch_chain(proj_merge_kernel, dim3(kMergeSplit * row_tiles + B), dim3(kMergeThreads), 0, st,
                                (const Partial *)w.partials, (const int *)w.prefix, (const int *)w.row_src,
                                (const int *)w.n_rows, geo.owners, geo.max_seg, row_tiles, geo.pair ? 1 : 0, V, L, T, ol, tl,
                                targets, gather ? match : nullptr, max_lprob, argmax, lse));
}

// Rows of padding (l >= m_b) are not projected: their gradient rows are zero.
__global__ void proj_zero_padding_rows_kernel(const int *__restrict__ prefix, int L, int V, __nv_bfloat16 *dlogits) {
    const int b = blockIdx.x;
    const int len_b = prefix[b + 1] - prefix[b];
    for (int l = len_b + blockIdx.y; l < L; l += gridDim.y) {
        __nv_bfloat16 *row = dlogits + ((size_t)b * L + l) * V;
        if ((V & 7) == 0) {
            for (int i = threadIdx.x; i < V / 8; i += blockDim.x) reinterpret_cast<uint4 *>(row)[i] = make_uint4(0u, 0u, 0u, 0u);
        } else {
            for (int i = threadIdx.x; i < V; i += blockDim.x) row[i] = __float2bfloat16_rn(0.f);
        }
    }
}

// Compact order: the padded index b * L + l of every compact row for the caller's gather / scatter of the states and
// their gradient, zero beyond the batch's real nodes; a batch with more real nodes than the buffer holds is flagged.
__global__ void proj_row_index_kernel(const int *__restrict__ row_src, const int *__restrict__ n_rows, int capacity,
                                      int64_t *row_index, int *n_rows_out, int *status) {
    const int n = *n_rows;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < capacity; i += gridDim.x * blockDim.x)
        row_index[i] = i < n ? row_src[i] : 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (n_rows_out) *n_rows_out = n;
        if (n > capacity) flag(status, PCFGNAT_STATUS_BAD_LENGTH);
    }
}

int launch_proj_dlogits(const void *hidden, const void *weight, const int64_t *targets, const int64_t *ol,
                        const int64_t *tl, const float *lse, const float *grad_match, int B, int L, int T, int V, int H,
                        void *dlogits, void *workspace, size_t ws_bytes, int *status, cudaStream_t st, int capacity,
                        int64_t *row_index, int *n_rows_out) {
    const int N = B * L;
    if (N == 0) return PCFGNAT_OK;
    if (H % BK != 0 || H > KC_MAX * BK) return PCFGNAT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(dlogits)) % 16)
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (ws_bytes < proj_workspace_bytes(B, L, T, V) || reinterpret_cast<uintptr_t>(workspace) % 16)
        return PCFGNAT_ERR_WORKSPACE;
    const Geometry geo = make_geometry(N, V);
    const Workspace w = carve(workspace, B, L, T, V);
    CUtensorMap map_w;
    if (!make_map(&map_w, weight, (uint64_t)V, (uint64_t)H, geo.pair ? BN / 2 : BN)) return PCFGNAT_ERR_CUDA;
    if (launch_chain(proj_prepare_kernel, dim3(B), dim3(128), 0, st, ol, targets, B, L, T, V, w.prefix, w.row_src, w.n_rows,
                     w.stok, w.sslot, status) != cudaSuccess)
        return PCFGNAT_ERR_CUDA;
    __nv_bfloat16 *dl = static_cast<__nv_bfloat16 *>(dlogits);
    const int compact = row_index != nullptr;
    if (compact)
        proj_row_index_kernel<<<(capacity + 1023) / 1024 > 0 ? (capacity + 1023) / 1024 : 1, 1024, 0, st>>>(
            w.row_src, w.n_rows, capacity, row_index, n_rows_out, status);
    else if (ol)
        proj_zero_padding_rows_kernel<<<dim3(B, 8), 256, 0, st>>>(w.prefix, L, V, dl);
    const size_t smem = (size_t)KC_MAX * A_CHUNK_BYTES + (size_t)NSTAGE * B_STAGE_BYTES + 1024;
    // compact rows are consecutive in the buffer, so a warp's 32 rows x 32 columns can leave as one TMA store
    CUtensorMap map_dl = map_w;
    const int tma_store = compact && capacity > 0 && V % 8 == 0 && make_store_map(&map_dl, dl, (uint64_t)capacity, (uint64_t)V);
    const GradArgs ga = {lse, grad_match, ol, tl, dl, compact, capacity, tma_store};
    return launch_proj_kernel<kGradLogits>(geo, smem, st, map_w, map_dl, static_cast<const __half *>(hidden), w.row_src,
                                           w.n_rows, V, H / BK, L, T, w.stok, w.sslot, nullptr, w.partials, ga, status);
}

}  // namespace pcfgnat
