// log-softmax over the vocabulary + gather of selected columns (+ optional in-place
// softmax for the backward).
//
// Replaces logsoftmax_gather_kernel of the reference
// (fs_plugins/custom_ops/logsoftmax_gather.cu:240-292), which sweeps each row three times
// from global memory (max, sum-exp, softmax write).  Here one CTA owns one row at a time and
// keeps it resident in shared memory in its storage type (fp16 rows of 40 000 entries are
// 80 KB, so two CTAs fit per SM): one HBM read, and one HBM write only when the softmax is
// asked for.  Rows that do not fit fall back to re-reading global memory.
//
// Rows that are 16-byte multiples and fit shared memory run on the streaming kernel further below (bulk
// asynchronous copies in chunks, sum of exponentials accumulated as the chunks land); the kernel here remains for
// the other rows.
// Like the reference this kernel uses the fast exp/log/divide intrinsics
// (logsoftmax_gather.cu:107-148), so parity with it is by tolerance.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"

namespace pcfgnat {

namespace {

constexpr int kLsgThreads = 512;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half(v); }

__device__ __forceinline__ float block_reduce(float v, bool is_max, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, w) : v + w;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // red[] may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = is_max ? -CUDART_INF_F : 0.f;
    for (int w = 0; w < kLsgThreads / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

template <typename T, bool STAGE>
__global__ void __launch_bounds__(kLsgThreads)
    logsoftmax_gather_kernel(T *logits, const int64_t *__restrict__ sel, int64_t sb, int64_t sl, int64_t ss,
                             int64_t rows, int64_t rpb, int V, int slen, int req_grad, float *selected, int *status,
                             int vec_ok) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float red[kLsgThreads / 32];
    T *srow = reinterpret_cast<T *>(smem_raw);
    const int tid = threadIdx.x;
    constexpr int kVec = 16 / sizeof(T);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        T *grow = logits + (size_t)r * V;
        const T *row = STAGE ? srow : grow;
        float mx = -CUDART_INF_F;
        if (STAGE) {
            if (vec_ok) {
                const uint4 *g4 = reinterpret_cast<const uint4 *>(grow);
                uint4 *s4 = reinterpret_cast<uint4 *>(srow);
                for (int i = tid; i < V / kVec; i += kLsgThreads) {
                    uint4 v = g4[i];
                    s4[i] = v;
                    const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
                    for (int k = 0; k < kVec; k++) mx = fmaxf(mx, to_f<T>(e[k]));
                }
            } else {
                for (int i = tid; i < V; i += kLsgThreads) {
                    T v = grow[i];
                    srow[i] = v;
                    mx = fmaxf(mx, to_f<T>(v));
                }
            }
        } else {
            for (int i = tid; i < V; i += kLsgThreads) mx = fmaxf(mx, to_f<T>(grow[i]));
        }
        mx = block_reduce(mx, true, red);  // also orders the staging stores before the reads below
        float sum = 0.f;
        for (int i = tid; i < V; i += kLsgThreads) sum += __expf(to_f<T>(row[i]) - mx);
        sum = block_reduce(sum, false, red);
        const float lse = __logf(sum);
        const int64_t bi = r / rpb, li = r % rpb;
        for (int s = tid; s < slen; s += kLsgThreads) {
            int64_t t = sel[bi * sb + li * sl + (int64_t)s * ss];
            float v;
            if (t < 0 || t >= V) {
                v = CUDART_NAN_F;
                flag(status, PCFGNAT_STATUS_BAD_INDEX);
            } else {
                v = (to_f<T>(row[t]) - mx) - lse;
            }
            selected[(size_t)r * slen + s] = v;
        }
        if (req_grad) {
            __syncthreads();  // every gather has read its logit before the row is overwritten
            if (STAGE && vec_ok) {
                uint4 *g4 = reinterpret_cast<uint4 *>(grow);
                const uint4 *s4 = reinterpret_cast<const uint4 *>(srow);
                for (int i = tid; i < V / kVec; i += kLsgThreads) {
                    uint4 v = s4[i];
                    T *e = reinterpret_cast<T *>(&v);
#pragma unroll
                    for (int k = 0; k < kVec; k++) e[k] = from_f<T>(__fdividef(__expf(to_f<T>(e[k]) - mx), sum));
                    g4[i] = v;
                }
            } else {
                for (int i = tid; i < V; i += kLsgThreads)
                    grow[i] = from_f<T>(__fdividef(__expf(to_f<T>(row[i]) - mx), sum));
            }
        }
        __syncthreads();  // the staged row is reused by the next iteration
    }
}

constexpr int kStreamThreads = 512;
constexpr uint32_t kChunkBytes = 32768;  // bytes per bulk copy and per barrier
constexpr int kMaxChunks = 7;            // 224 KB: the longest row one CTA can hold

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Bounded wait for a chunk's bytes; false when the limit ran out.
__device__ __forceinline__ bool bulk_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.b32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16 bytes of a row at a time: the maximum is taken in the storage type (packed halves stay packed), the
// exponentials in float32.
template <typename T>
struct Pack;
template <>
struct Pack<float> {
    static __device__ __forceinline__ float max_of(const uint4 &v) {
        return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)), fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
    }
    static __device__ __forceinline__ uint4 lowest() { return make_uint4(0xff800000u, 0xff800000u, 0xff800000u, 0xff800000u); }
    static __device__ __forceinline__ void unpack(const uint4 &v, float *f) {
        f[0] = __uint_as_float(v.x), f[1] = __uint_as_float(v.y), f[2] = __uint_as_float(v.z), f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float *f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};
template <>
struct Pack<__half> {
    static __device__ __forceinline__ __half2 h2(uint32_t u) { return *reinterpret_cast<const __half2 *>(&u); }
    static __device__ __forceinline__ float max_of(const uint4 &v) {
        const __half2 m = __hmax2(__hmax2(h2(v.x), h2(v.y)), __hmax2(h2(v.z), h2(v.w)));
        return __half2float(__hmax(__low2half(m), __high2half(m)));
    }
    static __device__ __forceinline__ uint4 lowest() { return make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u); }
    static __device__ __forceinline__ void unpack(const uint4 &v, float *f) {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 p = __half22float2(h2(u[k]));
            f[2 * k] = p.x, f[2 * k + 1] = p.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float *f) {
        uint32_t u[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const __half2 h = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
            u[k] = *reinterpret_cast<const uint32_t *>(&h);
        }
        return make_uint4(u[0], u[1], u[2], u[3]);
    }
};

// The streaming kernel.  A CTA holds one row in shared memory as nch chunks of kChunkBytes, every chunk with its own
// barrier; thread 0 fetches chunks with bulk asynchronous copies.  The sum of exponentials is accumulated chunk by
// chunk as the chunks land, against a running maximum per thread (when a thread meets a larger entry it rescales
// what it has summed), so that no sweep waits for the whole row.  Without the softmax a chunk is refilled with the
// next row's bytes as soon as it has been summed (the gathered logits are then re-read from global memory, which
// still holds them); with the softmax the row stays until the probabilities have been written, and each chunk is
// refilled as soon as it has been written out.  Two CTAs per SM (when two rows fit) run out of step with one
// another, which keeps both the exponential unit and the copy stream busy.
// Rows of V * sizeof(T) bytes, a multiple of 16, on a 16-byte aligned base; nch * kChunkBytes >= the row.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
    logsoftmax_gather_stream_kernel(T *logits, const int64_t *__restrict__ sel, int64_t sb, int64_t sl, int64_t ss,
                                    int64_t rows, int64_t rpb, int V, int slen, int req_grad, float *selected,
                                    int *status, int nch) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float2 red[2][kStreamThreads / 32];  // (maximum, sum) per warp; rows alternate between the two halves
    __shared__ __align__(8) uint64_t bars[kMaxChunks];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int kVec = 16 / sizeof(T);
    const uint32_t row_bytes = (uint32_t)V * sizeof(T);
    const uint32_t base = dsm_smem_u32(smem_raw);
    const uint32_t bar0 = dsm_smem_u32(&bars[0]);
    if (tid == 0) {
        for (int c = 0; c < nch; c++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8 * c) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto chunk_bytes = [&](int c) {
        const uint32_t off = (uint32_t)c * kChunkBytes;
        return row_bytes - off < kChunkBytes ? row_bytes - off : kChunkBytes;
    };
    auto fetch = [&](int64_t r, int c) {  // thread 0 only; every thread is past its reads of chunk c
        const uint32_t bar = bar0 + 8 * c, n = chunk_bytes(c);
        asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(n) : "memory");
        bulk_load(base + c * kChunkBytes, reinterpret_cast<const unsigned char *>(logits + (size_t)r * V) + (size_t)c * kChunkBytes,
                  n, bar);
    };
    if (tid == 0 && (int64_t)blockIdx.x < rows)
        for (int c = 0; c < nch; c++) fetch(blockIdx.x, c);
    const float kLog2e = 1.4426950408889634f;
    const bool early = slen <= kStreamThreads;
    uint32_t par = 0;  // every barrier completes one phase per row
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, par ^= 1) {
        const int64_t next = r + gridDim.x;
        const bool has_next = next < rows;
        // the logits to gather are fetched now, from global memory (the row there is rewritten only at the end of
        // this iteration), so that their latency is spent under the sweep
        T *grow = logits + (size_t)r * V;
        const int64_t bi = r / rpb, li = r % rpb;
        int64_t t_sel = 0;
        float x_sel = 0.f;
        if (early && tid < slen) {
            t_sel = sel[bi * sb + li * sl + (int64_t)tid * ss];
            if (t_sel < 0 || t_sel >= V) flag(status, PCFGNAT_STATUS_BAD_INDEX);
            else x_sel = to_f<T>(grow[t_sel]);
        }
        float m = -CUDART_INF_F, sum = 0.f, sum_b = 0.f, shift = 0.f;  // shift = -m * log2(e), 0 while m is still -inf
        bool ok = true;
        int failed_at = nch;
        for (int c = 0; c < nch; c++) {
            ok = ok && bulk_wait(bar0 + 8 * c, par);
            if (ok) {
                const uint4 *s4 = reinterpret_cast<const uint4 *>(smem_raw + (size_t)c * kChunkBytes);
                const int n16 = chunk_bytes(c) / 16;
                for (int i = tid; i < n16; i += 2 * kStreamThreads) {  // two independent 16-byte pieces at a time
                    const uint4 v0 = s4[i];
                    const uint4 v1 = i + kStreamThreads < n16 ? s4[i + kStreamThreads] : Pack<T>::lowest();
                    const float vm = fmaxf(Pack<T>::max_of(v0), Pack<T>::max_of(v1));
                    if (vm > m) {
                        const float scale = ex2_ftz((m - vm) * kLog2e);  // m == -inf: the sums are 0 and stay 0
                        sum *= scale, sum_b *= scale;
                        m = vm;
                        shift = -vm * kLog2e;
                    }
                    float f0[kVec], f1[kVec];
                    Pack<T>::unpack(v0, f0);
                    Pack<T>::unpack(v1, f1);
#pragma unroll
                    for (int k = 0; k < kVec; k++) {
                        sum += ex2_ftz(fmaf(f0[k], kLog2e, shift));
                        sum_b += ex2_ftz(fmaf(f1[k], kLog2e, shift));
                    }
                }
            }
            if (!req_grad) {  // the chunk is done with: hand it to the next row
                if (__syncthreads_or(!ok)) {
                    failed_at = c;
                    break;
                }
                if (tid == 0 && has_next) fetch(next, c);
            }
        }
        if (req_grad && __syncthreads_or(!ok)) failed_at = 0;
        if (failed_at < nch) {  // a copy never arrived: report, let no copy outlive the CTA, stop
            if (tid == 0) {
                flag(status, PCFGNAT_STATUS_TIMEOUT);
                for (int c = 0; c < nch; c++) {
                    if (c < failed_at && !has_next) continue;  // consumed and not refilled
                    bulk_wait(bar0 + 8 * c, c < failed_at ? par ^ 1 : par);
                }
            }
            __syncthreads();
            return;
        }
        // (maximum, sum) of the row: within each warp, through shared memory (one barrier), across the warps
        float wm = m;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
        float ws = m == -CUDART_INF_F ? 0.f : (sum + sum_b) * ex2_ftz((m - wm) * kLog2e);  // a thread without entries
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
        if (lane == 0) red[par][warp] = make_float2(wm, ws);
        __syncthreads();
        const float2 part = red[par][lane & (kStreamThreads / 32 - 1)];
        float mx = part.x;
#pragma unroll
        for (int o = kStreamThreads / 64; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        sum = part.x == -CUDART_INF_F ? 0.f : part.y * ex2_ftz((part.x - mx) * kLog2e);  // a warp without entries
#pragma unroll
        for (int o = kStreamThreads / 64; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float lse = __logf(sum);
        if (early) {
            if (tid < slen) selected[(size_t)r * slen + tid] = t_sel < 0 || t_sel >= V ? CUDART_NAN_F : (x_sel - mx) - lse;
        } else {
            const T *row = req_grad ? reinterpret_cast<const T *>(smem_raw) : grow;
            for (int s = tid; s < slen; s += kStreamThreads) {
                int64_t t = sel[bi * sb + li * sl + (int64_t)s * ss];
                float v;
                if (t < 0 || t >= V) {
                    v = CUDART_NAN_F;
                    flag(status, PCFGNAT_STATUS_BAD_INDEX);
                } else {
                    v = (to_f<T>(row[t]) - mx) - lse;
                }
                selected[(size_t)r * slen + s] = v;
            }
        }
        if (req_grad) {  // softmax = ex2(x * log2(e) - (mx * log2(e) + log2(sum))): the division is in the exponent
            const float shift2 = -mx * kLog2e - __log2f(sum);
            for (int c = 0; c < nch; c++) {
                const uint4 *s4 = reinterpret_cast<const uint4 *>(smem_raw + (size_t)c * kChunkBytes);
                uint4 *g4 = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(grow) + (size_t)c * kChunkBytes);
                const int n16 = chunk_bytes(c) / 16;
                for (int i = tid; i < n16; i += kStreamThreads) {
                    float f[kVec];
                    Pack<T>::unpack(s4[i], f);
#pragma unroll
                    for (int k = 0; k < kVec; k++) f[k] = ex2_ftz(fmaf(f[k], kLog2e, shift2));
                    g4[i] = Pack<T>::pack(f);
                }
                __syncthreads();  // the gathers and this sweep have read chunk c
                if (tid == 0 && has_next) fetch(next, c);
            }
        }
    }
}

template <typename T>
int launch_typed(T *logits, const int64_t *sel, int64_t sb, int64_t sl, int64_t ss, int64_t rows, int64_t rpb, int V,
                 int slen, int req_grad, float *selected, int *status, cudaStream_t st) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t row_bytes = ((size_t)V * sizeof(T) + 15) / 16 * 16;
    const int vec_ok = ((size_t)V * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(logits) % 16) == 0;
    cudaError_t e;
    const int nch = (int)(((size_t)V * sizeof(T) + kChunkBytes - 1) / kChunkBytes);
    const size_t stream_bytes = ((size_t)V * sizeof(T) + 127) / 128 * 128;
    const char *env = getenv("PCFGNAT_LSG_STREAM");  // "0": the single-buffer kernels only
    if (vec_ok && nch <= kMaxChunks && stream_bytes + 2048 <= (size_t)kSmemLimit && !(env && env[0] == '0')) {
        auto k = logsoftmax_gather_stream_kernel<T>;
        e = ensure_dynamic_smem(k, stream_bytes);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        int per_sm = (int)((size_t)kSmemLimit / (stream_bytes + 2048));
        if (per_sm > 2) per_sm = 2;  // two CTAs out of step fill each other's barriers and reductions
        int64_t grid = (int64_t)sms * per_sm;
        if (grid > rows) grid = rows;
        k<<<(unsigned)grid, kStreamThreads, stream_bytes, st>>>(logits, sel, sb, sl, ss, rows, rpb, V, slen, req_grad,
                                                               selected, status, nch);
    } else if (row_bytes <= (size_t)kSmemLimit - 2048) {
        auto k = logsoftmax_gather_kernel<T, true>;
        e = ensure_dynamic_smem(k, row_bytes);
        if (e != cudaSuccess) return PCFGNAT_ERR_CUDA;
        int per_sm = (int)(((size_t)kSmemLimit) / (row_bytes + 1024));
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 2048 / kLsgThreads) per_sm = 2048 / kLsgThreads;
        int64_t grid = (int64_t)sms * per_sm;
        if (grid > rows) grid = rows;
        k<<<(unsigned)grid, kLsgThreads, row_bytes, st>>>(logits, sel, sb, sl, ss, rows, rpb, V, slen, req_grad,
                                                         selected, status, vec_ok);
    } else {
        auto k = logsoftmax_gather_kernel<T, false>;
        int64_t grid = (int64_t)sms * (2048 / kLsgThreads);
        if (grid > rows) grid = rows;
        k<<<(unsigned)grid, kLsgThreads, 0, st>>>(logits, sel, sb, sl, ss, rows, rpb, V, slen, req_grad, selected,
                                                 status, 0);
    }
    return cuda_rc(cudaGetLastError());
}

}  // namespace

int launch_logsoftmax_gather(void *logits, int dtype, const int64_t *sel, int64_t sb, int64_t sl, int64_t ss,
                             int64_t rows, int64_t rpb, int V, int slen, int req_grad, float *selected, int *status,
                             cudaStream_t st) {
    if (rows == 0) return PCFGNAT_OK;
    if (dtype == PCFGNAT_DTYPE_F32)
        return launch_typed<float>(static_cast<float *>(logits), sel, sb, sl, ss, rows, rpb, V, slen, req_grad,
                                   selected, status, st);
    if (dtype == PCFGNAT_DTYPE_F16)
        return launch_typed<__half>(static_cast<__half *>(logits), sel, sb, sl, ss, rows, rpb, V, slen, req_grad,
                                    selected, status, st);
    return PCFGNAT_ERR_UNSUPPORTED;
}

}  // namespace pcfgnat
