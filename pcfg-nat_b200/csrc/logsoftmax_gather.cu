// log-softmax over the vocabulary + gather of selected columns (+ optional in-place
// softmax for the backward).
//
// Replaces logsoftmax_gather_kernel of the reference
// (fs_plugins/custom_ops/logsoftmax_gather.cu:240-292), which sweeps each row three times
// from global memory (max, sum-exp, softmax write).  Here one CTA owns one row at a time and
// keeps it resident in shared memory in its storage type (fp16 rows of 40 000 entries are
// 80 KB, so two CTAs fit per SM): one HBM read, and one HBM write only when the softmax is
// asked for.  Rows that do not fit fall back to re-reading global memory.
// Like the reference this kernel uses the fast exp/log/divide intrinsics
// (logsoftmax_gather.cu:107-148), so parity with it is by tolerance.
#include <cuda_fp16.h>

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
    extern __shared__ __align__(16) unsigned char smem_raw[];
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

template <typename T>
int launch_typed(T *logits, const int64_t *sel, int64_t sb, int64_t sl, int64_t ss, int64_t rows, int64_t rpb, int V,
                 int slen, int req_grad, float *selected, int *status, cudaStream_t st) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t row_bytes = ((size_t)V * sizeof(T) + 15) / 16 * 16;
    const int vec_ok = ((size_t)V * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(logits) % 16) == 0;
    cudaError_t e;
    if (row_bytes <= (size_t)kSmemLimit - 2048) {
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
