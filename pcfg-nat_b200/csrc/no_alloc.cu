// pcfgnat_loss_fwd_bwd_static: loss forward + backward for hosts that cannot provide scratch.
//
// The regular entry point (pcfgnat_loss_fwd_bwd) needs a caller-supplied workspace for the two
// DP tables (inside scores S and outside weights G).  Some hosts have no way to produce one: an
// FFI binding that only ever sees device pointers owned by another framework and links no CUDA
// runtime of its own, or a serving / training process that gave all device memory to its own
// arena at start-up and must not let a library call cudaMalloc behind its back (the call would
// fail, or stall every stream of the device while it runs).  For them the two tables live in a
// fixed array that is part of this library's device image.
//
// Consequences the caller has to know:
//   * the array costs PCFGNAT_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the
//     library, from load until process exit, whether or not this entry point is ever called;
//   * problems whose tables do not fit are refused with PCFGNAT_ERR_TOO_LARGE — nothing is
//     allocated as a fallback;
//   * every call on a device uses the same array, so two calls whose kernels may overlap on that
//     device (different streams, different host threads) race on it: serialise them;
//   * the array keeps the previous call's tables.  Nothing here relies on its contents: the
//     kernels overwrite every cell of both tables (fill -inf / 0, then the DP) before reading
//     them, so no clearing pass is needed;
//   * the first call on each device looks the array's device address up
//     (cudaGetSymbolAddress, which can initialise the CUDA context and load this module); make
//     that first call before starting any stream capture on the device.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kScratchBytes = PCFGNAT_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// The name `g_scratch` below is only a host-side handle in host code; kernels must be given the
// address cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

std::mutex g_mu;
void *g_scratch_addr[kMaxDevices] = {};

// Device address of g_scratch on the current device (looked up once per device).
int scratch_for_current_device(void **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PCFGNAT_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || !p) return PCFGNAT_ERR_CUDA;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return PCFGNAT_OK;
}

}  // namespace

extern "C" int pcfgnat_loss_fwd_bwd_static(const float *match_all, const float *links, const int64_t *output_length,
                                           const int64_t *target_length, int B, int L, int T, int max_left,
                                           float *loss, float *match_all_grad, float *links_grad, int *status,
                                           void *stream) {
    using namespace pcfgnat;
    if (max_left != 1) return PCFGNAT_ERR_UNSUPPORTED;
    if (B < 0 || L < 2 || T < 1) return PCFGNAT_ERR_INVALID_ARGUMENT;
    if (B && (!match_all || !links || !output_length || !target_length || !loss || !match_all_grad || !links_grad))
        return PCFGNAT_ERR_INVALID_ARGUMENT;
    // two tables of B x Mc x (T+2) floats, each rounded up to 256 bytes, and the frames of the linear-space pass
    const size_t table = ((size_t)B * main_slots(L, 1) * (size_t)(T + 2) * sizeof(float) + 255) / 256 * 256;
    if (2 * table + linear_frames_bytes(B, T) > kScratchBytes) return PCFGNAT_ERR_TOO_LARGE;
    if (B == 0) return PCFGNAT_OK;
    void *base = nullptr;
    int rc = scratch_for_current_device(&base);
    if (rc) return rc;
    return loss_fwd_bwd_in(match_all, links, output_length, target_length, B, L, T, base, table, loss, match_all_grad,
                           links_grad, status, static_cast<cudaStream_t>(stream));
}
