// Small wrappers around the sm_100a instructions the tensor-core kernels are built from: mbarriers with bounded
// waits, TMA tile loads (this CTA only, no multicast), tcgen05 shared-memory and instruction descriptors, MMA
// issue and commit, tensor-memory loads.  Shared by proj_fused.cu and proj_bwd_gemm.cu.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace pcfgnat {
namespace tc {

constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Bounded wait: false when the limit ran out or another role of the CTA already gave up (abort_flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.b32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
        if (it > 4096) __nanosleep(128);  // long waits only: a sleeping warp wakes up to 128 ns late
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// True in exactly one lane of a fully converged warp (the same lane on every call).
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.b32 %0, 1, 0, p; }" : "=r"(chosen));
    return chosen != 0;
}

// Tile (x = innermost coordinate, y) of a 2-d tensor map into this CTA's shared memory; the bytes are counted on bar.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory descriptors for 16-bit operands in 128-byte-swizzled tiles whose rows are 128 B (64 elements).
// K-major: a row holds 64 consecutive K of one M/N index; 8-row groups 1024 B apart.  Advancing K by 16
// elements inside the swizzle span adds 32 B to the start address (+2 in the address field).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) /* leading byte offset: unused */ |
           (64ull << 32) /* stride byte offset 1024 B */ | (1ull << 46) /* sm_100 descriptor */ | (2ull << 61) /* SWIZZLE_128B */;
}
// The same with rows of 64 B (32 elements) in 64-byte-swizzled tiles: 8-row groups 512 B apart.
__device__ __forceinline__ uint64_t desc_k_major_sw64(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (32ull << 32) /* 512 B */ | (1ull << 46) |
           (4ull << 61) /* SWIZZLE_64B */;
}
// MN-major: a row holds 64 consecutive M/N indices of one K; 8 rows (8 K) are a 1024-byte group (stride byte
// offset), and each further block of 64 M/N indices is a tile of its own `block_bytes` further on (leading byte
// offset).  Advancing K by 16 elements is 16 rows = 2048 B.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr, uint32_t block_bytes) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((block_bytes >> 4) & 0x3FFFu) << 16) | (64ull << 32) |
           (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16 with float32 accumulation: formats 0 = f16, 1 = bf16; major 0 = K, 1 = MN.
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n, int a_format, int b_format, int a_mn, int b_mn) {
    return (1u << 4) | ((uint32_t)a_format << 7) | ((uint32_t)b_format << 10) | ((uint32_t)a_mn << 15) |
           ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier when the MMAs issued so far by this thread are done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t columns) {  // one whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {  // the warp that allocated
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// Issues the load of 32 accumulator columns of this thread's row; valid only after tmem_ld_wait(r).
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
// Waits for the outstanding tcgen05.ld; the registers are in/out operands so that no use of them moves above it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t *r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda); null when unavailable.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

}  // namespace tc
}  // namespace pcfgnat
