// Staging of global memory into shared memory with many bytes in flight per thread:
//   * cp.async (16 bytes per instruction, no registers held), and
//   * the TMA's untiled bulk copy (cp.async.bulk) completing on an mbarrier, for contiguous,
//     16-byte aligned runs (a state row, a row of logits, a tile of scalars).
// Every wait is bounded: after kStageSpinLimit polls the waiter gives up, records it in an error
// word the host can read, and the kernel carries on to its end (no trap, no endless spin).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hsnw {

constexpr uint32_t kStageSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- cp.async -------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_global) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr(dst_smem)), "l"(src_global) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src_global) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr(dst_smem)), "l"(src_global) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// floats [0, n) from src to dst by the whole block, 16 bytes at a time where both sides allow it
// (else 4 bytes at a time). The caller commits and waits.
__device__ __forceinline__ void cp_async_floats(float* dst, const float* src, int n) {
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(smem_addr(dst))) & 15) == 0;
    if (vec) {
        const int n4 = n >> 2;
        for (int e = threadIdx.x; e < n4; e += blockDim.x) cp_async16(dst + 4 * e, src + 4 * e);
        for (int e = (n4 << 2) + threadIdx.x; e < n; e += blockDim.x) cp_async4(dst + e, src + e);
    } else {
        for (int e = threadIdx.x; e < n; e += blockDim.x) cp_async4(dst + e, src + e);
    }
}

// ---- mbarrier + bulk copy ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_global, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
            smem_addr(dst_smem)),
        "l"(src_global), "r"(bytes), "r"(smem_addr(bar))
        : "memory");
}
// Wait for the phase with the given parity; false (and *error set) if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t spin = 0; spin < kStageSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    if (error) atomicExch(error, 1);
    return false;
}
__device__ __forceinline__ bool bulk_ok(const void* src, const void* dst_smem, size_t bytes) {
    return ((reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(smem_addr(dst_smem)) | bytes) & 15) == 0 && bytes > 0;
}

}  // namespace hsnw
