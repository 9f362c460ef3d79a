// Helpers shared by the per-row cluster kernels (window_rows.cu, window_rows_bwd.cu): distributed
// shared memory access, the TMA ring's barriers, bf16 unpacking, asynchronous staging.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"
#include "stage.cuh"

namespace cg = cooperative_groups;
using namespace hsnw;

namespace {

constexpr int kConsumers = 256;       // compute threads (8 warps)

template <class T>
__device__ __forceinline__ T* peer(cg::cluster_group& cl, T* p, int rank) {
    return cl.map_shared_rank(p, rank);
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumers) : "memory"); }
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// sum_i a[i * sa] * w[i * sw] with bf16 weights, n a multiple of 8: four independent sums, the loads
// of a round issued before its products (a single chain of dependent multiply-adds waits for each).
__device__ __forceinline__ float dot_bf16w(const float* a, int sa, const uint16_t* w, int sw, int n) {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    for (int i = 0; i < n; i += 8) {
        const float* pa = a + i * sa;
        const uint16_t* pw = w + i * sw;
        const float a0 = pa[0], a1 = pa[sa], a2 = pa[2 * sa], a3 = pa[3 * sa];
        const float a4 = pa[4 * sa], a5 = pa[5 * sa], a6 = pa[6 * sa], a7 = pa[7 * sa];
        const uint16_t w0 = pw[0], w1 = pw[sw], w2 = pw[2 * sw], w3 = pw[3 * sw];
        const uint16_t w4 = pw[4 * sw], w5 = pw[5 * sw], w6 = pw[6 * sw], w7 = pw[7 * sw];
        s0 += a0 * bf16_value(w0); s1 += a1 * bf16_value(w1); s2 += a2 * bf16_value(w2); s3 += a3 * bf16_value(w3);
        s0 += a4 * bf16_value(w4); s1 += a5 * bf16_value(w5); s2 += a6 * bf16_value(w6); s3 += a7 * bf16_value(w7);
    }
    return (s0 + s1) + (s2 + s3);
}

// A bounded wait on a ring barrier. After the first wait of the block that ran out (recorded in
// *failed and in the status word) every later wait returns at once, so a broken pipeline costs one
// time-out, not one per stage: the kernel still reaches every cluster barrier and ends.
// The wait carries a suspend-time hint: without one a waiting warp comes back from the instruction
// almost at once and polls, taking issue slots from the warp of its scheduler that feeds the tensor
// cores or the copies (measured: 0.4 us a position of the forward sweep, 0.3 of the reverse); with it
// the warp sleeps in hardware until the phase completes or the hint (a microsecond) runs out. The
// bound: 2^20 rounds of at most a microsecond.
__device__ __forceinline__ void ring_wait(uint64_t* bar, uint32_t parity, int* status, volatile int* failed) {
    if (*failed) return;
    const uint32_t addr = smem_addr(bar);
    for (uint32_t spin = 0; spin < (1u << 20); ++spin) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(1000u)
            : "memory");
        if (done) return;
    }
    *failed = 1;
    if (status) atomicExch(status, 1);
}

// floats [0, n) from global to shared memory by the 256 compute threads, asynchronously.
__device__ __forceinline__ void prefetch_floats(float* dst, const float* src, int n, int tid, int threads = kConsumers) {
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(smem_addr(dst))) & 15) == 0;
    if (vec) {
        const int n4 = n >> 2;
        for (int e = tid; e < n4; e += threads) cp_async16(dst + 4 * e, src + 4 * e);
        for (int e = (n4 << 2) + tid; e < n; e += threads) cp_async4(dst + e, src + e);
    } else {
        for (int e = tid; e < n; e += threads) cp_async4(dst + e, src + e);
    }
}


}  // namespace
