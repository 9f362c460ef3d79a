// 5th-generation tensor core primitives for sm_100a as inline PTX: tensor memory (TMEM)
// allocation, shared-memory matrix descriptors, tcgen05.mma issue / commit, tcgen05.ld.
//
// Operand layout used throughout this library: K-major, no swizzle. An operand tile of R rows
// (R = M for A, N for B) and KT elements along K (bf16) is stored as KT/8 planes; plane kc holds,
// for every row r, the 8 consecutive K-elements 8 kc .. 8 kc + 7 as one 16-byte unit at byte
// offset kc * (R * 16) + r * 16. Eight consecutive rows of a plane are one 8 x 16-byte core
// matrix (128 contiguous bytes), so in the descriptor the stride between core matrices along the
// rows ("stride byte offset") is 128 and the stride between the two K-halves of a K = 16
// instruction ("leading byte offset") is R * 16. One tcgen05.mma consumes two planes; the next
// K-step starts 2 * R * 16 bytes further on.
//
// The accumulator D [128, N] fp32 lives in TMEM: lane i holds row i, column j holds column j.
// Warp w of the epilogue may touch lanes 32 w .. 32 w + 31 only.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "stage.cuh"

namespace hsnw {

// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, dense, M x N.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4)                                  // D format: F32
           | (1u << 7)                                // A format: BF16
           | (1u << 10)                               // B format: BF16
           | (static_cast<uint32_t>(N >> 3) << 17)    // N / 8
           | (static_cast<uint32_t>(M >> 4) << 24);   // M / 16
}

// Shared-memory matrix descriptor for the layout above (rows = R of the tile).
__device__ __forceinline__ uint64_t umma_desc(const void* smem_tile, int rows) {
    const uint32_t addr = smem_addr(smem_tile);
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);                                   // start address
    desc |= static_cast<uint64_t>((static_cast<uint32_t>(rows) * 16u >> 4) & 0x3fffu) << 16;  // leading byte offset
    desc |= static_cast<uint64_t>((128u >> 4) & 0x3fffu) << 32;                             // stride byte offset
    desc |= static_cast<uint64_t>(1) << 46;                                                 // descriptor version (sm_100)
    return desc;                                                                            // layout type 0: no swizzle
}

// Shared-memory matrix descriptor for a K-major tile in the 128-byte swizzle: rows of 64 bf16 (128
// bytes, one K-block), groups of 8 rows are 1024-byte atoms in which the 16-byte unit u of row r sits
// at unit u ^ (r % 8); the tile starts on a 1024-byte boundary. Stride between row groups 1024 bytes;
// the leading offset is not used by this layout. A K = 16 step inside the block moves the start
// address by 32 bytes; the next K-block of a wider tile starts rows x 128 bytes further on. The
// tensor cores fetch this layout a 128-byte row at a time (the unswizzled layout above goes 16 bytes
// at a time: an M = 128 product then costs ~256 cycles of operand fetch whatever N is).
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_tile) {
    const uint32_t addr = smem_addr(smem_tile);
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
    desc |= static_cast<uint64_t>(1) << 16;                     // leading byte offset: unused, 1
    desc |= static_cast<uint64_t>((1024u >> 4) & 0x3fffu) << 32;  // stride byte offset
    desc |= static_cast<uint64_t>(1) << 46;                     // descriptor version (sm_100)
    desc |= static_cast<uint64_t>(2) << 61;                     // layout type: 128-byte swizzle
    return desc;
}

// TMEM: `columns` is a power of two >= 32. Executed by one whole warp; the base address lands in
// *slot (shared memory). Every .sync.aligned instruction here is preceded by __syncwarp(): a warp
// that left a polling loop or a single-thread branch is not necessarily converged, and an aligned
// instruction run by a diverged warp returned the rows of the wrong lanes.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t columns) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(slot)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// Generic-proxy writes to shared memory become visible to the tensor core's (async proxy) reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- issuing products ------------------------------------------------------------------------------
// Every function below is executed by ALL 32 lanes of a CONVERGED warp; one lane, elected inside the
// instruction sequence itself (elect.sync, the same lane every time for a full warp), issues. The
// control flow around a tcgen05.mma therefore stays warp-uniform, and that matters: measured on a
// B200, a chain issued from a one-thread branch (`if (tid == 0)`) costs about 200 cycles per product
// whatever its shape (16 products M 128 x N 16: 3370 cycles from the first issue to the commit's
// arrival), the same chain issued this way 728 cycles (about 35 a product after a fixed ~250), and
// M 128 x N 256 products then run at the tensor pipe's own rate (136 cycles each). With this issue
// rate consecutive products into ONE accumulator are as fast as products spread over several (727
// cycles either way), so a product's K steps simply accumulate in place. Inside a kernel whose other
// warps are busy the issuing warp needs about 70 cycles of instructions per product (the chains are
// unrolled: as a rolled loop with run-time descriptor arithmetic they cost 50 cycles more each), twice
// the tensor pipe's time for an N = 16 product: chains that do not depend on one another are therefore
// issued by different warps (window_rows.cu).
//
// D[tmem] (+)= A[smem] * B[smem]^T for one K = 16 step.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n"
        ".reg .pred lead, acc;\n"
        "elect.sync _|lead, 0xffffffff;\n"
        "setp.ne.b32 acc, %4, 0;\n"
        "@lead tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, acc;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
        : "memory");
}
// A chain of `steps` K = 16 products into one accumulator: D = sum_s A_s B_s^T, the descriptors
// advancing by a_step / b_step (16-byte units) per product. `onto`: add to what the accumulator holds
// (a sum that runs over several chains).
__device__ __forceinline__ void umma_chain(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, int steps,
                                           uint32_t a_step, uint32_t b_step, bool onto = false) {
    __syncwarp();
    // Kept rolled: left to the compiler's own four-fold unrolling of this run-time count, one instantiation
    // (the grouped unit pass's first weight gradient) issued the first four products of a six-step chain
    // with the rows of A taken modulo 8, as if the descriptor's stride between core matrices were zero,
    // and the two of the remainder loop correctly; with one product per iteration every chain is right.
#pragma unroll 1
    for (int s = 0; s < steps; ++s)
        umma_bf16(tmem_d, desc_a + static_cast<uint64_t>(s) * a_step, desc_b + static_cast<uint64_t>(s) * b_step, idesc,
                  onto || s > 0);
}
// The same with the count known at compile time: the loop unrolls to a few instructions per product.
template <int STEPS>
__device__ __forceinline__ void umma_chain_fixed(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t a_step, uint32_t b_step, bool onto) {
    __syncwarp();
#pragma unroll
    for (int s = 0; s < STEPS; ++s)
        umma_bf16(tmem_d, desc_a + static_cast<uint64_t>(s) * a_step, desc_b + static_cast<uint64_t>(s) * b_step, idesc,
                  onto || s > 0);
}
// The chain for an A tile in the 128-byte swizzle (K-blocks of 64: four K = 16 steps of 32 bytes, then
// the next block a_block 16-byte units further on) and a B tile in the unswizzled layout.
template <int STEPS>
__device__ __forceinline__ void umma_chain_sw128(uint32_t tmem_d, uint64_t desc_a, uint32_t a_block, uint64_t desc_b,
                                                 uint32_t b_step, uint32_t idesc, bool onto) {
    __syncwarp();
#pragma unroll
    for (int s = 0; s < STEPS; ++s)
        umma_bf16(tmem_d, desc_a + static_cast<uint64_t>(s >> 2) * a_block + static_cast<uint64_t>(s & 3) * 2u,
                  desc_b + static_cast<uint64_t>(s) * b_step, idesc, onto || s > 0);
}
// The step between two K = 16 products of a tile of `rows` rows in the layout above.
__host__ __device__ constexpr uint32_t umma_kstep(int rows) { return static_cast<uint32_t>((2 * rows * 16) >> 4); }
// All products issued so far by the elected lane arrive on `bar` when they have completed (executed by
// the whole converged warp, like the products themselves: the commit tracks the issuing thread's).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile(
        "{\n"
        ".reg .pred lead;\n"
        "elect.sync _|lead, 0xffffffff;\n"
        "@lead tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
        "}\n" ::"r"(smem_addr(bar))
        : "memory");
}
// Eight consecutive fp32 columns of this thread's TMEM lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float out[8]) {
    uint32_t r[8];
    __syncwarp();  // .sync.aligned: the warp must be converged (it may come out of a polling loop)
    // The load and its wait are ONE asm statement: the registers are defined only after the wait,
    // so the compiler cannot schedule a use of them between the two instructions.
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __uint_as_float(r[i]);
}
// Thirty-two consecutive fp32 columns of this thread's TMEM lane, one wait.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float out[32]) {
    uint32_t r[32];
    __syncwarp();
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = __uint_as_float(r[i]);
}
// Four consecutive fp32 columns at taddr and the four 16 columns further on (an accumulator pair's
// same four slots), one wait for both loads.
__device__ __forceinline__ void tmem_ld4x2(uint32_t taddr, float out[8]) {
    uint32_t r[8];
    __syncwarp();
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%8];\n"
        "tcgen05.ld.sync.aligned.32x32b.x4.b32 {%4, %5, %6, %7}, [%9];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr), "r"(taddr + 16u)
        : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int column) {
    return base + (static_cast<uint32_t>(lane) << 16) + static_cast<uint32_t>(column);
}

}  // namespace hsnw
