// Warp-level tensor-core tiles (mma.sync m16n8k16, bf16 in, float32 sums in registers) for the passes whose
// products are narrow and whose results are needed in registers by row-wise float32 math right after (norms,
// activations): fragment helpers shared by tail.cu and gate.cu. Device code only.
//
// Fragment layout, g = lane / 4, t = lane % 4: A (16 x 16, row major) holds in a[0..3] the pairs (row g, columns 2t,
// 2t + 1), (g + 8, 2t..), (g, 2t + 8..), (g + 8, 2t + 8..); B (16 x 8) holds in b0, b1 the pairs (rows 2t, 2t + 1 of
// column g) and (rows 2t + 8, 2t + 9); the accumulator c[0..3] holds (row g, columns 2t, 2t + 1) and (row g + 8, same).
#pragma once
#include "common.cuh"

namespace hsnw {

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    return static_cast<uint32_t>(bf16_bits(lo)) | (static_cast<uint32_t>(bf16_bits(hi)) << 16);
}

// c += a b for one 16 x 8 tile: a 16 x 16 (row major fragments), b 16 x 8 (column fragments), bf16 in, float32 sums.
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four (two) 8 x 8 blocks of bf16 values, each handed out transposed: a lane ends up with the elements [2t][g] and
// [2t + 1][g] of block i in r[i]. Lane l gives the address of row l % 8 of block l / 8.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row) {
    const uint32_t at = static_cast<uint32_t>(__cvta_generic_to_shared(row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(at));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], const void* row) {
    const uint32_t at = static_cast<uint32_t>(__cvta_generic_to_shared(row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(at));
}

// acc[nt] = the warp's 16 rows r0.. of A (bf16 rows of pitch PWA words in shared memory, K = 16 KS along a row) times
// B, with B(k, n) read as the packed pair (k, k + 1) of row n of Bs (pitch PWB words): Bs holds the right-hand side
// with its summed index along a row.
template <int NT, int KS, int PWA, int PWB>
__device__ __forceinline__ void warp_rows_product(float (&acc)[NT][4], const uint32_t* As, const uint32_t* Bs, int r0, int g, int t) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        uint32_t a[4];
        a[0] = As[(r0 + g) * PWA + 8 * ks + t];
        a[1] = As[(r0 + g + 8) * PWA + 8 * ks + t];
        a[2] = As[(r0 + g) * PWA + 8 * ks + 4 + t];
        a[3] = As[(r0 + g + 8) * PWA + 8 * ks + 4 + t];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_bf16(acc[nt], a, Bs[(8 * nt + g) * PWB + 8 * ks + t], Bs[(8 * nt + g) * PWB + 8 * ks + 4 + t]);
    }
}

__device__ __forceinline__ float sum4_lanes(float v) {   // over the 4 lanes that share a row of a fragment
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

}  // namespace hsnw
