// Shared device helpers of the window kernels: bf16 rounding, activations, block reductions and
// 16-byte row copies. Device code only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace hsnw {

constexpr float kSqrtHalf = 0.7071067811865475244f;
constexpr float kInvSqrt2Pi = 0.3989422804014326779f;

// float32 -> nearest bfloat16 (ties to even), returned as the float32 of that value. A NaN stays
// a NaN (the canonical one). The cast up from bfloat16 is exact, so a value rounded here is what a
// bf16 buffer would hold.
__device__ __forceinline__ float bf16r(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));   // one conversion instruction each way
}
__device__ __forceinline__ float maybe_bf16(float x, bool on) { return on ? bf16r(x) : x; }
__device__ __forceinline__ uint16_t bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf16_value(uint16_t h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }

// The record of the hidden pre-activations: float32, or bfloat16 when the products are bf16 (the values
// are bfloat16 then, so nothing is lost and the record is half the bytes).
__device__ __forceinline__ void store_hidden(void* base, int64_t at, float v, bool half) {
    if (half) static_cast<uint16_t*>(base)[at] = bf16_bits(v);
    else static_cast<float*>(base)[at] = v;
}
__device__ __forceinline__ float load_hidden(const void* base, int64_t at, bool half) {
    return half ? bf16_value(static_cast<const uint16_t*>(base)[at]) : static_cast<const float*>(base)[at];
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * kSqrtHalf)); }
__device__ __forceinline__ float gelu_erf_grad(float x) {
    return 0.5f * (1.0f + erff(x * kSqrtHalf)) + x * expf(-0.5f * x * x) * kInvSqrt2Pi;
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// A float as an unsigned key of the same order (-0 and +0 compare equal, as in a float compare).
__device__ __forceinline__ uint32_t float_order(float x) {
    x += 0.0f;  // -0 -> +0
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// (score, cell) as one key: a larger key is a higher score, or the same score at a lower index.
__device__ __forceinline__ uint64_t pack_key(float score, int cell) {
    return (static_cast<uint64_t>(float_order(score)) << 32) | (0xffffffffu - static_cast<uint32_t>(cell));
}
__device__ __forceinline__ int key_cell(uint64_t key) { return static_cast<int>(0xffffffffu - static_cast<uint32_t>(key)); }

__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t v, int lane_mask) {
    const uint32_t lo = __shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(v), lane_mask);
    const uint32_t hi = __shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(v >> 32), lane_mask);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v) {
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) {
        const uint64_t o = shfl_xor_u64(v, w);
        v = o > v ? o : v;
    }
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) v += __shfl_xor_sync(0xffffffffu, v, w);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, w));
    return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) v += __shfl_xor_sync(0xffffffffu, v, w);
    return v;
}

// Block-wide reductions over a scratch of 33 words of 8 bytes; every thread gets the result.
// Two barriers each; blockDim.x is a multiple of 32, at most 1024.
__device__ __forceinline__ uint64_t block_max_u64(uint64_t v, uint64_t* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    v = warp_max_u64(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    uint64_t r = lane < warps ? scratch[lane] : 0ull;
    r = warp_max_u64(r);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max_float(float v, uint64_t* scratch) {
    float* s = reinterpret_cast<float*>(scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    v = warp_max(v);
    if (lane == 0) s[warp] = v;
    __syncthreads();
    float r = lane < warps ? s[lane] : -INFINITY;
    r = warp_max(r);
    __syncthreads();
    return r;
}
__device__ __forceinline__ int block_sum_int(int v, uint64_t* scratch) {
    int* s = reinterpret_cast<int*>(scratch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    v = warp_sum_int(v);
    if (lane == 0) s[warp] = v;
    __syncthreads();
    int r = lane < warps ? s[lane] : 0;
    r = warp_sum_int(r);
    __syncthreads();
    return r;
}

// sum_i a[i * sa] * b[i * sb], i < n, with four independent accumulators and eight products per
// round, every operand of a round loaded before the first product: a single chain of dependent
// multiply-adds would wait for each load in turn. The order of the sum is fixed.
__device__ __forceinline__ float dot4(const float* a, int sa, const float* b, int sb, int n) {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        const float* pa = a + i * sa;
        const float* pb = b + i * sb;
        const float a0 = pa[0], a1 = pa[sa], a2 = pa[2 * sa], a3 = pa[3 * sa];
        const float a4 = pa[4 * sa], a5 = pa[5 * sa], a6 = pa[6 * sa], a7 = pa[7 * sa];
        const float b0 = pb[0], b1 = pb[sb], b2 = pb[2 * sb], b3 = pb[3 * sb];
        const float b4 = pb[4 * sb], b5 = pb[5 * sb], b6 = pb[6 * sb], b7 = pb[7 * sb];
        s0 += a0 * b0; s1 += a1 * b1; s2 += a2 * b2; s3 += a3 * b3;
        s0 += a4 * b4; s1 += a5 * b5; s2 += a6 * b6; s3 += a7 * b7;
    }
    for (; i < n; ++i) s0 += a[i * sa] * b[i * sb];
    return (s0 + s1) + (s2 + s3);
}
// Up to four dot products that share b: out[r] = sum_i a[r * lda + i] * b[i * sb], r < rows <= 4,
// each in dot4's order (bit for bit the same sums). A value of b is loaded once for the four rows.
__device__ __forceinline__ void dot4_rows(const float* a, int lda, int rows, const float* b, int sb, int n,
                                          float out[4]) {
    float s[4][4] = {};
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        float bv[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) bv[w] = b[(i + w) * sb];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            if (r < rows) {
                const float* pa = a + r * lda + i;
                float av[8];
#pragma unroll
                for (int w = 0; w < 8; ++w) av[w] = pa[w];
#pragma unroll
                for (int w = 0; w < 8; ++w) s[r][w & 3] += av[w] * bv[w];
            }
        }
    }
    for (; i < n; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (r < rows) s[r][0] += a[r * lda + i] * b[i * sb];
#pragma unroll
    for (int r = 0; r < 4; ++r) out[r] = (s[r][0] + s[r][1]) + (s[r][2] + s[r][3]);
}
// e / n for a run-time n >= 2 as one multiply-high: magic_of(n) = ceil(2^32 / n), exact while e n < 2^32
// (an integer division by a run-time value costs about twenty instructions, and the index arithmetic
// of the element loops is full of them).
__device__ __forceinline__ uint32_t magic_of(int n) { return 0xffffffffu / static_cast<uint32_t>(n) + 1u; }
__device__ __forceinline__ int div_magic(int e, uint32_t magic) {
    return static_cast<int>(__umulhi(static_cast<uint32_t>(e), magic));
}
// sum_i a[i * sa], i < n, the same way.
__device__ __forceinline__ float sum4(const float* a, int64_t sa, int n) {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int i = 0;
    for (; i + 4 <= n; i += 4) {
        const float a0 = a[i * sa], a1 = a[(i + 1) * sa], a2 = a[(i + 2) * sa], a3 = a[(i + 3) * sa];
        s0 += a0; s1 += a1; s2 += a2; s3 += a3;
    }
    for (; i < n; ++i) s0 += a[i * sa];
    return (s0 + s1) + (s2 + s3);
}

// dst[0..n) = src[0..n) floats by the whole block; 16-byte transfers when both are aligned and
// n is a multiple of 4.
__device__ __forceinline__ void block_copy_f32(float* dst, const float* src, int n) {
    const bool vec = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0 && (n & 3) == 0;
    if (vec) {
        const float4* s4 = reinterpret_cast<const float4*>(src);
        float4* d4 = reinterpret_cast<float4*>(dst);
        for (int e = threadIdx.x; e < (n >> 2); e += blockDim.x) d4[e] = s4[e];
    } else {
        for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = src[e];
    }
}

}  // namespace hsnw
