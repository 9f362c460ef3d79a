// Shared device helpers of the window kernels: bf16 rounding, activations, block reductions and
// 16-byte row copies. Device code only.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace hsnw {

constexpr float kSqrtHalf = 0.7071067811865475244f;
constexpr float kInvSqrt2Pi = 0.3989422804014326779f;

// float32 -> nearest bfloat16 (ties to even), returned as the float32 of that value. A NaN stays
// a quiet NaN. The cast up from bfloat16 is exact, so a value rounded here is what a bf16 buffer
// would hold.
__device__ __forceinline__ float bf16r(float x) {
    const uint32_t u = __float_as_uint(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float((u | 0x00400000u) & 0xffff0000u);
    return __uint_as_float((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
}
__device__ __forceinline__ float maybe_bf16(float x, bool on) { return on ? bf16r(x) : x; }
__device__ __forceinline__ uint16_t bf16_bits(float x) { return static_cast<uint16_t>(__float_as_uint(bf16r(x)) >> 16); }
__device__ __forceinline__ float bf16_value(uint16_t h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }

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
