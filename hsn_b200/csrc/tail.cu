// The end of the replay's cell pass over every slot of a window at once, and its backward:
//   y = W_out(unit_out), pre = RMSNorm_g(y), c = tanh(alpha * pre)      (reference python/hsn/model/cell.py:719-721)
// with autograd's gradients of unit_out, alpha, W_out.weight and the norm's gain. The slots are independent, so a
// tile of 64 slots is one block's work: the tile and W_out sit in shared memory, a thread holds 4 slots x d/16
// columns of the product, the norm's row sums are shuffles over the 16 lanes that share a slot. The pass is bound by
// the tensors it reads and writes once (y and c are 2 x 4 d bytes a slot, the product 2 d^2 flops); the backward
// keeps each block's share of d_W_out in registers over all of its tiles and a second kernel adds the blocks' shares
// in block order, so the sums have the same bits every run.
#include "../../include/hsn_tail_b200.h"
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "host_util.h"

#include <algorithm>
#include <cstdint>

namespace {
using namespace hsnw;

constexpr int kThreads = 256;
constexpr int kTile = 64;        // slots a tile: 16 thread rows x 4 slots
constexpr int kSumLanes = 4;     // interleaved partial sums of the final reduction (a fixed order)

template <int D>
struct Shape {
    static constexpr int CPT = D / 16;     // columns a thread
    static constexpr int WP = D + 1;       // pitch of a row of W_out: lanes that read a column hit 16 banks
    static constexpr int XP = D + 4;       // pitch of a tile row: rows stay 16-byte aligned
    static constexpr size_t fwd_bytes = sizeof(float) * (kTile * XP + D * WP + D);
    static constexpr size_t bwd_bytes = sizeof(float) * (2 * kTile * XP + D * WP + D + 16 * D);
};

__device__ __forceinline__ float sum16(float v) {   // over the 16 lanes of a half warp
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

// A tile of unit_out as float rows in shared memory; rows beyond the last slot are zero.
template <int D, bool BF>
__device__ __forceinline__ void load_tile(float* X, const void* src, int64_t first, int64_t slots, int tid) {
    constexpr int XP = Shape<D>::XP, Q = D / 4;
    for (int e = tid; e < kTile * Q; e += kThreads) {
        const int p = e / Q, q = e - p * Q;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (first + p < slots) {
            if constexpr (BF) {
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(src) + (first + p) * D) + q);
                v.x = bf16_value(static_cast<uint16_t>(raw.x & 0xffffu));
                v.y = bf16_value(static_cast<uint16_t>(raw.x >> 16));
                v.z = bf16_value(static_cast<uint16_t>(raw.y & 0xffffu));
                v.w = bf16_value(static_cast<uint16_t>(raw.y >> 16));
            } else {
                v = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(src) + (first + p) * D) + q);
            }
        }
        *reinterpret_cast<float4*>(X + p * XP + 4 * q) = v;
    }
}

template <int D, bool BF>
__device__ __forceinline__ void load_weights(float* W, float* G, const float* w_out, const float* gain, int tid) {
    for (int e = tid; e < D * D; e += kThreads) {
        const int j = e / D, k = e - j * D;
        W[j * Shape<D>::WP + k] = maybe_bf16(__ldg(w_out + e), BF);
    }
    for (int e = tid; e < D; e += kThreads) G[e] = __ldg(gain + e);
}

// acc[i][c] = sum_k A[(ty 4 + i)][k] * B(k, tx + 16 c), A a tile in shared memory read four k at a time.
template <int D, typename BAt>
__device__ __forceinline__ void tile_product(float (&acc)[4][Shape<D>::CPT], const float* A, int ty, BAt&& b_at) {
    constexpr int CPT = Shape<D>::CPT, XP = Shape<D>::XP;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < CPT; ++c) acc[i][c] = 0.0f;
#pragma unroll 2
    for (int k = 0; k < D; k += 4) {
        float4 a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(A + (ty * 4 + i) * XP + k);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const float w = b_at(k + kk, c);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float av = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
                    acc[i][c] = fmaf(av, w, acc[i][c]);
                }
            }
        }
    }
}

template <int D, bool BF>
__global__ void __launch_bounds__(kThreads)
k_tail_fwd(const float* __restrict__ w_out, const float* __restrict__ gain, float eps, const void* __restrict__ unit_out,
           const float* __restrict__ alpha, int64_t slots, float* __restrict__ y_out, float* __restrict__ c_out) {
    constexpr int CPT = Shape<D>::CPT, WP = Shape<D>::WP, XP = Shape<D>::XP;
    extern __shared__ __align__(16) float smem[];
    float* X = smem;               // [kTile][XP]
    float* W = X + kTile * XP;     // [D][WP]: W_out[j][k]
    float* G = W + D * WP;         // [D]
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kTile;
    load_weights<D, BF>(W, G, w_out, gain, tid);
    load_tile<D, BF>(X, unit_out, first, slots, tid);
    __syncthreads();
    float acc[4][CPT];
    tile_product<D>(acc, X, ty, [&](int k, int c) { return W[(tx + 16 * c) * WP + k]; });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t p = first + ty * 4 + i;
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            acc[i][c] = maybe_bf16(acc[i][c], BF);
            ss = fmaf(acc[i][c], acc[i][c], ss);
        }
        ss = sum16(ss);
        const float rho = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
        if (p < slots) {
            const float a = __ldg(alpha + p);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int j = tx + 16 * c;
                y_out[p * D + j] = acc[i][c];
                c_out[p * D + j] = tanhf(a * (acc[i][c] * rho * G[j]));
            }
        }
    }
}

// `partial` [blocks][D D + D]: the block's share of d_W_out, then of the gain's gradient.
template <int D, bool BF>
__global__ void __launch_bounds__(kThreads)
k_tail_bwd(const float* __restrict__ w_out, const float* __restrict__ gain, float eps, const void* __restrict__ unit_out,
           const float* __restrict__ alpha, const float* __restrict__ y_in, const float* __restrict__ d_c, int64_t slots,
           void* __restrict__ d_unit_out, float* __restrict__ d_alpha, float* __restrict__ partial) {
    constexpr int CPT = Shape<D>::CPT, WP = Shape<D>::WP, XP = Shape<D>::XP;
    extern __shared__ __align__(16) float smem[];
    float* X = smem;                // [kTile][XP] unit_out
    float* DY = X + kTile * XP;     // [kTile][XP] d_y
    float* W = DY + kTile * XP;     // [D][WP]
    float* G = W + D * WP;          // [D]
    float* GS = G + D;              // [16][D] the thread rows' shares of the gain's gradient
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    load_weights<D, BF>(W, G, w_out, gain, tid);
    float dw[CPT][CPT];
    float dg[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
        dg[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) dw[i][c] = 0.0f;
    }
    const int64_t tiles = (slots + kTile - 1) / kTile;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t first = tile * kTile;
        __syncthreads();   // the previous tile's reads are over; the weights are in place
        load_tile<D, BF>(X, unit_out, first, slots, tid);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t p = first + ty * 4 + i;
            const bool in = p < slots;
            float yv[CPT], dc[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                yv[c] = in ? __ldg(y_in + p * D + tx + 16 * c) : 0.0f;
                dc[c] = in ? __ldg(d_c + p * D + tx + 16 * c) : 0.0f;
            }
            const float a = in ? __ldg(alpha + p) : 0.0f;
            float ss = 0.0f;
#pragma unroll
            for (int c = 0; c < CPT; ++c) ss = fmaf(yv[c], yv[c], ss);
            ss = sum16(ss);
            const float rho = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
            float scaled[CPT];
            float da = 0.0f, dot = 0.0f;
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const float g = G[tx + 16 * c];
                const float pre = yv[c] * rho * g;
                const float cv = tanhf(a * pre);
                const float dz = dc[c] * (1.0f - cv * cv);
                da = fmaf(dz, pre, da);
                const float dpre = a * dz;
                dg[c] = fmaf(dpre * yv[c], rho, dg[c]);
                scaled[c] = dpre * g;
                dot = fmaf(yv[c], scaled[c], dot);
            }
            da = sum16(da);
            dot = sum16(dot);
            const float mean = dot / static_cast<float>(D);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const float dy = rho * scaled[c] - rho * rho * rho * yv[c] * mean;
                DY[(ty * 4 + i) * XP + tx + 16 * c] = maybe_bf16(dy, BF);
            }
            if (in && tx == 0) d_alpha[p] = da;
        }
        __syncthreads();
        // d_unit_out = d_y W_out
        float acc[4][CPT];
        tile_product<D>(acc, DY, ty, [&](int j, int c) { return W[j * WP + tx + 16 * c]; });
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t p = first + ty * 4 + i;
            if (p < slots) {
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    const int64_t at = p * D + tx + 16 * c;
                    if constexpr (BF) static_cast<uint16_t*>(d_unit_out)[at] = bf16_bits(acc[i][c]);
                    else static_cast<float*>(d_unit_out)[at] = acc[i][c];
                }
            }
        }
        // d_W_out[j][k] += sum_p d_y[p][j] unit_out[p][k], j = ty + 16 i, k = tx + 16 c
#pragma unroll 4
        for (int p = 0; p < kTile; ++p) {
            float av[CPT], bv[CPT];
#pragma unroll
            for (int i = 0; i < CPT; ++i) {
                av[i] = DY[p * XP + ty + 16 * i];
                bv[i] = X[p * XP + tx + 16 * i];
            }
#pragma unroll
            for (int i = 0; i < CPT; ++i)
#pragma unroll
                for (int c = 0; c < CPT; ++c) dw[i][c] = fmaf(av[i], bv[c], dw[i][c]);
        }
    }
    float* mine = partial + static_cast<int64_t>(blockIdx.x) * (D * D + D);
#pragma unroll
    for (int i = 0; i < CPT; ++i)
#pragma unroll
        for (int c = 0; c < CPT; ++c) mine[(ty + 16 * i) * D + tx + 16 * c] = dw[i][c];
#pragma unroll
    for (int c = 0; c < CPT; ++c) GS[ty * D + tx + 16 * c] = dg[c];
    __syncthreads();
    for (int e = tid; e < D; e += kThreads) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 16; ++r) s += GS[r * D + e];
        mine[D * D + e] = s;
    }
}

// The blocks' shares added in block order (kSumLanes interleaved sums, then those in order).
template <bool BF>
__global__ void __launch_bounds__(kThreads)
k_tail_wgrad(const float* __restrict__ partial, int blocks, int d, float* __restrict__ d_w_out, float* __restrict__ d_gain) {
    const int outputs = d * d + d;
    const int e = static_cast<int>(blockIdx.x) * kThreads + static_cast<int>(threadIdx.x);
    if (e >= outputs) return;
    float s[kSumLanes];
#pragma unroll
    for (int l = 0; l < kSumLanes; ++l) s[l] = 0.0f;
    int b = 0;
    for (; b + kSumLanes <= blocks; b += kSumLanes) {
#pragma unroll
        for (int l = 0; l < kSumLanes; ++l) s[l] += __ldg(partial + static_cast<int64_t>(b + l) * outputs + e);
    }
    for (int l = 0; b + l < blocks; ++l) s[l] += __ldg(partial + static_cast<int64_t>(b + l) * outputs + e);
    float total = s[0];
#pragma unroll
    for (int l = 1; l < kSumLanes; ++l) total += s[l];
    if (e < d * d) d_w_out[e] = maybe_bf16(total, BF);
    else d_gain[e - d * d] = total;
}

int blocks_per_sm(int d) { return d <= 64 ? 2 : 1; }

int check(const HsnwTail* t, int64_t slots, const char* what) {
    if (!t || slots < 0) return hsnw_fail(HSNW_E_ARG, what);
    if (!t->w_out) return hsnw_fail(HSNW_E_ARG, "tail: null W_out");
    if (!t->norm_weight) return hsnw_fail(HSNW_E_ARG, "tail: the pass without the candidate norm is not taken here");
    if (t->d != 16 && t->d != 32 && t->d != 64 && t->d != 128) return hsnw_fail(HSNW_E_UNSUPPORTED, "tail: d must be 16, 32, 64 or 128");
    if (!(t->norm_eps >= 0.0f)) return hsnw_fail(HSNW_E_ARG, "tail: negative or NaN norm_eps");
    return HSNW_OK;
}

int64_t bwd_blocks(int d, int64_t slots, int sms) {
    const int64_t tiles = (slots + kTile - 1) / kTile;
    return std::max<int64_t>(1, std::min<int64_t>(tiles, static_cast<int64_t>(sms) * blocks_per_sm(d)));
}

template <int D, bool BF>
void launch_fwd(const HsnwTail* t, const void* unit_out, const float* alpha, int64_t slots, float* y, float* c, cudaStream_t stream) {
    const unsigned tiles = static_cast<unsigned>((slots + kTile - 1) / kTile);
    k_tail_fwd<D, BF><<<tiles, kThreads, Shape<D>::fwd_bytes, stream>>>(t->w_out, t->norm_weight, t->norm_eps, unit_out, alpha, slots, y, c);
}

template <int D, bool BF>
void launch_bwd(const HsnwTail* t, const void* unit_out, const float* alpha, const float* y, const float* d_c, int64_t slots,
                void* d_unit_out, float* d_alpha, float* partial, int blocks, cudaStream_t stream) {
    k_tail_bwd<D, BF><<<static_cast<unsigned>(blocks), kThreads, Shape<D>::bwd_bytes, stream>>>(
        t->w_out, t->norm_weight, t->norm_eps, unit_out, alpha, y, d_c, slots, d_unit_out, d_alpha, partial);
}

}  // namespace

extern "C" int64_t hsnw_tail_scratch_bytes(const HsnwTail* tail, int64_t slots) {
    if (!tail || slots < 0 || tail->d < 16 || tail->d > 128) return 0;
    const int sms = std::max(148, hsnw_sm_count_current());
    const int64_t bytes = bwd_blocks(tail->d, slots, sms) * (static_cast<int64_t>(tail->d) * tail->d + tail->d) * static_cast<int64_t>(sizeof(float));
    return (bytes + 255) / 256 * 256;
}

extern "C" int hsnw_tail_forward(const HsnwTail* tail, const void* unit_out, const float* alpha, int64_t slots, float* y, float* c,
                                 void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(tail, slots, "tail_forward: null or negative")) return rc;
    if (slots == 0) return HSNW_OK;
    if (!unit_out || !alpha || !y || !c) return hsnw_fail(HSNW_E_ARG, "tail_forward: null tensor");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    hsnw_profile_mark(HSNW_K_TAIL_FWD, stream);
#define HSNW_TAIL_FWD(D) \
    case D: \
        if (tail->prod_bf16) launch_fwd<D, true>(tail, unit_out, alpha, slots, y, c, stream); \
        else launch_fwd<D, false>(tail, unit_out, alpha, slots, y, c, stream); \
        break
    switch (tail->d) {
        HSNW_TAIL_FWD(16);
        HSNW_TAIL_FWD(32);
        HSNW_TAIL_FWD(64);
        HSNW_TAIL_FWD(128);
    }
#undef HSNW_TAIL_FWD
    return hsnw_check_launch("tail_forward");
}

extern "C" int hsnw_tail_backward(const HsnwTail* tail, const void* unit_out, const float* alpha, const float* y, const float* d_c,
                                  int64_t slots, void* d_unit_out, float* d_alpha, float* d_w_out, float* d_norm_weight,
                                  void* scratch, int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(tail, slots, "tail_backward: null or negative")) return rc;
    if (!d_w_out || !d_norm_weight) return hsnw_fail(HSNW_E_ARG, "tail_backward: null gradient");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int d = tail->d;
    if (slots == 0) {
        if (cudaMemsetAsync(d_w_out, 0, sizeof(float) * d * d, stream) != cudaSuccess
            || cudaMemsetAsync(d_norm_weight, 0, sizeof(float) * d, stream) != cudaSuccess)
            return hsnw_check_launch("tail_backward");
        return HSNW_OK;
    }
    if (!unit_out || !alpha || !y || !d_c || !d_unit_out || !d_alpha) return hsnw_fail(HSNW_E_ARG, "tail_backward: null tensor");
    if (!scratch || scratch_bytes < hsnw_tail_scratch_bytes(tail, slots)) return hsnw_fail(HSNW_E_ARG, "tail_backward: scratch too small");
    if (reinterpret_cast<uintptr_t>(scratch) % 16) return hsnw_fail(HSNW_E_ARG, "tail_backward: scratch not 16-byte aligned");
    const int blocks = static_cast<int>(bwd_blocks(d, slots, std::max(1, hsnw_sm_count_current())));
    float* partial = static_cast<float*>(scratch);
    hsnw_profile_mark(HSNW_K_TAIL_BWD, stream);
#define HSNW_TAIL_BWD(D) \
    case D: \
        if (tail->prod_bf16) launch_bwd<D, true>(tail, unit_out, alpha, y, d_c, slots, d_unit_out, d_alpha, partial, blocks, stream); \
        else launch_bwd<D, false>(tail, unit_out, alpha, y, d_c, slots, d_unit_out, d_alpha, partial, blocks, stream); \
        break
    switch (d) {
        HSNW_TAIL_BWD(16);
        HSNW_TAIL_BWD(32);
        HSNW_TAIL_BWD(64);
        HSNW_TAIL_BWD(128);
    }
#undef HSNW_TAIL_BWD
    const unsigned out_blocks = static_cast<unsigned>((d * d + d + kThreads - 1) / kThreads);
    if (tail->prod_bf16) k_tail_wgrad<true><<<out_blocks, kThreads, 0, stream>>>(partial, blocks, d, d_w_out, d_norm_weight);
    else k_tail_wgrad<false><<<out_blocks, kThreads, 0, stream>>>(partial, blocks, d, d_w_out, d_norm_weight);
    return hsnw_check_launch("tail_backward");
}

void hsnw_tail_set_attributes() {
    bool ok = true;
#define HSNW_TAIL_OPT(D) \
    ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_fwd<D, true>), "tail_fwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_fwd<D, false>), "tail_fwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_bwd<D, true>), "tail_bwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_bwd<D, false>), "tail_bwd")
    HSNW_TAIL_OPT(16);
    HSNW_TAIL_OPT(32);
    HSNW_TAIL_OPT(64);
    HSNW_TAIL_OPT(128);
#undef HSNW_TAIL_OPT
    if (!ok) hsnw_attribute_failed();
}
