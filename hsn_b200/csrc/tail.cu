// The end of the replay's cell pass over every slot of a window at once, and its backward:
//   y = W_out(unit_out), pre = RMSNorm_g(y), c = tanh(alpha * pre)      (reference python/hsn/model/cell.py:719-721)
// with autograd's gradients of unit_out, alpha, W_out.weight and the norm's gain. The slots are independent, so a
// tile of slots is one block's work with the tile and W_out in shared memory. The pass is bound by the tensors it
// reads and writes once (y and c are 2 x 4 d bytes a slot against 2 d^2 flops), so the products only have to stay out
// of the way: with bf16 products a warp takes 16 slots through warp-level tensor-core products (mma.sync m16n8k16,
// fp32 accumulators in registers, where the norm's row sums and the tanh need them: 2 shuffles a row, no round trip
// through tensor memory for a 64-wide row); in float32 a thread holds 4 slots x d/16 columns on the CUDA cores.
// The backward keeps each block's share of d_W_out in registers over all of its tiles and a second kernel adds the
// blocks' shares in a fixed order, so the sums have the same bits every run.
#include "../../include/hsn_tail_b200.h"
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "host_util.h"
#include "mma_tiles.cuh"

#include <algorithm>
#include <cstdint>

namespace {
using namespace hsnw;

constexpr int kThreads = 256;
constexpr int kTile = 64;        // slots a tile of the float32 kernels: 16 thread rows x 4 slots

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
template <int D>
__device__ __forceinline__ void load_tile(float* X, const float* src, int64_t first, int64_t slots, int tid) {
    constexpr int XP = Shape<D>::XP, Q = D / 4;
    for (int e = tid; e < kTile * Q; e += kThreads) {
        const int p = e / Q, q = e - p * Q;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (first + p < slots) v = __ldg(reinterpret_cast<const float4*>(src + (first + p) * D) + q);
        *reinterpret_cast<float4*>(X + p * XP + 4 * q) = v;
    }
}

template <int D>
__device__ __forceinline__ void load_weights(float* W, float* G, const float* w_out, const float* gain, int tid) {
    for (int e = tid; e < D * D; e += kThreads) {
        const int j = e / D, k = e - j * D;
        W[j * Shape<D>::WP + k] = __ldg(w_out + e);
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

template <int D>
__global__ void __launch_bounds__(kThreads)
k_tail_fwd(const float* __restrict__ w_out, const float* __restrict__ gain, float eps, const float* __restrict__ unit_out,
           const float* __restrict__ alpha, int64_t slots, float* __restrict__ y_out, float* __restrict__ c_out) {
    constexpr int CPT = Shape<D>::CPT, WP = Shape<D>::WP, XP = Shape<D>::XP;
    extern __shared__ __align__(16) float smem[];
    float* X = smem;               // [kTile][XP]
    float* W = X + kTile * XP;     // [D][WP]: W_out[j][k]
    float* G = W + D * WP;         // [D]
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kTile;
    load_weights<D>(W, G, w_out, gain, tid);
    load_tile<D>(X, unit_out, first, slots, tid);
    __syncthreads();
    float acc[4][CPT];
    tile_product<D>(acc, X, ty, [&](int k, int c) { return W[(tx + 16 * c) * WP + k]; });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t p = first + ty * 4 + i;
        float ss = 0.0f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
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
template <int D>
__global__ void __launch_bounds__(kThreads)
k_tail_bwd(const float* __restrict__ w_out, const float* __restrict__ gain, float eps, const float* __restrict__ unit_out,
           const float* __restrict__ alpha, const float* __restrict__ y_in, const float* __restrict__ d_c, int64_t slots,
           float* __restrict__ d_unit_out, float* __restrict__ d_alpha, float* __restrict__ partial) {
    constexpr int CPT = Shape<D>::CPT, WP = Shape<D>::WP, XP = Shape<D>::XP;
    extern __shared__ __align__(16) float smem[];
    float* X = smem;                // [kTile][XP] unit_out
    float* DY = X + kTile * XP;     // [kTile][XP] d_y
    float* W = DY + kTile * XP;     // [D][WP]
    float* G = W + D * WP;          // [D]
    float* GS = G + D;              // [16][D] the thread rows' shares of the gain's gradient
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    load_weights<D>(W, G, w_out, gain, tid);
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
        load_tile<D>(X, unit_out, first, slots, tid);
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
                DY[(ty * 4 + i) * XP + tx + 16 * c] = dy;
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
                for (int c = 0; c < CPT; ++c) d_unit_out[p * D + tx + 16 * c] = acc[i][c];
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

// ---------------------------------------------------------------------------------------------------------------
// bf16 products: a tile of 128 slots, a warp owns 16 of them.

constexpr int kTileMma = 128;

template <int D>
struct MmaShape {
    static constexpr int PB = D + 8;        // pitch of a row of bf16 values: rows 16-byte aligned, fragment loads hit 32 banks
    static constexpr int PW = PB / 2;       // the same in 32-bit words
    static constexpr int NT = D / 8;        // 8-column tiles of a row
    static constexpr int KS = D / 16;       // 16-deep steps of a product over d
    static constexpr int MT = D / 16;       // 16-row tiles of d_W_out
    static constexpr int TILES = MT * NT;
    static constexpr int TPW = (TILES + 7) / 8;   // d_W_out tiles a warp
    static constexpr size_t fwd_bytes = sizeof(uint32_t) * (kTileMma * PW + D * PW) + sizeof(float) * D;
    static constexpr size_t bwd_bytes = sizeof(uint32_t) * (2 * kTileMma * PW + D * PW) + sizeof(float) * (D + 8 * D);
};

// A tile of unit_out (bf16) into shared memory rows of pitch PB; rows beyond the last slot are zero.
template <int D>
__device__ __forceinline__ void load_tile_bf16(uint32_t* Xs, const uint16_t* src, int64_t first, int64_t slots, int tid) {
    constexpr int PW = MmaShape<D>::PW, Q = D / 8;
    for (int e = tid; e < kTileMma * Q; e += kThreads) {
        const int p = e / Q, q = e - p * Q;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (first + p < slots) v = __ldg(reinterpret_cast<const uint4*>(src + (first + p) * D) + q);
        *reinterpret_cast<uint4*>(Xs + p * PW + 4 * q) = v;
    }
}

// acc[nt] = the warp's 16 rows of A (rows r0.. of a tile in shared memory) times B, B(k, n) read as the packed pair
// (k, k + 1) of row n of Bs: Bs holds the right-hand side with its summed index along a row.
template <int D>
__device__ __forceinline__ void warp_product(float (&acc)[MmaShape<D>::NT][4], const uint32_t* As, const uint32_t* Bs, int r0, int g, int t) {
    constexpr int PW = MmaShape<D>::PW, NT = MmaShape<D>::NT, KS = MmaShape<D>::KS;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        uint32_t a[4];
        a[0] = As[(r0 + g) * PW + 8 * ks + t];
        a[1] = As[(r0 + g + 8) * PW + 8 * ks + t];
        a[2] = As[(r0 + g) * PW + 8 * ks + 4 + t];
        a[3] = As[(r0 + g + 8) * PW + 8 * ks + 4 + t];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t b0 = Bs[(8 * nt + g) * PW + 8 * ks + t];
            const uint32_t b1 = Bs[(8 * nt + g) * PW + 8 * ks + 4 + t];
            mma_bf16(acc[nt], a, b0, b1);
        }
    }
}

// A lane holds, of row g + 8 h of its warp's 16 rows, the columns 8 nt + 2 t and + 1 in acc[nt][2 h], [2 h + 1].
template <int D>
__global__ void __launch_bounds__(kThreads)
k_tail_fwd_mma(const float* __restrict__ w_out, const float* __restrict__ gain, float eps, const uint16_t* __restrict__ unit_out,
               const float* __restrict__ alpha, int64_t slots, float* __restrict__ y_out, float* __restrict__ c_out) {
    constexpr int PW = MmaShape<D>::PW, NT = MmaShape<D>::NT;
    extern __shared__ __align__(16) uint32_t smem_w[];
    uint32_t* Xs = smem_w;                  // [kTileMma][PW] unit_out
    uint32_t* Ws = Xs + kTileMma * PW;      // [D][PW] W_out[j][k]
    float* G = reinterpret_cast<float*>(Ws + D * PW);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kTileMma;
    for (int e = tid; e < D * D / 2; e += kThreads) {
        const int j = e / (D / 2), k2 = e - j * (D / 2);
        const float2 v = __ldg(reinterpret_cast<const float2*>(w_out) + e);
        Ws[j * PW + k2] = pack_bf16(v.x, v.y);
    }
    for (int e = tid; e < D; e += kThreads) G[e] = __ldg(gain + e);
    load_tile_bf16<D>(Xs, unit_out, first, slots, tid);
    __syncthreads();
    float acc[NT][4];
    warp_product<D>(acc, Xs, Ws, warp * 16, g, t);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int64_t p = first + warp * 16 + g + 8 * h;
        float ss = 0.0f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            acc[nt][2 * h] = bf16r(acc[nt][2 * h]);
            acc[nt][2 * h + 1] = bf16r(acc[nt][2 * h + 1]);
            ss = fmaf(acc[nt][2 * h], acc[nt][2 * h], ss);
            ss = fmaf(acc[nt][2 * h + 1], acc[nt][2 * h + 1], ss);
        }
        ss = sum4_lanes(ss);
        const float rho = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
        if (p < slots) {
            const float a = __ldg(alpha + p);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int j = 8 * nt + 2 * t;
                const float y0 = acc[nt][2 * h], y1 = acc[nt][2 * h + 1];
                *reinterpret_cast<float2*>(y_out + p * D + j) = make_float2(y0, y1);
                *reinterpret_cast<float2*>(c_out + p * D + j) = make_float2(tanhf(a * (y0 * rho * G[j])), tanhf(a * (y1 * rho * G[j + 1])));
            }
        }
    }
}

template <int D>
__global__ void __launch_bounds__(kThreads)
k_tail_bwd_mma(const float* __restrict__ w_out, const float* __restrict__ gain, float eps, const uint16_t* __restrict__ unit_out,
               const float* __restrict__ alpha, const float* __restrict__ y_in, const float* __restrict__ d_c, int64_t slots,
               uint16_t* __restrict__ d_unit_out, float* __restrict__ d_alpha, float* __restrict__ partial) {
    using S = MmaShape<D>;
    constexpr int PB = S::PB, PW = S::PW, NT = S::NT, MT = S::MT, TILES = S::TILES, TPW = S::TPW;
    extern __shared__ __align__(16) uint32_t smem_w[];
    uint32_t* Xs = smem_w;                   // [kTileMma][PW] unit_out
    uint32_t* DYs = Xs + kTileMma * PW;      // [kTileMma][PW] d_y
    uint32_t* Wt = DYs + kTileMma * PW;      // [D][PW] Wt[k][j] = W_out[j][k]
    float* G = reinterpret_cast<float*>(Wt + D * PW);
    float* GS = G + D;                       // [8][D] the warps' shares of the gain's gradient
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    for (int e = tid; e < D * D / 2; e += kThreads) {
        const int k = e / (D / 2), j2 = e - k * (D / 2);
        Wt[k * PW + j2] = pack_bf16(__ldg(w_out + (2 * j2) * D + k), __ldg(w_out + (2 * j2 + 1) * D + k));
    }
    for (int e = tid; e < D; e += kThreads) G[e] = __ldg(gain + e);
    float dw[TPW][4];
    float dg[NT][2];
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) dw[i][c] = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) dg[nt][0] = dg[nt][1] = 0.0f;
    const int r0 = warp * 16;
    const int mt = warp % MT;
    const int64_t tiles = (slots + kTileMma - 1) / kTileMma;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t first = tile * kTileMma;
        __syncthreads();   // the previous tile's reads are over; the weights are in place
        load_tile_bf16<D>(Xs, unit_out, first, slots, tid);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r0 + g + 8 * h;
            const int64_t p = first + row;
            const bool in = p < slots;
            float2 yv[NT], sc[NT];   // sc: the cotangent, then g d_pre
            float ss = 0.0f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int j = 8 * nt + 2 * t;
                yv[nt] = in ? __ldg(reinterpret_cast<const float2*>(y_in + p * D + j)) : make_float2(0.0f, 0.0f);
                sc[nt] = in ? __ldg(reinterpret_cast<const float2*>(d_c + p * D + j)) : make_float2(0.0f, 0.0f);
                ss = fmaf(yv[nt].x, yv[nt].x, ss);
                ss = fmaf(yv[nt].y, yv[nt].y, ss);
            }
            const float a = in ? __ldg(alpha + p) : 0.0f;
            ss = sum4_lanes(ss);
            const float rho = 1.0f / sqrtf(ss / static_cast<float>(D) + eps);
            float da = 0.0f, dot = 0.0f;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float gj = G[8 * nt + 2 * t + c];
                    const float yj = c ? yv[nt].y : yv[nt].x;
                    const float dcj = c ? sc[nt].y : sc[nt].x;
                    const float pre = yj * rho * gj;
                    const float cv = tanhf(a * pre);
                    const float dz = dcj * (1.0f - cv * cv);
                    da = fmaf(dz, pre, da);
                    const float dpre = a * dz;
                    dg[nt][c] = fmaf(dpre * yj, rho, dg[nt][c]);
                    const float scaled = dpre * gj;
                    dot = fmaf(yj, scaled, dot);
                    if (c) sc[nt].y = scaled;
                    else sc[nt].x = scaled;
                }
            }
            da = sum4_lanes(da);
            dot = sum4_lanes(dot);
            const float mean = dot / static_cast<float>(D);
            const float rho3 = rho * rho * rho;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                DYs[row * PW + 4 * nt + t] = pack_bf16(rho * sc[nt].x - rho3 * yv[nt].x * mean, rho * sc[nt].y - rho3 * yv[nt].y * mean);
            if (in && t == 0) d_alpha[p] = da;
        }
        __syncthreads();   // the tile and every row of d_y are in place
        {   // d_unit_out = d_y W_out on the warp's own rows
            float acc[NT][4];
            warp_product<D>(acc, DYs, Wt, r0, g, t);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t p = first + r0 + g + 8 * h;
                if (p < slots) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        *reinterpret_cast<uint32_t*>(d_unit_out + p * D + 8 * nt + 2 * t) = pack_bf16(acc[nt][2 * h], acc[nt][2 * h + 1]);
                }
            }
        }
        // d_W_out[j][k] += sum_p d_y[p][j] unit_out[p][k]: both operands are stored with p along the rows, so both
        // fragments come transposed; the warp's tiles share the rows 16 mt.. of d_W_out
        const uint16_t* dy16 = reinterpret_cast<const uint16_t*>(DYs);
        const uint16_t* x16 = reinterpret_cast<const uint16_t*>(Xs);
#pragma unroll 2
        for (int ks = 0; ks < kTileMma / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4_trans(a, dy16 + (16 * ks + (lane & 7) + 8 * (lane >> 4)) * PB + 16 * mt + 8 * ((lane >> 3) & 1));
#pragma unroll
            for (int i = 0; i < TPW; ++i) {
                const int at = warp + 8 * i;
                if (at < TILES) {
                    uint32_t b[2];
                    ldmatrix_x2_trans(b, x16 + (16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1)) * PB + 8 * (at / MT));
                    mma_bf16(dw[i], a, b[0], b[1]);
                }
            }
        }
    }
    float* mine = partial + static_cast<int64_t>(blockIdx.x) * (D * D + D);
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
        const int at = warp + 8 * i;
        if (at < TILES) {
            const int m = 16 * mt + g, n = 8 * (at / MT) + 2 * t;
            mine[m * D + n] = dw[i][0];
            mine[m * D + n + 1] = dw[i][1];
            mine[(m + 8) * D + n] = dw[i][2];
            mine[(m + 8) * D + n + 1] = dw[i][3];
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float v = dg[nt][c];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (g == 0) GS[warp * D + 8 * nt + 2 * t + c] = v;
        }
    }
    __syncthreads();
    for (int e = tid; e < D; e += kThreads) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) s += GS[r * D + e];
        mine[D * D + e] = s;
    }
}

// The blocks' shares added in a fixed order: eight threads an output take every eighth block, their sums meet in
// shared memory and are added in order.
template <bool BF>
__global__ void __launch_bounds__(kThreads)
k_tail_wgrad(const float* __restrict__ partial, int blocks, int d, float* __restrict__ d_w_out, float* __restrict__ d_gain) {
    __shared__ float part[8][32];
    const int outputs = d * d + d;
    const int lane = static_cast<int>(threadIdx.x) & 31, w = static_cast<int>(threadIdx.x) >> 5;
    const int e = static_cast<int>(blockIdx.x) * 32 + lane;
    float s = 0.0f;
    if (e < outputs) {
#pragma unroll 4
        for (int b = w; b < blocks; b += 8) s += __ldg(partial + static_cast<int64_t>(b) * outputs + e);
    }
    part[w][lane] = s;
    __syncthreads();
    if (w == 0 && e < outputs) {
        float total = part[0][lane];
#pragma unroll
        for (int r = 1; r < 8; ++r) total += part[r][lane];
        if (e < d * d) d_w_out[e] = maybe_bf16(total, BF);
        else d_gain[e - d * d] = total;
    }
}

int check(const HsnwTail* t, int64_t slots, const char* what) {
    if (!t || slots < 0) return hsnw_fail(HSNW_E_ARG, what);
    if (!t->w_out) return hsnw_fail(HSNW_E_ARG, "tail: null W_out");
    if (!t->norm_weight) return hsnw_fail(HSNW_E_ARG, "tail: the pass without the candidate norm is not taken here");
    if (t->d != 16 && t->d != 32 && t->d != 64 && t->d != 128) return hsnw_fail(HSNW_E_UNSUPPORTED, "tail: d must be 16, 32, 64 or 128");
    if (!(t->norm_eps >= 0.0f)) return hsnw_fail(HSNW_E_ARG, "tail: negative or NaN norm_eps");
    return HSNW_OK;
}

// The backward's blocks: at most two an SM (one at d = 128: registers and shared memory), every block the same number of tiles
// where the tiles allow it.
int64_t bwd_blocks(const HsnwTail* t, int64_t slots, int sms) {
    const int tile = t->prod_bf16 ? kTileMma : kTile;
    const int per_sm = t->d <= 64 ? 2 : 1;
    const int64_t tiles = std::max<int64_t>(1, (slots + tile - 1) / tile);
    const int64_t cap = static_cast<int64_t>(sms) * per_sm;
    const int64_t rounds = (tiles + cap - 1) / cap;
    return (tiles + rounds - 1) / rounds;
}

template <int D>
void launch_fwd(const HsnwTail* t, const void* unit_out, const float* alpha, int64_t slots, float* y, float* c, cudaStream_t stream) {
    if (t->prod_bf16) {
        const unsigned tiles = static_cast<unsigned>((slots + kTileMma - 1) / kTileMma);
        k_tail_fwd_mma<D><<<tiles, kThreads, MmaShape<D>::fwd_bytes, stream>>>(t->w_out, t->norm_weight, t->norm_eps,
                                                                             static_cast<const uint16_t*>(unit_out), alpha, slots, y, c);
    } else {
        const unsigned tiles = static_cast<unsigned>((slots + kTile - 1) / kTile);
        k_tail_fwd<D><<<tiles, kThreads, Shape<D>::fwd_bytes, stream>>>(t->w_out, t->norm_weight, t->norm_eps,
                                                                       static_cast<const float*>(unit_out), alpha, slots, y, c);
    }
}

template <int D>
void launch_bwd(const HsnwTail* t, const void* unit_out, const float* alpha, const float* y, const float* d_c, int64_t slots,
                void* d_unit_out, float* d_alpha, float* partial, int blocks, cudaStream_t stream) {
    if (t->prod_bf16)
        k_tail_bwd_mma<D><<<static_cast<unsigned>(blocks), kThreads, MmaShape<D>::bwd_bytes, stream>>>(
            t->w_out, t->norm_weight, t->norm_eps, static_cast<const uint16_t*>(unit_out), alpha, y, d_c, slots,
            static_cast<uint16_t*>(d_unit_out), d_alpha, partial);
    else
        k_tail_bwd<D><<<static_cast<unsigned>(blocks), kThreads, Shape<D>::bwd_bytes, stream>>>(
            t->w_out, t->norm_weight, t->norm_eps, static_cast<const float*>(unit_out), alpha, y, d_c, slots,
            static_cast<float*>(d_unit_out), d_alpha, partial);
}

}  // namespace

extern "C" int64_t hsnw_tail_scratch_bytes(const HsnwTail* tail, int64_t slots) {
    if (!tail || slots < 0 || tail->d < 16 || tail->d > 128) return 0;
    const int sms = std::max(148, hsnw_sm_count_current());
    const int64_t bytes = bwd_blocks(tail, slots, sms) * (static_cast<int64_t>(tail->d) * tail->d + tail->d) * static_cast<int64_t>(sizeof(float));
    return (bytes + 255) / 256 * 256;
}

extern "C" int hsnw_tail_forward(const HsnwTail* tail, const void* unit_out, const float* alpha, int64_t slots, float* y, float* c,
                                 void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(tail, slots, "tail_forward: null or negative")) return rc;
    if (slots == 0) return HSNW_OK;
    if (!unit_out || !alpha || !y || !c) return hsnw_fail(HSNW_E_ARG, "tail_forward: null tensor");
    if (reinterpret_cast<uintptr_t>(unit_out) % 16 || reinterpret_cast<uintptr_t>(y) % 8 || reinterpret_cast<uintptr_t>(c) % 8)
        return hsnw_fail(HSNW_E_ARG, "tail_forward: unit_out must be 16-byte aligned, y and c 8-byte");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    hsnw_profile_mark(HSNW_K_TAIL_FWD, stream);
#define HSNW_TAIL_FWD(D) \
    case D: \
        launch_fwd<D>(tail, unit_out, alpha, slots, y, c, stream); \
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
    if (reinterpret_cast<uintptr_t>(scratch) % 16 || reinterpret_cast<uintptr_t>(unit_out) % 16 || reinterpret_cast<uintptr_t>(y) % 8
        || reinterpret_cast<uintptr_t>(d_c) % 8 || reinterpret_cast<uintptr_t>(d_unit_out) % 4 || reinterpret_cast<uintptr_t>(tail->w_out) % 8)
        return hsnw_fail(HSNW_E_ARG, "tail_backward: scratch and unit_out must be 16-byte aligned, y, d_c and W_out 8-byte, d_unit_out 4-byte");
    const int blocks = static_cast<int>(bwd_blocks(tail, slots, std::max(1, hsnw_sm_count_current())));
    float* partial = static_cast<float*>(scratch);
    hsnw_profile_mark(HSNW_K_TAIL_BWD, stream);
#define HSNW_TAIL_BWD(D) \
    case D: \
        launch_bwd<D>(tail, unit_out, alpha, y, d_c, slots, d_unit_out, d_alpha, partial, blocks, stream); \
        break
    switch (d) {
        HSNW_TAIL_BWD(16);
        HSNW_TAIL_BWD(32);
        HSNW_TAIL_BWD(64);
        HSNW_TAIL_BWD(128);
    }
#undef HSNW_TAIL_BWD
    const unsigned out_blocks = static_cast<unsigned>((d * d + d + 31) / 32);
    if (tail->prod_bf16) k_tail_wgrad<true><<<out_blocks, kThreads, 0, stream>>>(partial, blocks, d, d_w_out, d_norm_weight);
    else k_tail_wgrad<false><<<out_blocks, kThreads, 0, stream>>>(partial, blocks, d, d_w_out, d_norm_weight);
    return hsnw_check_launch("tail_backward");
}

void hsnw_tail_set_attributes() {
    bool ok = true;
#define HSNW_TAIL_OPT(D) \
    ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_fwd<D>), "tail_fwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_fwd_mma<D>), "tail_fwd_mma") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_bwd<D>), "tail_bwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_tail_bwd_mma<D>), "tail_bwd_mma")
    HSNW_TAIL_OPT(16);
    HSNW_TAIL_OPT(32);
    HSNW_TAIL_OPT(64);
    HSNW_TAIL_OPT(128);
#undef HSNW_TAIL_OPT
    if (!ok) hsnw_attribute_failed();
}
