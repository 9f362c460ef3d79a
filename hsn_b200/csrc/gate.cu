// The cell norm and the gate of the replay's cell pass over every slot of a window at once, and their backward:
//   v = RMSNorm_w(v_raw), gate_pre = gate(v), b = sigmoid(gate_pre)       (reference python/hsn/model/cell.py:707-709)
// with autograd's gradients of v_raw, the norm's gain, the gate's weight and bias; the unit pass's gradient of v is an
// input of the backward. A slot's row of v_raw is 4 d floats (1 KB at d = 64) read once forward and, with the unit
// pass's gradient, once more backward; v and d_v_raw are written once: the pass is bound by those four tensors
// (forward 32 d + 8 d + 4 bytes a slot, backward 48 d + 8 d), the gate's product is 8 d^2 flops a slot.
//
// A block takes tiles of 128 slots forward (a warp 16 of them) and of 64 backward (two blocks an SM). Everything
// row-wise (the norm and its backward, sigmoid) runs with a warp on one row at a time and a lane on 4 consecutive
// features per 128, so global accesses are whole rows, streamed; the products run on warp-level tensor-core tiles
// (mma_tiles.cuh) from bf16 copies in shared memory of the tile and of the gate's weight, which every block converts
// as it stages it (read through L1 from global memory, the products' B fragments took a third of the forward's time).
// Backward, per tile: v and d_gate_pre into shared memory; d_W_gate += d_gate_pre^T v (both read transposed, a warp
// keeps d * 4 d / 1024 accumulator tiles over all of the block's tiles); d_gate_pre W_gate (a warp 16 rows x half the
// columns), written as bf16 over those rows of v (that sum IS a bf16 value in the reference); then the norm's backward
// row by row. Blocks write their shares of the three parameter gradients once, a last kernel adds them in a fixed
// order.
#include "../../include/hsn_gate_b200.h"
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "host_util.h"
#include "mma_tiles.cuh"

#include <algorithm>
#include <cstdint>

namespace {
using namespace hsnw;

constexpr int kThreads = 256;
constexpr int kTile = 128;      // slots a tile of the forward: a warp 16 of them
constexpr int kTileB = 64;      // of the backward: 8 rows a warp in the row-wise phases, 16 rows x half the columns in the product
constexpr int kRowsAtOnce = 4;

template <int D>
struct GateShape {
    static constexpr int F = 4 * D;
    static constexpr int PBF = F + 8, PWF = PBF / 2;   // pitch of a row of F bf16 values, in elements and in words
    static constexpr int PBD = D + 8, PWD = PBD / 2;
    static constexpr int NT = D / 8, NTF = F / 8;      // 8-column tiles of a row of d, of 4 d
    static constexpr int KSD = D / 16, KSF = F / 16;   // 16-deep steps over d, over 4 d
    static constexpr int MT = D / 16;                  // 16-row tiles of d_W_gate
    static constexpr int TILES = MT * NTF;
    static constexpr int TPW = (TILES + 7) / 8;        // d_W_gate tiles a warp
    static constexpr int LV = (F + 127) / 128;         // groups of 4 features a lane
    static constexpr int OUTPUTS = D * F + F + D;      // a block's shares: d_W_gate, the gain's gradient, d_b_gate
    static constexpr size_t fwd_bytes = sizeof(uint32_t) * (kTile * PWF + D * PWF) + sizeof(float) * (F + D);
    static constexpr size_t bwd_bytes = sizeof(uint32_t) * (kTileB * PWF + kTileB * PWD + F * PWD) + sizeof(float) * (F + kTileB + 8 * (F + D));
};

__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The slots' rows are read once: streaming loads and stores (evict first), so that the gate's packed weight, which
// every product step reads through L1, stays there.
__device__ __forceinline__ float4 ld4_or_zero(const float* base, bool on) {
    return on ? __ldcs(reinterpret_cast<const float4*>(base)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

template <int D>
__global__ void __launch_bounds__(kThreads)
k_gate_fwd(const float* __restrict__ gate_w, const float* __restrict__ norm_w, const float* __restrict__ gate_b, float eps,
           const float* __restrict__ v_raw, int64_t slots, float* __restrict__ v_out, float* __restrict__ rms_out,
           float* __restrict__ gp_out, float* __restrict__ b_out) {
    using S = GateShape<D>;
    constexpr int F = S::F, PWF = S::PWF, NT = S::NT, KSF = S::KSF, LV = S::LV;
    extern __shared__ __align__(16) uint32_t smem_w[];
    uint32_t* Vs = smem_w;                                          // [kTile][PWF] v as bf16
    uint32_t* Ws = Vs + kTile * PWF;                                // [D][PWF] W_gate[j][f] as bf16
    float* NW = reinterpret_cast<float*>(Ws + D * PWF);             // [F]
    float* GB = NW + F;                                             // [D] the bias as bf16 values
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kTile;
    for (int e = tid; e < D * (F / 4); e += kThreads) {   // four weights at a time
        const int j = e / (F / 4), q = e - j * (F / 4);
        const float4 w4 = __ldg(reinterpret_cast<const float4*>(gate_w) + e);
        *reinterpret_cast<uint2*>(Ws + j * PWF + 2 * q) = make_uint2(pack_bf16(w4.x, w4.y), pack_bf16(w4.z, w4.w));
    }
    for (int e = tid; e < F; e += kThreads) NW[e] = __ldg(norm_w + e);
    for (int e = tid; e < D; e += kThreads) GB[e] = bf16r(__ldg(gate_b + e));
    __syncthreads();
    const int r0 = warp * 16;
    for (int rr = 0; rr < 16; rr += kRowsAtOnce) {
        float4 x[kRowsAtOnce][LV];
#pragma unroll
        for (int q = 0; q < kRowsAtOnce; ++q) {
            const int64_t p = first + r0 + rr + q;
#pragma unroll
            for (int i = 0; i < LV; ++i) {
                const int f = 4 * lane + 128 * i;
                x[q][i] = ld4_or_zero(v_raw + p * F + f, p < slots && f < F);
            }
        }
#pragma unroll
        for (int q = 0; q < kRowsAtOnce; ++q) {
            const int row = r0 + rr + q;
            const int64_t p = first + row;
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < LV; ++i) ss += x[q][i].x * x[q][i].x + x[q][i].y * x[q][i].y + x[q][i].z * x[q][i].z + x[q][i].w * x[q][i].w;
            ss = warp_total(ss);
            const float rms = 1.0f / sqrtf(ss / static_cast<float>(F) + eps);
#pragma unroll
            for (int i = 0; i < LV; ++i) {
                const int f = 4 * lane + 128 * i;
                if (f < F) {
                    const float4 nw = *reinterpret_cast<const float4*>(NW + f);
                    const float4 v = make_float4(x[q][i].x * rms * nw.x, x[q][i].y * rms * nw.y, x[q][i].z * rms * nw.z, x[q][i].w * rms * nw.w);
                    if (p < slots) __stcs(reinterpret_cast<float4*>(v_out + p * F + f), v);
                    *reinterpret_cast<uint2*>(Vs + row * PWF + f / 2) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
                }
            }
            if (lane == 0 && p < slots) rms_out[p] = rms;
        }
    }
    __syncwarp();
    // gate_pre on the warp's 16 rows: A = v (K = 4 d), B(k = f, n = j) = W_gate[j][f] read as packed pairs along f
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
#pragma unroll 2
    for (int ks = 0; ks < KSF; ++ks) {
        uint32_t a[4];
        a[0] = Vs[(r0 + g) * PWF + 8 * ks + t];
        a[1] = Vs[(r0 + g + 8) * PWF + 8 * ks + t];
        a[2] = Vs[(r0 + g) * PWF + 8 * ks + 4 + t];
        a[3] = Vs[(r0 + g + 8) * PWF + 8 * ks + 4 + t];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t b0 = Ws[(8 * nt + g) * PWF + 8 * ks + t];
            const uint32_t b1 = Ws[(8 * nt + g) * PWF + 8 * ks + 4 + t];
            mma_bf16(acc[nt], a, b0, b1);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int64_t p = first + r0 + g + 8 * h;
        if (p < slots) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int j = 8 * nt + 2 * t;
                const float g0 = bf16r(acc[nt][2 * h] + GB[j]), g1 = bf16r(acc[nt][2 * h + 1] + GB[j + 1]);
                *reinterpret_cast<float2*>(gp_out + p * D + j) = make_float2(g0, g1);
                *reinterpret_cast<float2*>(b_out + p * D + j) = make_float2(sigmoid_f(g0), sigmoid_f(g1));
            }
        }
    }
}

// `partial` [blocks][D F + F + D]: the block's shares of d_W_gate, of the gain's gradient and of d_b_gate.
template <int D>
__global__ void __launch_bounds__(kThreads, 2)   // two blocks an SM: the d_W_gate accumulators leave the registers between products
k_gate_bwd(const float* __restrict__ gate_w, const float* __restrict__ norm_w, float eps, const float* __restrict__ v_raw,
           const float* __restrict__ gate_pre, const float* __restrict__ d_v_units, const float* __restrict__ d_b, int64_t slots,
           float* __restrict__ d_v_raw, float* __restrict__ partial) {
    using S = GateShape<D>;
    constexpr int F = S::F, PBF = S::PBF, PWF = S::PWF, PBD = S::PBD, PWD = S::PWD, NTF = S::NTF, KSD = S::KSD, MT = S::MT,
                  TILES = S::TILES, TPW = S::TPW, LV = S::LV;
    extern __shared__ __align__(16) uint32_t smem_w[];
    uint32_t* Vs = smem_w;                                          // [kTileB][PWF] v as bf16, then d_gate_pre W_gate as bf16
    uint32_t* DGs = Vs + kTileB * PWF;                              // [kTileB][PWD] d_gate_pre as bf16
    uint32_t* WT = DGs + kTileB * PWD;                               // [F][PWD] WT[f][j] = W_gate[j][f] as bf16
    float* NW = reinterpret_cast<float*>(WT + F * PWD);             // [F]
    float* RMS = NW + F;                                            // [kTileB]
    float* RS = RMS + kTileB;                                        // [8][F + D] the warps' shares at the end
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    for (int e = tid; e < (D / 2) * F; e += kThreads) {   // a pair of the gate's rows at a time, f along the lanes
        const int j2 = e / F, f = e - j2 * F;
        WT[f * PWD + j2] = pack_bf16(__ldg(gate_w + (2 * j2) * F + f), __ldg(gate_w + (2 * j2 + 1) * F + f));
    }
    for (int e = tid; e < F; e += kThreads) NW[e] = __ldg(norm_w + e);
    float dw[TPW][4];
    float4 dnw[LV];
    float2 dbg = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) dw[i][c] = 0.0f;
#pragma unroll
    for (int i = 0; i < LV; ++i) dnw[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    constexpr int RW = kTileB / 8;            // rows a warp in the row-wise phases
    const int r0 = warp * RW;
    const int rm = (warp & 3) * 16;           // the warp's 16 rows in the product of phase (c)
    const int nt0 = (warp >> 2) * (NTF / 2);  // and its half of the columns
    const int mt = warp % MT;
    const bool has_j = 2 * lane < D;   // the lane's pair of gate columns
    const int64_t tiles = (slots + kTileB - 1) / kTileB;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t first = tile * kTileB;
        __syncthreads();   // the previous tile's reads are over; the gain is in place
        // (a) v and d_gate_pre of the warp's rows, as bf16 in shared memory
        for (int rr = 0; rr < RW; rr += kRowsAtOnce) {
            float4 x[kRowsAtOnce][LV];
            float2 gp[kRowsAtOnce], db[kRowsAtOnce];
#pragma unroll
            for (int q = 0; q < kRowsAtOnce; ++q) {
                const int64_t p = first + r0 + rr + q;
#pragma unroll
                for (int i = 0; i < LV; ++i) {
                    const int f = 4 * lane + 128 * i;
                    x[q][i] = ld4_or_zero(v_raw + p * F + f, p < slots && f < F);
                }
                const bool on = has_j && p < slots;
                gp[q] = on ? __ldg(reinterpret_cast<const float2*>(gate_pre + p * D) + lane) : make_float2(0.0f, 0.0f);
                db[q] = on ? __ldg(reinterpret_cast<const float2*>(d_b + p * D) + lane) : make_float2(0.0f, 0.0f);
            }
#pragma unroll
            for (int q = 0; q < kRowsAtOnce; ++q) {
                const int row = r0 + rr + q;
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < LV; ++i) ss += x[q][i].x * x[q][i].x + x[q][i].y * x[q][i].y + x[q][i].z * x[q][i].z + x[q][i].w * x[q][i].w;
                ss = warp_total(ss);
                const float rms = 1.0f / sqrtf(ss / static_cast<float>(F) + eps);
                if (lane == 0) RMS[row] = rms;
#pragma unroll
                for (int i = 0; i < LV; ++i) {
                    const int f = 4 * lane + 128 * i;
                    if (f < F) {
                        const float4 nw = *reinterpret_cast<const float4*>(NW + f);
                        *reinterpret_cast<uint2*>(Vs + row * PWF + f / 2) =
                            make_uint2(pack_bf16(x[q][i].x * rms * nw.x, x[q][i].y * rms * nw.y), pack_bf16(x[q][i].z * rms * nw.z, x[q][i].w * rms * nw.w));
                    }
                }
                if (has_j) {
                    const float b0 = sigmoid_f(gp[q].x), b1 = sigmoid_f(gp[q].y);
                    const float g0 = bf16r(db[q].x * b0 * (1.0f - b0)), g1 = bf16r(db[q].y * b1 * (1.0f - b1));
                    dbg.x += g0;
                    dbg.y += g1;
                    DGs[row * PWD + lane] = pack_bf16(g0, g1);
                }
            }
        }
        __syncthreads();
        // (b) d_W_gate[j][f] += sum_p d_gate_pre[p][j] v[p][f]: both operands hold p along their rows, so both come transposed
        {
            const uint16_t* dg16 = reinterpret_cast<const uint16_t*>(DGs);
            const uint16_t* v16 = reinterpret_cast<const uint16_t*>(Vs);
#pragma unroll 1
            for (int ks = 0; ks < kTileB / 16; ++ks) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, dg16 + (16 * ks + (lane & 7) + 8 * (lane >> 4)) * PBD + 16 * mt + 8 * ((lane >> 3) & 1));
#pragma unroll
                for (int i = 0; i < TPW; ++i) {
                    const int at = warp + 8 * i;
                    if (at < TILES) {
                        uint32_t b[2];
                        ldmatrix_x2_trans(b, v16 + (16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1)) * PBF + 8 * (at / MT));
                        mma_bf16(dw[i], a, b[0], b[1]);
                    }
                }
            }
        }
        __syncthreads();   // every warp has read every row of v: the rows can be overwritten
        // (c) d_gate_pre W_gate (K = d, N = 4 d) on 16 rows x half the columns a warp, rounded to bf16 over those rows of v
        {
            uint32_t a[KSD][4];
#pragma unroll
            for (int ks = 0; ks < KSD; ++ks) {
                a[ks][0] = DGs[(rm + g) * PWD + 8 * ks + t];
                a[ks][1] = DGs[(rm + g + 8) * PWD + 8 * ks + t];
                a[ks][2] = DGs[(rm + g) * PWD + 8 * ks + 4 + t];
                a[ks][3] = DGs[(rm + g + 8) * PWD + 8 * ks + 4 + t];
            }
#pragma unroll 4
            for (int nt = nt0; nt < nt0 + NTF / 2; ++nt) {
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int ks = 0; ks < KSD; ++ks) {
                    const uint32_t b0 = WT[(8 * nt + g) * PWD + 8 * ks + t];
                    const uint32_t b1 = WT[(8 * nt + g) * PWD + 8 * ks + 4 + t];
                    mma_bf16(acc, a[ks], b0, b1);
                }
                Vs[(rm + g) * PWF + 4 * nt + t] = pack_bf16(acc[0], acc[1]);
                Vs[(rm + g + 8) * PWF + 4 * nt + t] = pack_bf16(acc[2], acc[3]);
            }
        }
        __syncthreads();   // a row's columns came from two warps
        // (d) the norm's backward, a row at a time
        for (int rr = 0; rr < RW; rr += kRowsAtOnce) {
            float4 x[kRowsAtOnce][LV], dv[kRowsAtOnce][LV];
#pragma unroll
            for (int q = 0; q < kRowsAtOnce; ++q) {
                const int64_t p = first + r0 + rr + q;
#pragma unroll
                for (int i = 0; i < LV; ++i) {
                    const int f = 4 * lane + 128 * i;
                    x[q][i] = ld4_or_zero(v_raw + p * F + f, p < slots && f < F);
                    dv[q][i] = ld4_or_zero(d_v_units + p * F + f, p < slots && f < F);
                }
            }
#pragma unroll
            for (int q = 0; q < kRowsAtOnce; ++q) {
                const int row = r0 + rr + q;
                const int64_t p = first + row;
                const float rms = RMS[row];
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < LV; ++i) {
                    const int f = 4 * lane + 128 * i;
                    if (f < F) {
                        const uint2 gw = *reinterpret_cast<const uint2*>(Vs + row * PWF + f / 2);
                        const float4 nw = *reinterpret_cast<const float4*>(NW + f);
                        float4& d = dv[q][i];
                        d.x += bf16_value(static_cast<uint16_t>(gw.x & 0xffffu));
                        d.y += bf16_value(static_cast<uint16_t>(gw.x >> 16));
                        d.z += bf16_value(static_cast<uint16_t>(gw.y & 0xffffu));
                        d.w += bf16_value(static_cast<uint16_t>(gw.y >> 16));
                        const float4 xi = x[q][i];
                        dnw[i].x = fmaf(d.x * xi.x, rms, dnw[i].x);
                        dnw[i].y = fmaf(d.y * xi.y, rms, dnw[i].y);
                        dnw[i].z = fmaf(d.z * xi.z, rms, dnw[i].z);
                        dnw[i].w = fmaf(d.w * xi.w, rms, dnw[i].w);
                        d = make_float4(d.x * nw.x, d.y * nw.y, d.z * nw.z, d.w * nw.w);   // w d_v
                        dot += xi.x * d.x + xi.y * d.y + xi.z * d.z + xi.w * d.w;
                    }
                }
                dot = warp_total(dot);
                const float mean = dot / static_cast<float>(F);
                const float rms3 = rms * rms * rms;
                if (p < slots) {
#pragma unroll
                    for (int i = 0; i < LV; ++i) {
                        const int f = 4 * lane + 128 * i;
                        if (f < F) {
                            const float4 xi = x[q][i], d = dv[q][i];
                            __stcs(reinterpret_cast<float4*>(d_v_raw + p * F + f),
                                   make_float4(rms * d.x - rms3 * xi.x * mean, rms * d.y - rms3 * xi.y * mean, rms * d.z - rms3 * xi.z * mean,
                                               rms * d.w - rms3 * xi.w * mean));
                        }
                    }
                }
            }
        }
    }
    float* mine = partial + static_cast<int64_t>(blockIdx.x) * S::OUTPUTS;
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
        const int at = warp + 8 * i;
        if (at < TILES) {
            const int m = 16 * mt + g, n = 8 * (at / MT) + 2 * t;
            mine[m * F + n] = dw[i][0];
            mine[m * F + n + 1] = dw[i][1];
            mine[(m + 8) * F + n] = dw[i][2];
            mine[(m + 8) * F + n + 1] = dw[i][3];
        }
    }
    __syncthreads();   // the last tile's shared memory is free
#pragma unroll
    for (int i = 0; i < LV; ++i) {
        const int f = 4 * lane + 128 * i;
        if (f < F) *reinterpret_cast<float4*>(RS + warp * (F + D) + f) = dnw[i];
    }
    if (has_j) *reinterpret_cast<float2*>(RS + warp * (F + D) + F + 2 * lane) = dbg;
    __syncthreads();
    for (int e = tid; e < F + D; e += kThreads) {
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) s += RS[r * (F + D) + e];
        mine[D * F + e] = s;
    }
}

// The blocks' shares added in a fixed order: eight threads an output take every eighth block, their sums meet in
// shared memory and are added in order. d_W_gate and d_b_gate are bf16 values, the gain's gradient is float32.
__global__ void __launch_bounds__(kThreads)
k_gate_wgrad(const float* __restrict__ partial, int blocks, int d, float* __restrict__ d_gate_w, float* __restrict__ d_norm_w,
             float* __restrict__ d_gate_b) {
    __shared__ float part[8][32];
    const int F = 4 * d, outputs = d * F + F + d;
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
        if (e < d * F) d_gate_w[e] = bf16r(total);
        else if (e < d * F + F) d_norm_w[e - d * F] = total;
        else d_gate_b[e - d * F - F] = bf16r(total);
    }
}

int check(const HsnwGate* s, int64_t slots, const char* what) {
    if (!s || slots < 0) return hsnw_fail(HSNW_E_ARG, what);
    if (!s->norm_weight || !s->gate_w || !s->gate_b) return hsnw_fail(HSNW_E_ARG, "gate: null weight");
    if (!s->prod_bf16) return hsnw_fail(HSNW_E_UNSUPPORTED, "gate: float32 products are not taken here");
    if (s->d != 16 && s->d != 32 && s->d != 64) return hsnw_fail(HSNW_E_UNSUPPORTED, "gate: d must be 16, 32 or 64");
    if (!(s->norm_eps >= 0.0f)) return hsnw_fail(HSNW_E_ARG, "gate: negative or NaN norm_eps");
    if (reinterpret_cast<uintptr_t>(s->gate_w) % 16) return hsnw_fail(HSNW_E_ARG, "gate: the weight must be 16-byte aligned");
    return HSNW_OK;
}

int64_t outputs_of(int d) { return static_cast<int64_t>(d) * 4 * d + 4 * d + d; }

// The backward's blocks: two an SM, every block the same number of tiles where the tiles allow it.
int64_t bwd_blocks(int d, int64_t slots, int sms) {
    const int64_t tiles = std::max<int64_t>(1, (slots + kTileB - 1) / kTileB);
    const int64_t cap = static_cast<int64_t>(sms) * 2;
    (void)d;
    const int64_t rounds = (tiles + cap - 1) / cap;
    return (tiles + rounds - 1) / rounds;
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

extern "C" int64_t hsnw_gate_scratch_bytes(const HsnwGate* gate, int64_t slots, int backward) {
    if (!gate || slots < 0 || gate->d < 16 || gate->d > 64) return 0;
    if (!backward) return 256;   // the forward keeps nothing between its launches
    const int sms = std::max(148, hsnw_sm_count_current());
    return (bwd_blocks(gate->d, slots, sms) * outputs_of(gate->d) * static_cast<int64_t>(sizeof(float)) + 255) / 256 * 256;
}

extern "C" int hsnw_gate_forward(const HsnwGate* gate, const float* v_raw, int64_t slots, float* v, float* rms, float* gate_pre, float* b,
                                 void* scratch, int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(gate, slots, "gate_forward: null or negative")) return rc;
    if (slots == 0) return HSNW_OK;
    if (!v_raw || !v || !rms || !gate_pre || !b) return hsnw_fail(HSNW_E_ARG, "gate_forward: null tensor");
    if (!scratch || scratch_bytes < hsnw_gate_scratch_bytes(gate, slots, 0)) return hsnw_fail(HSNW_E_ARG, "gate_forward: scratch too small");
    if (!aligned16(v_raw) || !aligned16(v) || !aligned16(scratch) || reinterpret_cast<uintptr_t>(gate_pre) % 8 || reinterpret_cast<uintptr_t>(b) % 8)
        return hsnw_fail(HSNW_E_ARG, "gate_forward: v_raw, v and scratch must be 16-byte aligned, gate_pre and b 8-byte");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int d = gate->d;
    hsnw_profile_mark(HSNW_K_GATE_FWD, stream);
    const unsigned tiles = static_cast<unsigned>((slots + kTile - 1) / kTile);
#define HSNW_GATE_FWD(D) \
    case D: \
        k_gate_fwd<D><<<tiles, kThreads, GateShape<D>::fwd_bytes, stream>>>(gate->gate_w, gate->norm_weight, gate->gate_b, gate->norm_eps, v_raw, slots, \
                                                                          v, rms, gate_pre, b); \
        break
    switch (d) {
        HSNW_GATE_FWD(16);
        HSNW_GATE_FWD(32);
        HSNW_GATE_FWD(64);
    }
#undef HSNW_GATE_FWD
    return hsnw_check_launch("gate_forward");
}

extern "C" int hsnw_gate_backward(const HsnwGate* gate, const float* v_raw, const float* gate_pre, const float* d_v_units, const float* d_b,
                                  int64_t slots, float* d_v_raw, float* d_norm_weight, float* d_gate_w, float* d_gate_b,
                                  void* scratch, int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(gate, slots, "gate_backward: null or negative")) return rc;
    if (!d_norm_weight || !d_gate_w || !d_gate_b) return hsnw_fail(HSNW_E_ARG, "gate_backward: null gradient");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int d = gate->d;
    if (slots == 0) {
        if (cudaMemsetAsync(d_gate_w, 0, sizeof(float) * d * 4 * d, stream) != cudaSuccess
            || cudaMemsetAsync(d_norm_weight, 0, sizeof(float) * 4 * d, stream) != cudaSuccess
            || cudaMemsetAsync(d_gate_b, 0, sizeof(float) * d, stream) != cudaSuccess)
            return hsnw_check_launch("gate_backward");
        return HSNW_OK;
    }
    if (!v_raw || !gate_pre || !d_v_units || !d_b || !d_v_raw) return hsnw_fail(HSNW_E_ARG, "gate_backward: null tensor");
    if (!scratch || scratch_bytes < hsnw_gate_scratch_bytes(gate, slots, 1)) return hsnw_fail(HSNW_E_ARG, "gate_backward: scratch too small");
    if (!aligned16(v_raw) || !aligned16(d_v_units) || !aligned16(d_v_raw) || !aligned16(scratch) || reinterpret_cast<uintptr_t>(gate_pre) % 8
        || reinterpret_cast<uintptr_t>(d_b) % 8)
        return hsnw_fail(HSNW_E_ARG, "gate_backward: v_raw, d_v_units, d_v_raw and scratch must be 16-byte aligned, gate_pre and d_b 8-byte");
    float* partial = static_cast<float*>(scratch);
    const int blocks = static_cast<int>(bwd_blocks(d, slots, std::max(1, hsnw_sm_count_current())));
    hsnw_profile_mark(HSNW_K_GATE_BWD, stream);
#define HSNW_GATE_BWD(D) \
    case D: \
        k_gate_bwd<D><<<static_cast<unsigned>(blocks), kThreads, GateShape<D>::bwd_bytes, stream>>>( \
            gate->gate_w, gate->norm_weight, gate->norm_eps, v_raw, gate_pre, d_v_units, d_b, slots, d_v_raw, partial); \
        break
    switch (d) {
        HSNW_GATE_BWD(16);
        HSNW_GATE_BWD(32);
        HSNW_GATE_BWD(64);
    }
#undef HSNW_GATE_BWD
    const unsigned out_blocks = static_cast<unsigned>((outputs_of(d) + 31) / 32);
    k_gate_wgrad<<<out_blocks, kThreads, 0, stream>>>(partial, blocks, d, d_gate_w, d_norm_weight, d_gate_b);
    return hsnw_check_launch("gate_backward");
}

void hsnw_gate_set_attributes() {
    bool ok = true;
#define HSNW_GATE_OPT(D) \
    ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_gate_fwd<D>), "gate_fwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_gate_bwd<D>), "gate_bwd")
    HSNW_GATE_OPT(16);
    HSNW_GATE_OPT(32);
    HSNW_GATE_OPT(64);
#undef HSNW_GATE_OPT
    if (!ok) hsnw_attribute_failed();
}
