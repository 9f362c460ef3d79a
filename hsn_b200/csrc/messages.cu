// The messages and the gathered inputs of the replay's cell pass over every slot of a window at once, and their
// backward:  sources_j = V(h[src_j]), m = sum_j w_j sources_j, v_raw = [u; eps; h[cell]; m]
// (reference python/hsn/model/cell.py:698-705) with autograd's gradients of u, eps, V and the padded edge weights; the
// state is a constant of the replay. A slot reads its cell's row and the rows of up to four in-neighbours from the
// recorded state (256 bytes each at d = 64, wherever the router sent it) and writes 4 d floats: the pass is bound by
// those rows and by v_raw (forward 4 d (degree + 1) + 8 + 16 d bytes a slot, backward 4 d degree + 8 + 16 d), V's
// product is 2 d^2 flops a neighbour.
//
// A block takes tiles of 32 slots = 128 (slot, neighbour) rows, gathered as bf16 into shared memory; a warp owns 16
// rows = 4 slots, V's product is a warp-level tensor-core tile (mma_tiles.cuh) and the weighted sum over a slot's four
// neighbours two shuffles between the lanes that hold them. Backward, per tile: the sources again (cheaper than a
// record), each row's <d_m, sources_j> to a per-slot buffer, w_j d_m as a bf16 tile, and d_V += (w d_m)^T h[src] with
// both operands read transposed, a warp keeping its tiles of d_V over all of the block's tiles. The edge weights'
// gradient is a sum over the slots of each cell: every block keeps a table [n_cells][4] in shared memory that four
// lanes fill in slot order, and the blocks' tables are added in block order (no atomics: the same bits every run; a
// graph of more than 2048 cells takes a scan per cell instead); d_u and d_eps are sums over a row's k slots.
#include "../../include/hsn_messages_b200.h"
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "host_util.h"
#include "mma_tiles.cuh"

#include <algorithm>
#include <cstdint>

namespace {
using namespace hsnw;

constexpr int kThreads = 256;
constexpr int kSlots = 32;           // slots a tile
constexpr int kRows = 4 * kSlots;    // (slot, neighbour) rows a tile: a warp 16 of them

template <int D>
struct MsgShape {
    static constexpr int PB = D + 8, PW = PB / 2;
    static constexpr int NT = D / 8, KS = D / 16, MT = D / 16;
    static constexpr int TILES = MT * NT;
    static constexpr int TPW = (TILES + 7) / 8;
    static constexpr size_t fwd_bytes = sizeof(uint32_t) * (kRows * PW + D * PW) + sizeof(float) * kRows + sizeof(int64_t) * kRows;
    static constexpr size_t bwd_bytes = sizeof(uint32_t) * (2 * kRows * PW + D * PW) + sizeof(float) * (kRows + kSlots * D + kRows) + sizeof(int) * kSlots
                                        + sizeof(int64_t) * kRows;   // (+ the table [n_cells][4] with FOLD)
};

struct Graph {
    const float* edge_w;
    const int64_t* pad_src;
    int n_cells, degree, k;
};

// V as bf16 pairs, Ws[o][e / 2].
template <int D>
__device__ __forceinline__ void stage_weight(uint32_t* Ws, const float* v_w, int tid) {
    for (int e = tid; e < D * D / 2; e += kThreads) {
        const int o = e / (D / 2), k2 = e - o * (D / 2);
        const float2 v = __ldg(reinterpret_cast<const float2*>(v_w) + e);
        Ws[o * MsgShape<D>::PW + k2] = pack_bf16(v.x, v.y);
    }
}

// The tile's rows: row 4 s + j is neighbour j of slot s. SRC: the row's offset in h (in floats), -1 for none; WE: its
// weight as a bf16 value; Hs: the gathered rows as bf16. Ends with a block barrier.
template <int D>
__device__ __forceinline__ void stage_tile(uint32_t* Hs, int64_t* SRC, float* WE, const Graph& gr, const float* h, const int64_t* cells,
                                           int64_t first, int64_t slots, int tid) {
    constexpr int PW = MsgShape<D>::PW;
    if (tid < kRows) {
        const int s = tid >> 2, j = tid & 3;
        const int64_t p = first + s;
        int64_t off = -1;
        float w = 0.0f;
        if (p < slots && j < gr.degree) {
            const int64_t r = p / gr.k, n = __ldg(cells + p);
            off = (r * gr.n_cells + __ldg(gr.pad_src + n * gr.degree + j)) * D;
            w = bf16r(__ldg(gr.edge_w + n * gr.degree + j));
        }
        SRC[tid] = off;
        WE[tid] = w;
    }
    __syncthreads();
    for (int e = tid; e < kRows * (D / 4); e += kThreads) {
        const int row = e / (D / 4), q = e - row * (D / 4);
        const int64_t off = SRC[row];
        const float4 v = off >= 0 ? __ldg(reinterpret_cast<const float4*>(h + off) + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        *reinterpret_cast<uint2*>(Hs + row * PW + 2 * q) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    }
    __syncthreads();
}

template <int D>
__global__ void __launch_bounds__(kThreads)
k_msg_fwd(const float* __restrict__ v_w, Graph gr, const float* __restrict__ u, const float* __restrict__ eps, const float* __restrict__ h,
          const int64_t* __restrict__ cells, int64_t slots, float* __restrict__ v_raw) {
    using S = MsgShape<D>;
    constexpr int PW = S::PW, NT = S::NT, KS = S::KS;
    extern __shared__ __align__(16) uint32_t smem_w[];
    uint32_t* Hs = smem_w;                                        // [kRows][PW]
    uint32_t* Ws = Hs + kRows * PW;                               // [D][PW]
    int64_t* SRC = reinterpret_cast<int64_t*>(Ws + D * PW);       // [kRows]
    float* WE = reinterpret_cast<float*>(SRC + kRows);            // [kRows]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kSlots;
    stage_weight<D>(Ws, v_w, tid);
    stage_tile<D>(Hs, SRC, WE, gr, h, cells, first, slots, tid);
    // [u; eps; h[cell]] of the tile's slots, 16 bytes at a time
    for (int e = tid; e < kSlots * (3 * D / 4); e += kThreads) {
        const int s = e / (3 * D / 4), q = e - s * (3 * D / 4);
        const int64_t p = first + s;
        if (p < slots) {
            const int seg = q / (D / 4), qq = q - seg * (D / 4);
            const int64_t r = p / gr.k;
            const float* from = seg == 0 ? u + r * D : seg == 1 ? eps + r * D : h + (r * gr.n_cells + __ldg(cells + p)) * D;
            __stcs(reinterpret_cast<float4*>(v_raw + p * 4 * D + seg * D) + qq, __ldg(reinterpret_cast<const float4*>(from) + qq));
        }
    }
    float acc[NT][4];
    const int r0 = warp * 16;
    warp_rows_product<NT, KS, PW, PW>(acc, Hs, Ws, r0, g, t);
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = r0 + g + 8 * h2;
        const float w = WE[row];
        const int64_t p = first + (row >> 2);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float m0 = bf16r(bf16r(acc[nt][2 * h2]) * w), m1 = bf16r(bf16r(acc[nt][2 * h2 + 1]) * w);
            m0 += __shfl_xor_sync(0xffffffffu, m0, 4);   // the slot's four neighbours sit in the lanes g, g ^ 1, g ^ 2, g ^ 3
            m1 += __shfl_xor_sync(0xffffffffu, m1, 4);
            m0 += __shfl_xor_sync(0xffffffffu, m0, 8);
            m1 += __shfl_xor_sync(0xffffffffu, m1, 8);
            if ((g & 3) == 0 && p < slots)
                __stcs(reinterpret_cast<float2*>(v_raw + p * 4 * D + 3 * D + 8 * nt + 2 * t), make_float2(bf16r(m0), bf16r(m1)));
        }
    }
}

// `partial` [blocks][D D]: the block's share of d_V. The rows' <d_m, sources_j> go, with FOLD, into the block's own
// table [n_cells][4] in shared memory (four lanes, one a neighbour, add a tile's 32 slots in slot order while the other
// warps multiply) and from there to `edges` [blocks][n_cells][4]; without (a graph too large for the table) to `edges`
// [slots][4], which a scan per cell sums.
template <int D, bool FOLD>
__global__ void __launch_bounds__(kThreads)
k_msg_bwd(const float* __restrict__ v_w, Graph gr, const float* __restrict__ h, const int64_t* __restrict__ cells,
          const float* __restrict__ d_v_raw, int64_t slots, float* __restrict__ edges, float* __restrict__ partial) {
    using S = MsgShape<D>;
    constexpr int PB = S::PB, PW = S::PW, NT = S::NT, KS = S::KS, MT = S::MT, TILES = S::TILES, TPW = S::TPW;
    extern __shared__ __align__(16) uint32_t smem_w[];
    uint32_t* Hs = smem_w;                                        // [kRows][PW] h[src]
    uint32_t* DS = Hs + kRows * PW;                               // [kRows][PW] w_j d_m
    uint32_t* Ws = DS + kRows * PW;                               // [D][PW]
    int64_t* SRC = reinterpret_cast<int64_t*>(Ws + D * PW);       // [kRows]
    float* WE = reinterpret_cast<float*>(SRC + kRows);            // [kRows]
    float* DM = WE + kRows;                                       // [kSlots][D] d_m as bf16 values
    float* ROWV = DM + kSlots * D;                                // [kRows] <d_m, sources_j> of the tile's rows
    int* CELL = reinterpret_cast<int*>(ROWV + kRows);             // [kSlots] the tile's cells, -1 beyond the last slot
    float* ACC = reinterpret_cast<float*>(CELL + kSlots);         // [n_cells][4] (FOLD)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    stage_weight<D>(Ws, v_w, tid);
    if constexpr (FOLD)
        for (int e = tid; e < gr.n_cells * 4; e += kThreads) ACC[e] = 0.0f;
    float dv[TPW][4];
#pragma unroll
    for (int i = 0; i < TPW; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) dv[i][c] = 0.0f;
    const int r0 = warp * 16;
    const int mt = warp % MT;
    const int64_t tiles = (slots + kSlots - 1) / kSlots;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t first = tile * kSlots;
        __syncthreads();   // the previous tile's reads are over
        if (FOLD && tid < kSlots) CELL[tid] = first + tid < slots ? static_cast<int>(__ldg(cells + first + tid)) : -1;
        for (int e = tid; e < kSlots * (D / 4); e += kThreads) {
            const int s = e / (D / 4), q = e - s * (D / 4);
            const int64_t p = first + s;
            const float4 v = p < slots ? __ldcs(reinterpret_cast<const float4*>(d_v_raw + p * 4 * D + 3 * D) + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            *reinterpret_cast<float4*>(DM + s * D + 4 * q) = make_float4(bf16r(v.x), bf16r(v.y), bf16r(v.z), bf16r(v.w));
        }
        stage_tile<D>(Hs, SRC, WE, gr, h, cells, first, slots, tid);
        // the sources again, and each row's <d_m, sources_j>
        {
            float acc[NT][4];
            warp_rows_product<NT, KS, PW, PW>(acc, Hs, Ws, r0, g, t);
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const int row = r0 + g + 8 * h2;
                const float* dm = DM + (row >> 2) * D;
                float sum = 0.0f;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    sum += bf16r(dm[8 * nt + 2 * t] * bf16r(acc[nt][2 * h2])) + bf16r(dm[8 * nt + 2 * t + 1] * bf16r(acc[nt][2 * h2 + 1]));
                sum = sum4_lanes(sum);
                const int64_t p = first + (row >> 2);
                if constexpr (FOLD) {
                    if (t == 0) ROWV[row] = bf16r(sum);
                } else {
                    if (t == 0 && p < slots) edges[p * 4 + (row & 3)] = bf16r(sum);
                }
            }
        }
        for (int e = tid; e < kRows * (D / 2); e += kThreads) {
            const int row = e / (D / 2), w2 = e - row * (D / 2);
            const float w = WE[row];
            const float* dm = DM + (row >> 2) * D + 2 * w2;
            DS[row * PW + w2] = pack_bf16(dm[0] * w, dm[1] * w);
        }
        __syncthreads();
        if (FOLD && tid < 4) {   // neighbour tid of every slot of the tile, in slot order
            for (int s2 = 0; s2 < kSlots; ++s2) {
                const int c = CELL[s2];
                if (c >= 0) ACC[c * 4 + tid] += ROWV[4 * s2 + tid];
            }
        }
        // d_V[o][e] += sum_rows (w d_m)[row][o] h[src][row][e]: both operands hold the rows along their rows
        const uint16_t* ds16 = reinterpret_cast<const uint16_t*>(DS);
        const uint16_t* hs16 = reinterpret_cast<const uint16_t*>(Hs);
#pragma unroll 2
        for (int ks = 0; ks < kRows / 16; ++ks) {
            uint32_t a[4];
            ldmatrix_x4_trans(a, ds16 + (16 * ks + (lane & 7) + 8 * (lane >> 4)) * PB + 16 * mt + 8 * ((lane >> 3) & 1));
#pragma unroll
            for (int i = 0; i < TPW; ++i) {
                const int at = warp + 8 * i;
                if (at < TILES) {
                    uint32_t b[2];
                    ldmatrix_x2_trans(b, hs16 + (16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1)) * PB + 8 * (at / MT));
                    mma_bf16(dv[i], a, b[0], b[1]);
                }
            }
        }
    }
    float* mine = partial + static_cast<int64_t>(blockIdx.x) * (D * D);
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
        const int at = warp + 8 * i;
        if (at < TILES) {
            const int m = 16 * mt + g, n = 8 * (at / MT) + 2 * t;
            mine[m * D + n] = dv[i][0];
            mine[m * D + n + 1] = dv[i][1];
            mine[(m + 8) * D + n] = dv[i][2];
            mine[(m + 8) * D + n + 1] = dv[i][3];
        }
    }
    if constexpr (FOLD) {
        __syncthreads();
        float* table = edges + static_cast<int64_t>(blockIdx.x) * gr.n_cells * 4;
        for (int e = tid; e < gr.n_cells * 4; e += kThreads) table[e] = ACC[e];
    }
}

// The blocks' tables of the edge weights' gradient added in block order (eight threads an output, then those eight in
// order), as bf16 values; output e = 4 n + j goes to d_edge_w[n][j] for j < degree.
__global__ void __launch_bounds__(kThreads)
k_msg_etable(const float* __restrict__ tables, int blocks, int n_cells, int degree, float* __restrict__ d_edge_w) {
    __shared__ float part[8][32];
    const int outputs = n_cells * 4;
    const int lane = static_cast<int>(threadIdx.x) & 31, w = static_cast<int>(threadIdx.x) >> 5;
    const int e = static_cast<int>(blockIdx.x) * 32 + lane;
    float s = 0.0f;
    if (e < outputs) {
#pragma unroll 4
        for (int b = w; b < blocks; b += 8) s += __ldg(tables + static_cast<int64_t>(b) * outputs + e);
    }
    part[w][lane] = s;
    __syncthreads();
    if (w == 0 && e < outputs && (e & 3) < degree) {
        float total = part[0][lane];
#pragma unroll
        for (int r = 1; r < 8; ++r) total += part[r][lane];
        d_edge_w[(e >> 2) * degree + (e & 3)] = bf16r(total);
    }
}

// The blocks' shares of d_V added in a fixed order (eight threads an output, then those eight in order), as bf16 values.
__global__ void __launch_bounds__(kThreads)
k_msg_vgrad(const float* __restrict__ partial, int blocks, int outputs, float* __restrict__ d_v_w) {
    __shared__ float part[8][32];
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
        d_v_w[e] = bf16r(total);
    }
}

// d_edge_w[n][j] = the sum of rowval[p][j] over the slots p of cell n: a block a cell, a thread every 256th slot in
// order, then a fixed tree.
__global__ void __launch_bounds__(kThreads)
k_msg_egrad(const int64_t* __restrict__ cells, const float* __restrict__ rowval, int64_t slots, int degree, float* __restrict__ d_edge_w) {
    __shared__ float part[8][4];
    const int64_t n = blockIdx.x;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int64_t p = threadIdx.x; p < slots; p += kThreads) {
        if (__ldg(cells + p) == n) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(rowval) + p);
            acc[0] += v.x;
            acc[1] += v.y;
            acc[2] += v.z;
            acc[3] += v.w;
        }
    }
    const int lane = static_cast<int>(threadIdx.x) & 31, w = static_cast<int>(threadIdx.x) >> 5;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        if (lane == 0) part[w][j] = acc[j];
    }
    __syncthreads();
    if (threadIdx.x < static_cast<unsigned>(degree)) {
        float total = part[0][threadIdx.x];
#pragma unroll
        for (int r = 1; r < 8; ++r) total += part[r][threadIdx.x];
        d_edge_w[n * degree + threadIdx.x] = bf16r(total);
    }
}

// d_u[r] and d_eps[r]: the first two blocks of d_v_raw summed over the row's k slots.
__global__ void k_msg_ugrad(const float* __restrict__ d_v_raw, int64_t rows, int k, int d, float* __restrict__ d_u, float* __restrict__ d_eps) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * 2 * d) return;
    const int64_t r = i / (2 * d);
    const int e = static_cast<int>(i - r * 2 * d);
    float s = 0.0f;
    for (int s_k = 0; s_k < k; ++s_k) s += __ldg(d_v_raw + (r * k + s_k) * 4 * d + e);
    if (e < d) d_u[r * d + e] = s;
    else d_eps[r * d + e - d] = s;
}

int check(const HsnwMessages* m, int64_t rows, const char* what) {
    if (!m || rows < 0) return hsnw_fail(HSNW_E_ARG, what);
    if (!m->v_w || !m->edge_w || !m->pad_src) return hsnw_fail(HSNW_E_ARG, "messages: null table");
    if (!m->prod_bf16) return hsnw_fail(HSNW_E_UNSUPPORTED, "messages: float32 products are not taken here");
    if (m->d != 16 && m->d != 32 && m->d != 64) return hsnw_fail(HSNW_E_UNSUPPORTED, "messages: d must be 16, 32 or 64");
    if (m->degree < 1 || m->degree > 4) return hsnw_fail(HSNW_E_UNSUPPORTED, "messages: 1 to 4 in-neighbours a cell");
    if (m->n_cells < 1 || m->k < 1) return hsnw_fail(HSNW_E_ARG, "messages: n_cells and k must be positive");
    if (reinterpret_cast<uintptr_t>(m->v_w) % 8) return hsnw_fail(HSNW_E_ARG, "messages: V must be 8-byte aligned");
    return HSNW_OK;
}

int64_t bwd_blocks(int64_t slots, int sms) {
    const int64_t tiles = std::max<int64_t>(1, (slots + kSlots - 1) / kSlots);
    const int64_t cap = static_cast<int64_t>(sms) * 2;
    const int64_t rounds = (tiles + cap - 1) / cap;
    return (tiles + rounds - 1) / rounds;
}

constexpr int kFoldCells = 2048;   // the largest graph whose table [n_cells][4] a block keeps in shared memory
// The edge buffer: the blocks' tables, or a value per slot and neighbour.
int64_t edges_bytes(const HsnwMessages* m, int64_t slots, int64_t blocks) {
    const int64_t floats = m->n_cells <= kFoldCells ? blocks * m->n_cells * 4 : slots * 4;
    return (floats * static_cast<int64_t>(sizeof(float)) + 255) / 256 * 256;
}
bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

extern "C" int64_t hsnw_messages_scratch_bytes(const HsnwMessages* msg, int64_t rows) {
    if (!msg || rows < 0 || msg->k < 1 || msg->d < 16 || msg->d > 64) return 0;
    const int64_t slots = rows * msg->k;
    const int sms = std::max(148, hsnw_sm_count_current());
    const int64_t blocks = bwd_blocks(slots, sms);
    return edges_bytes(msg, slots, blocks) + (blocks * msg->d * msg->d * static_cast<int64_t>(sizeof(float)) + 255) / 256 * 256;
}

extern "C" int hsnw_messages_forward(const HsnwMessages* msg, const float* u, const float* eps, const float* h, const int64_t* cells,
                                     int64_t rows, float* v_raw, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(msg, rows, "messages_forward: null or negative")) return rc;
    if (rows == 0) return HSNW_OK;
    if (!u || !eps || !h || !cells || !v_raw) return hsnw_fail(HSNW_E_ARG, "messages_forward: null tensor");
    if (!aligned16(u) || !aligned16(eps) || !aligned16(h) || !aligned16(v_raw)) return hsnw_fail(HSNW_E_ARG, "messages_forward: tensors must be 16-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t slots = rows * msg->k;
    const Graph gr{msg->edge_w, msg->pad_src, msg->n_cells, msg->degree, msg->k};
    const unsigned tiles = static_cast<unsigned>((slots + kSlots - 1) / kSlots);
    hsnw_profile_mark(HSNW_K_MSG_FWD, stream);
#define HSNW_MSG_FWD(D) \
    case D: \
        k_msg_fwd<D><<<tiles, kThreads, MsgShape<D>::fwd_bytes, stream>>>(msg->v_w, gr, u, eps, h, cells, slots, v_raw); \
        break
    switch (msg->d) {
        HSNW_MSG_FWD(16);
        HSNW_MSG_FWD(32);
        HSNW_MSG_FWD(64);
    }
#undef HSNW_MSG_FWD
    return hsnw_check_launch("messages_forward");
}

extern "C" int hsnw_messages_backward(const HsnwMessages* msg, const float* h, const int64_t* cells, const float* d_v_raw, int64_t rows,
                                      float* d_u, float* d_eps, float* d_edge_w, float* d_v_w, void* scratch, int64_t scratch_bytes,
                                      void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(msg, rows, "messages_backward: null or negative")) return rc;
    if (!d_edge_w || !d_v_w) return hsnw_fail(HSNW_E_ARG, "messages_backward: null gradient");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int d = msg->d;
    if (rows == 0) {
        if (cudaMemsetAsync(d_v_w, 0, sizeof(float) * d * d, stream) != cudaSuccess
            || cudaMemsetAsync(d_edge_w, 0, sizeof(float) * msg->n_cells * msg->degree, stream) != cudaSuccess)
            return hsnw_check_launch("messages_backward");
        return HSNW_OK;
    }
    if (!h || !cells || !d_v_raw || !d_u || !d_eps) return hsnw_fail(HSNW_E_ARG, "messages_backward: null tensor");
    if (!scratch || scratch_bytes < hsnw_messages_scratch_bytes(msg, rows)) return hsnw_fail(HSNW_E_ARG, "messages_backward: scratch too small");
    if (!aligned16(h) || !aligned16(d_v_raw) || !aligned16(scratch)) return hsnw_fail(HSNW_E_ARG, "messages_backward: tensors and scratch must be 16-byte aligned");
    const int64_t slots = rows * msg->k;
    const Graph gr{msg->edge_w, msg->pad_src, msg->n_cells, msg->degree, msg->k};
    const int blocks = static_cast<int>(bwd_blocks(slots, std::max(1, hsnw_sm_count_current())));
    const bool fold = msg->n_cells <= kFoldCells;
    // (the scratch was sized for at least as many blocks: the partial sums start behind the larger edge buffer)
    const int64_t edge_bytes = edges_bytes(msg, slots, bwd_blocks(slots, std::max(148, hsnw_sm_count_current())));
    float* edges = static_cast<float*>(scratch);
    float* partial = reinterpret_cast<float*>(static_cast<char*>(scratch) + edge_bytes);
    const size_t table_bytes = fold ? sizeof(float) * 4 * static_cast<size_t>(msg->n_cells) : 0;
    hsnw_profile_mark(HSNW_K_MSG_BWD, stream);
    if (!fold && cudaMemsetAsync(edges, 0, static_cast<size_t>(edge_bytes), stream) != cudaSuccess) return hsnw_check_launch("messages_backward");
#define HSNW_MSG_BWD(D) \
    case D: \
        if (fold) k_msg_bwd<D, true><<<static_cast<unsigned>(blocks), kThreads, MsgShape<D>::bwd_bytes + table_bytes, stream>>>(msg->v_w, gr, h, cells, d_v_raw, slots, edges, partial); \
        else k_msg_bwd<D, false><<<static_cast<unsigned>(blocks), kThreads, MsgShape<D>::bwd_bytes, stream>>>(msg->v_w, gr, h, cells, d_v_raw, slots, edges, partial); \
        break
    switch (d) {
        HSNW_MSG_BWD(16);
        HSNW_MSG_BWD(32);
        HSNW_MSG_BWD(64);
    }
#undef HSNW_MSG_BWD
    k_msg_vgrad<<<static_cast<unsigned>((d * d + 31) / 32), kThreads, 0, stream>>>(partial, blocks, d * d, d_v_w);
    if (fold) k_msg_etable<<<static_cast<unsigned>((msg->n_cells * 4 + 31) / 32), kThreads, 0, stream>>>(edges, blocks, msg->n_cells, msg->degree, d_edge_w);
    else k_msg_egrad<<<static_cast<unsigned>(msg->n_cells), kThreads, 0, stream>>>(cells, edges, slots, msg->degree, d_edge_w);
    const int64_t outs = rows * 2 * d;
    k_msg_ugrad<<<static_cast<unsigned>((outs + 255) / 256), 256, 0, stream>>>(d_v_raw, rows, msg->k, d, d_u, d_eps);
    return hsnw_check_launch("messages_backward");
}

void hsnw_messages_set_attributes() {
    bool ok = true;
#define HSNW_MSG_OPT(D) \
    ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_msg_fwd<D>), "msg_fwd") && hsnw_opt_in(reinterpret_cast<const void*>(k_msg_bwd<D, true>), "msg_bwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_msg_bwd<D, false>), "msg_bwd")
    HSNW_MSG_OPT(16);
    HSNW_MSG_OPT(32);
    HSNW_MSG_OPT(64);
#undef HSNW_MSG_OPT
    if (!ok) hsnw_attribute_failed();
}
