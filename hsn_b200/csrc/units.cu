// The replay's grouped unit pass and its backward on the device: for P pairs (v_p [4d], unit_p) the chosen
// unit's two-layer perceptron out_p = act(v_p W1[u] + b1[u]) W2[u] + b2[u], every pair of a window at once,
// and the gradients of v and of the four stacked parameters for a cotangent of out (reference
// python/hsn/model/units.py:356-414, UnitBank.forward_grouped, and autograd's backward of its addmm /
// activation / addmm per present unit; python/hsn/model/cell.py:716 is the call in the replay).
//
// The reference sorts the pairs by unit on the host's reading of the unit histogram, cuts the sorted rows
// with one split and runs two addmm per present unit. Here nothing is read by the host: three small kernels
// sort the pairs stably by unit (per-block unit counts, one scan, placement) and cut the sorted order into
// tiles of 128 pairs (never across two units) and, for the weight gradients, into segments of `seg` pairs;
// every product then is ONE launch over all units' tiles:
//
//   forward   pre  = v W1[u] + b1[u]                     rows: a tile's pairs,   K = 4d
//             out  = act(pre) W2[u] + b2[u]              rows: a tile's pairs,   K = H
//   backward  dpre = (dout W2[u]^T) * act'(pre)          rows: a tile's pairs,   K = d   (kept in sorted order)
//             dv   = dpre W1[u]^T                        rows: a tile's pairs,   K = H
//             dW1 += v^T dpre, dW2 += act(pre)^T dout    rows: 4d resp. H,       K = a segment's pairs
//             db1  = sum dpre, db2 = sum dout            column sums per unit
//
// With bf16 products each is a tcgen05 tile product: a 128 x BN output tile per block with the accumulator
// in tensor memory, K in chunks of 128 staged by the block's threads as K-major core-matrix planes, 16 bytes
// (8 consecutive K elements of one row) per store. Every operand is therefore kept with its K contiguous:
// the weights are packed once per call as bfloat16 in both orientations ([K, N] and [N, K]); the operands of
// the weight gradients, whose K is the pair, are written transposed — v and dout by a transposing gather
// through the sorted order, dpre and act(pre) by the epilogue of the dpre product itself, which holds both
// — as [width, sorted position] with every unit's range starting on a multiple of 8 and zeros in the
// padding, so that a segment's 8 pairs are one aligned 16-byte load. The epilogues add the bias, round,
// apply the activation's derivative, and write through the sorted order so that every result lands in the
// pairs' input order. The weight gradients' segments write float32 partial tiles that a last kernel sums per
// unit in segment order (a fixed order: the same bits every run), rounds as the reference's bfloat16
// product does and widens to the parameters' float32; the bias gradients are row sums of the transposed
// operands. With fp32 products the operand functions read the tensors as they are and feed a CUDA-core tile
// kernel (sums in K order).
#include "../../include/hsn_units_b200.h"
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "stage.cuh"
#include "host_util.h"
#include "umma.cuh"

#include <algorithm>

using namespace hsnw;

namespace {

constexpr int kTile = 128;       // pairs of a row tile = rows of a tensor-core product
constexpr int kChunk = 64;       // K elements of one stage of the tensor-core products
constexpr int kSortBlock = 1024;
constexpr int kMaxUnits = 256;

struct Tables {
    int* order;        // [P] sorted position -> pair
    int* block_off;    // [blocks][M] pairs of unit u in earlier sort blocks
    int* unit_base;    // [M + 1] first sorted position of a unit, a multiple of 8 (the positions between a
                       // unit's last pair and the next unit's first hold no pair: order = -1)
    int* unit_count;   // [M] pairs of a unit
    int* tile_first;   // [M + 1] first tile of a unit
    int* seg_first;    // [M + 1] first segment of a unit
    int* tile_unit;    // [max tiles]
    int* tile_start;   // sorted position of the tile's first pair
    int* tile_rows;
    int* seg_unit;     // [max segments]
    int* seg_start;
    int* seg_len;
    int* counts;       // [0] tiles, [1] segments
};

// ---- sorting the pairs by unit ----------------------------------------------------------------------

// A warp's lanes with the same unit, in lane order: the rank of this lane among them and their number.
__device__ __forceinline__ void warp_rank(int unit, int lane, int& rank, int& peers_n) {
    const unsigned peers = __match_any_sync(0xffffffffu, unit);
    rank = __popc(peers & ((1u << lane) - 1u));
    peers_n = __popc(peers);
}

__device__ __forceinline__ int read_unit(const int64_t* unit_idx, int64_t p, int64_t pairs, int M, int* status) {
    if (p >= pairs) return -1;
    const int64_t u = unit_idx[p];
    if (u < 0 || u >= M) {
        atomicExch(status, 2);
        return -1;
    }
    return static_cast<int>(u);
}

// counts[warp][unit] of one sort block in shared memory (all 1024 threads call)
__device__ __forceinline__ void block_unit_counts(int* warp_count, int unit, int M, int& rank) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int e = tid; e < 32 * M; e += kSortBlock) warp_count[e] = 0;
    __syncthreads();
    int peers_n;
    warp_rank(unit, lane, rank, peers_n);
    if (unit >= 0 && rank == 0) warp_count[warp * M + unit] = peers_n;
    __syncthreads();
}

__global__ void __launch_bounds__(kSortBlock) k_units_count(const int64_t* unit_idx, int64_t pairs, int M, Tables tb, int* status) {
    extern __shared__ int warp_count[];
    const int64_t p = static_cast<int64_t>(blockIdx.x) * kSortBlock + threadIdx.x;
    int rank;
    block_unit_counts(warp_count, read_unit(unit_idx, p, pairs, M, status), M, rank);
    for (int u = threadIdx.x; u < M; u += kSortBlock) {
        int n = 0;
        for (int w = 0; w < 32; ++w) n += warp_count[w * M + u];
        tb.block_off[static_cast<int64_t>(blockIdx.x) * M + u] = n;   // the scan turns counts into offsets
    }
}

// One block: per unit the exclusive scan of its counts over the sort blocks, then the units' bases and the
// lists of tiles and segments.
__global__ void __launch_bounds__(256) k_units_scan(int blocks, int M, int seg, Tables tb) {
    __shared__ int total[kMaxUnits];
    const int tid = threadIdx.x;
    for (int u = tid >> 5; u < M; u += 8) {   // a warp a unit: 32 sort blocks a round, an exclusive scan by shuffles
        const int lane = tid & 31;
        int run = 0;
        for (int b0 = 0; b0 < blocks; b0 += 32) {
            const int b = b0 + lane;
            const int n = b < blocks ? tb.block_off[static_cast<int64_t>(b) * M + u] : 0;
            int inc = n;
#pragma unroll
            for (int w = 1; w < 32; w <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, inc, w);
                if (lane >= w) inc += up;
            }
            if (b < blocks) tb.block_off[static_cast<int64_t>(b) * M + u] = run + inc - n;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) total[u] = run;
    }
    __syncthreads();
    if (tid == 0) {
        int base = 0, tiles = 0, segs = 0;
        for (int u = 0; u < M; ++u) {
            tb.unit_base[u] = base;
            tb.unit_count[u] = total[u];
            tb.tile_first[u] = tiles;
            tb.seg_first[u] = segs;
            base += (total[u] + 7) & ~7;
            tiles += (total[u] + kTile - 1) / kTile;
            segs += (total[u] + seg - 1) / seg;
        }
        tb.unit_base[M] = base;
        tb.tile_first[M] = tiles;
        tb.seg_first[M] = segs;
        tb.counts[0] = tiles;
        tb.counts[1] = segs;
    }
    __syncthreads();
    const int tiles = tb.tile_first[M], segs = tb.seg_first[M];
    for (int t = tid; t < tiles; t += 256) {
        int u = 0;
        while (tb.tile_first[u + 1] <= t) ++u;
        const int at = (t - tb.tile_first[u]) * kTile;
        tb.tile_unit[t] = u;
        tb.tile_start[t] = tb.unit_base[u] + at;
        tb.tile_rows[t] = min(kTile, total[u] - at);
    }
    for (int s = tid; s < segs; s += 256) {
        int u = 0;
        while (tb.seg_first[u + 1] <= s) ++u;
        const int at = (s - tb.seg_first[u]) * seg;
        tb.seg_unit[s] = u;
        tb.seg_start[s] = tb.unit_base[u] + at;
        tb.seg_len[s] = min(seg, total[u] - at);
    }
}

__global__ void __launch_bounds__(kSortBlock) k_units_place(const int64_t* unit_idx, int64_t pairs, int M, Tables tb, int* status) {
    extern __shared__ int warp_count[];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int64_t p = static_cast<int64_t>(blockIdx.x) * kSortBlock + tid;
    const int unit = read_unit(unit_idx, p, pairs, M, status);
    int rank;
    block_unit_counts(warp_count, unit, M, rank);
    for (int u = tid; u < M; u += kSortBlock) {   // exclusive scan over the block's warps
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int n = warp_count[w * M + u];
            warp_count[w * M + u] = run;
            run += n;
        }
    }
    __syncthreads();
    if (unit >= 0)
        tb.order[tb.unit_base[unit] + tb.block_off[static_cast<int64_t>(blockIdx.x) * M + unit] + warp_count[warp * M + unit] + rank] =
            static_cast<int>(p);
}

// ---- operands and results of the six products -------------------------------------------------------------
// E: the type of pre, out, dout and dpre (bfloat16 with bf16 products, else float); BF: round as the bf16 pass
// does. Every product has two views of its operands: a(), b() give 8 consecutive K elements as floats from
// the tensors as the caller holds them (the CUDA-core kernel); a_row(), b_row() give the address of a row's
// K elements, contiguous, in the packed, sorted and transposed bfloat16 copies (the tensor-core kernel, BF only;
// a product's store() takes its 8 biases from `bias8`).

template <bool BF>
__device__ __forceinline__ float rnd(float x) {
    return BF ? bf16r(x) : x;
}
__device__ __forceinline__ void load8(const float* src, float x[8]) {
    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* src, float x[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ float load1(const float* src) { return *src; }
__device__ __forceinline__ float load1(const __nv_bfloat16* src) { return __bfloat162float(*src); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&pair);
}
__device__ __forceinline__ uint4 pack8(const float x[8]) {
    return make_uint4(pack2(x[0], x[1]), pack2(x[2], x[3]), pack2(x[4], x[5]), pack2(x[6], x[7]));
}
__device__ __forceinline__ void store8(float* dst, const float x[8]) {
    *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float x[8]) { *reinterpret_cast<uint4*>(dst) = pack8(x); }
__device__ __forceinline__ void zero8(float x[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = 0.0f;
}

// What every product knows: the sizes, the weights (float32 as the caller holds them; bfloat16 packed
// [N, K] for the product that reads them), the tables, and (after setup) its unit and range.
struct Base {
    int Din, H, D;
    int ld;                 // sorted positions a row of a transposed operand holds
    const float *w1, *b1, *w2, *b2;
    const __nv_bfloat16* wp;   // this product's packed weights
    Tables tb;
    int unit, start, len;   // a row tile's pairs or a segment's
    int item;               // the tile's or segment's number
    __device__ bool tile(int x) {
        if (x >= tb.counts[0]) return false;
        item = x, unit = tb.tile_unit[x], start = tb.tile_start[x], len = tb.tile_rows[x];
        return true;
    }
    __device__ bool segment(int x) {
        if (x >= tb.counts[1]) return false;
        item = x, unit = tb.seg_unit[x], start = tb.seg_start[x], len = tb.seg_len[x];
        return true;
    }
    __device__ int64_t pair(int sorted_offset) const { return tb.order[start + sorted_offset]; }
    __device__ uint4 aux(int, int) const { return make_uint4(0, 0, 0, 0); }   // nothing to request ahead
};

// pre[pair] = v[pair] W1[u] + b1[u]                      wp: W1 as [M, H, Din]; with bf16 products A is the
// sorted bfloat16 copy of v, and act(pre) is also written in sorted order for the second layer
template <class E, bool BF>
struct First : Base {
    static constexpr bool kTransposed = false;
    static constexpr int kStagedTiles = BF ? 2 : 0;   // pre and act(pre) leave through shared memory, whole rows at a time
    using Staged = __nv_bfloat16;
    const float* v;
    const __nv_bfloat16* v_s;   // [ld, Din]
    E* pre;
    __nv_bfloat16* hid_s;       // [ld, H]
    __device__ bool setup(int x) { return tile(x); }
    __device__ int rows() const { return len; }
    __device__ int cols() const { return H; }
    __device__ int depth() const { return Din; }
    __device__ const float* bias_row() const { return b1 + static_cast<int64_t>(unit) * H; }
    __device__ void a(int m, int k, float x[8]) const {
        if (m < len && k < Din) load8(v + pair(m) * Din + k, x);
        else zero8(x);
    }
    __device__ void b(int c, int k, float x[8]) const {
        const float* src = w1 + (static_cast<int64_t>(unit) * Din + k) * H + c;
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (c < H && k + i < Din) ? src[static_cast<int64_t>(i) * H] : 0.0f;
    }
    __device__ const __nv_bfloat16* a_row(int m) const { return m < len ? v_s + static_cast<int64_t>(start + m) * Din : nullptr; }
    __device__ const __nv_bfloat16* b_row(int c) const { return c < H ? wp + (static_cast<int64_t>(unit) * H + c) * Din : nullptr; }
    __device__ bool store(int m, int c0, float acc[8], const float* bias8, float* second, uint4) const {
        if (m >= len || c0 >= H) return false;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = rnd<BF>(acc[i] + rnd<BF>(bias8[i]));
        if constexpr (BF) {   // the tensor-core kernel collects pre and act(pre) in shared memory and writes whole rows
#pragma unroll
            for (int i = 0; i < 8; ++i) second[i] = gelu_erf(acc[i]);
        } else {
            store8(pre + pair(m) * H + c0, acc);
        }
        return true;
    }
    // where row m of the tile's two results goes (column 0 of the tensors), null past the tile's pairs
    __device__ void row_out(int m, __nv_bfloat16*& first, __nv_bfloat16*& other) const {
        first = other = nullptr;
        if constexpr (BF) {
            if (m < len) {
                first = pre + pair(m) * H;
                other = hid_s + static_cast<int64_t>(start + m) * H;
            }
        }
    }
};

// out[pair] = act(pre[pair]) W2[u] + b2[u]               wp: W2 as [M, D, H]; with bf16 products A is act(pre)
// in sorted order as the first layer left it
template <class E, bool BF>
struct Second : Base {
    static constexpr bool kTransposed = false;
    static constexpr int kStagedTiles = BF ? 1 : 0;
    using Staged = __nv_bfloat16;
    const E* pre;
    const __nv_bfloat16* hid_s;
    E* out;
    __device__ bool setup(int x) { return tile(x); }
    __device__ int rows() const { return len; }
    __device__ int cols() const { return D; }
    __device__ int depth() const { return H; }
    __device__ const float* bias_row() const { return b2 + static_cast<int64_t>(unit) * D; }
    __device__ void a(int m, int k, float x[8]) const {
        if (m < len && k < H) {
            load8(pre + pair(m) * H + k, x);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = rnd<BF>(gelu_erf(x[i]));
        } else {
            zero8(x);
        }
    }
    __device__ void b(int c, int k, float x[8]) const {
        const float* src = w2 + (static_cast<int64_t>(unit) * H + k) * D + c;
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (c < D && k + i < H) ? src[static_cast<int64_t>(i) * D] : 0.0f;
    }
    __device__ const __nv_bfloat16* a_row(int m) const { return m < len ? hid_s + static_cast<int64_t>(start + m) * H : nullptr; }
    __device__ const __nv_bfloat16* b_row(int c) const { return c < D ? wp + (static_cast<int64_t>(unit) * D + c) * H : nullptr; }
    __device__ bool store(int m, int c0, float acc[8], const float* bias8, float*, uint4) const {
        if (m >= len || c0 >= D) return false;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = rnd<BF>(acc[i] + rnd<BF>(bias8[i]));
        if constexpr (!BF) store8(out + pair(m) * D + c0, acc);
        return true;
    }
    __device__ void row_out(int m, __nv_bfloat16*& first, __nv_bfloat16*& other) const {
        other = nullptr;
        first = nullptr;
        if constexpr (BF)
            if (m < len) first = out + pair(m) * D;
    }
};

// dpre[sorted] = (dout[pair] W2[u]^T) * act'(pre[pair])   wp: W2 as [M, H, D]; with bf16 products also
// dpre and act(pre) transposed, [H, ld], zeros in the positions up to the next multiple of 8
template <class E, bool BF>
struct DPre : Base {
    static constexpr bool kTransposed = BF;
    static constexpr int kStagedTiles = BF ? 1 : 0;
    using Staged = __nv_bfloat16;
    const E *pre, *dout;
    E* dpre;   // in sorted order
    __nv_bfloat16 *dpre_t, *hid_t;
    __device__ bool setup(int x) { return tile(x); }
    __device__ int rows() const { return len; }
    __device__ int cols() const { return H; }
    __device__ int depth() const { return D; }
    __device__ const float* bias_row() const { return nullptr; }
    __device__ void a(int m, int k, float x[8]) const {
        if (m < len && k < D) load8(dout + pair(m) * D + k, x);
        else zero8(x);
    }
    __device__ void b(int c, int k, float x[8]) const {
        if (c < H && k < D) load8(w2 + (static_cast<int64_t>(unit) * H + c) * D + k, x);
        else zero8(x);
    }
    __device__ const E* a_row(int m) const { return m < len ? dout + pair(m) * D : nullptr; }
    __device__ const __nv_bfloat16* b_row(int c) const { return c < H ? wp + (static_cast<int64_t>(unit) * H + c) * D : nullptr; }
    // acc: in the product, out dpre; second: out act(pre)
    // the 8 pre-activations the store of (m, c0) reads, requested ahead of the accumulator
    __device__ uint4 aux(int m, int c0) const {
        if (m >= len || c0 >= H) return make_uint4(0, 0, 0, 0);
        const E* src = pre + pair(m) * H + c0;
        if constexpr (BF) return *reinterpret_cast<const uint4*>(src);
        else return make_uint4(0, 0, 0, 0);
    }
    __device__ bool store(int m, int c0, float acc[8], const float*, float* second, uint4 held) const {
        if (m >= len || c0 >= H) return false;
        float p[8];
        if constexpr (BF) {
            const uint32_t w[4] = {held.x, held.y, held.z, held.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                p[2 * i] = __uint_as_float(w[i] << 16);
                p[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
            load8(pre + pair(m) * H + c0, p);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {   // one erf for the activation and its derivative
            const float cdf = 0.5f * (1.0f + erff(p[i] * kSqrtHalf));
            acc[i] = rnd<BF>(rnd<BF>(acc[i]) * (cdf + p[i] * expf(-0.5f * p[i] * p[i]) * kInvSqrt2Pi));
            second[i] = p[i] * cdf;
        }
        if constexpr (!BF) store8(dpre + static_cast<int64_t>(start + m) * H + c0, acc);
        return true;
    }
    __device__ void row_out(int m, __nv_bfloat16*& first, __nv_bfloat16*& other) const {
        other = nullptr;
        first = nullptr;
        if constexpr (BF)
            if (m < len) first = dpre + static_cast<int64_t>(start + m) * H;
    }
    // unit j (8 sorted positions) of column c of the transposed tile, a word {dpre, act(pre)} a position: 16
    // consecutive threads write a column's 256 contiguous bytes of each result; zeros past the tile's pairs
    __device__ void store_unit(int c, int m0, int j, const uint32_t* column) const {
        if (c >= H || 8 * j >= ((min(len - m0, 128) + 7) & ~7)) return;
        const int64_t at = static_cast<int64_t>(c) * ld + start + m0 + 8 * j;
        const uint4 lo = *reinterpret_cast<const uint4*>(column + 8 * j), hi = *reinterpret_cast<const uint4*>(column + 8 * j + 4);
        // __byte_perm(a, b, 0x5410): the low halves of a and b; 0x7632: their high halves
        *reinterpret_cast<uint4*>(dpre_t + at) = make_uint4(__byte_perm(lo.x, lo.y, 0x5410), __byte_perm(lo.z, lo.w, 0x5410),
                                                             __byte_perm(hi.x, hi.y, 0x5410), __byte_perm(hi.z, hi.w, 0x5410));
        *reinterpret_cast<uint4*>(hid_t + at) = make_uint4(__byte_perm(lo.x, lo.y, 0x7632), __byte_perm(lo.z, lo.w, 0x7632),
                                                            __byte_perm(hi.x, hi.y, 0x7632), __byte_perm(hi.z, hi.w, 0x7632));
    }
};

// dv[pair] = dpre[sorted] W1[u]^T                          wp: W1 as [M, Din, H]
template <class E, bool BF>
struct DInput : Base {
    static constexpr bool kTransposed = false;
    static constexpr int kStagedTiles = BF ? 1 : 0;
    using Staged = float;
    const E* dpre;
    float* dv;
    __device__ bool setup(int x) { return tile(x); }
    __device__ int rows() const { return len; }
    __device__ int cols() const { return Din; }
    __device__ int depth() const { return H; }
    __device__ const float* bias_row() const { return nullptr; }
    __device__ void a(int m, int k, float x[8]) const {
        if (m < len && k < H) load8(dpre + static_cast<int64_t>(start + m) * H + k, x);
        else zero8(x);
    }
    __device__ void b(int c, int k, float x[8]) const {
        if (c < Din && k < H) load8(w1 + (static_cast<int64_t>(unit) * Din + c) * H + k, x);
        else zero8(x);
    }
    __device__ const E* a_row(int m) const { return m < len ? dpre + static_cast<int64_t>(start + m) * H : nullptr; }
    __device__ const __nv_bfloat16* b_row(int c) const { return c < Din ? wp + (static_cast<int64_t>(unit) * Din + c) * H : nullptr; }
    __device__ bool store(int m, int c0, float acc[8], const float*, float*, uint4) const {
        if (m >= len || c0 >= Din) return false;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = rnd<BF>(acc[i]);
        if constexpr (!BF) store8(dv + pair(m) * Din + c0, acc);
        return true;
    }
    __device__ void row_out(int m, float*& first, float*& other) const {
        other = nullptr;
        first = m < len ? dv + pair(m) * Din : nullptr;
    }
};

// partial[segment] = v[pairs]^T dpre[sorted]      [4d, H], K = the segment's pairs
template <class E, bool BF>
struct DWeight1 : Base {
    static constexpr bool kTransposed = false;
    static constexpr int kStagedTiles = 0;
    using Staged = float;
    const float* v;
    const E* dpre;
    const __nv_bfloat16 *v_t, *dpre_t;   // [Din, ld], [H, ld]
    float* partial;
    __device__ bool setup(int x) { return segment(x); }
    __device__ int rows() const { return Din; }
    __device__ int cols() const { return H; }
    __device__ int depth() const { return len; }
    __device__ const float* bias_row() const { return nullptr; }
    __device__ void a(int m, int k, float x[8]) const {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (m < Din && k + i < len) ? v[pair(k + i) * Din + m] : 0.0f;
    }
    __device__ void b(int c, int k, float x[8]) const {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (c < H && k + i < len) ? load1(dpre + static_cast<int64_t>(start + k + i) * H + c) : 0.0f;
    }
    __device__ const __nv_bfloat16* a_row(int m) const { return m < Din ? v_t + static_cast<int64_t>(m) * ld + start : nullptr; }
    __device__ const __nv_bfloat16* b_row(int c) const { return c < H ? dpre_t + static_cast<int64_t>(c) * ld + start : nullptr; }
    __device__ bool store(int m, int c0, float acc[8], const float*, float*, uint4) const {
        if (m >= Din || c0 >= H) return false;
        store8(partial + (static_cast<int64_t>(item) * Din + m) * H + c0, acc);
        return true;
    }
};

// partial[segment] = act(pre[pairs])^T dout[pairs]      [H, d], K = the segment's pairs
template <class E, bool BF>
struct DWeight2 : Base {
    static constexpr bool kTransposed = false;
    static constexpr int kStagedTiles = 0;
    using Staged = float;
    const E *pre, *dout;
    const __nv_bfloat16 *hid_t, *dout_t;   // [H, ld], [D, ld]
    float* partial;
    __device__ bool setup(int x) { return segment(x); }
    __device__ int rows() const { return H; }
    __device__ int cols() const { return D; }
    __device__ int depth() const { return len; }
    __device__ const float* bias_row() const { return nullptr; }
    __device__ void a(int m, int k, float x[8]) const {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (m < H && k + i < len) ? rnd<BF>(gelu_erf(load1(pre + pair(k + i) * H + m))) : 0.0f;
    }
    __device__ void b(int c, int k, float x[8]) const {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (c < D && k + i < len) ? load1(dout + pair(k + i) * D + c) : 0.0f;
    }
    __device__ const __nv_bfloat16* a_row(int m) const { return m < H ? hid_t + static_cast<int64_t>(m) * ld + start : nullptr; }
    __device__ const __nv_bfloat16* b_row(int c) const { return c < D ? dout_t + static_cast<int64_t>(c) * ld + start : nullptr; }
    __device__ bool store(int m, int c0, float acc[8], const float*, float*, uint4) const {
        if (m >= H || c0 >= D) return false;
        store8(partial + (static_cast<int64_t>(item) * H + m) * D + c0, acc);
        return true;
    }
};

// ---- the tile products ----------------------------------------------------------------------------------

// 16 bytes global -> shared without passing through registers; `src` null: 16 zero bytes (nothing is read,
// `safe` only has to be an address of the same space)
__device__ __forceinline__ void copy16_or_zero(void* dst_smem, const void* src, const void* safe) {
    const unsigned bytes = src ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst_smem)), "l"(src ? src : safe), "r"(bytes) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait_but() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

constexpr int kStages = 2;
constexpr int kTcThreads = 256;
constexpr int kTilePitch = 128 + 4;   // words between the columns of a transposed tile: a quarter warp's 16-byte reads of 8 columns fall on 8 groups of banks

// One K = 16 step of a product whose two operands are in the 128-byte swizzle: inside the 128-byte K block a
// step moves both start addresses by 32 bytes.
template <int STEPS>
__device__ __forceinline__ void umma_block_sw128(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, int steps, bool onto) {
    __syncwarp();
#pragma unroll
    for (int s = 0; s < STEPS; ++s)
        if (s < steps) umma_bf16(tmem_d, desc_a + static_cast<uint64_t>(2 * s), desc_b + static_cast<uint64_t>(2 * s), idesc, onto || s > 0);
}

// bf16 operands on the tensor cores: block (x: tile or segment, y: 128 rows, z: BN columns). K goes in
// blocks of 64 elements — one 128-byte row of the 128-byte swizzle per operand row — through the stages of
// shared memory: 8 consecutive lanes request the 8 units of one row (a fully used 128-byte line of global
// memory) as asynchronous 16-byte copies to their swizzled places (unit u of row r at u ^ (r % 8), so a
// warp's 4 rows fill 512 contiguous bytes), the next block while the tensor cores work on this one; a stage
// is requested again when the commit of the products that read it has arrived. The epilogue reads the
// accumulator 32 columns at a time, a thread its own row and half of the columns; a product whose result is also wanted transposed
// (dpre) collects it with its companion as a tile [column, row] of bfloat16 pairs in the stages' memory and
// writes the two 16 threads a column, 16 bytes a store.
template <class Op, int BN>
__global__ void __launch_bounds__(kTcThreads) k_units_tc(Op op, int* status) {
    static_assert(kChunk == 64, "a K block is one 128-byte swizzle row");
    constexpr int kStageBytes = (128 + BN) * 128;   // A tile then B tile, 128 bytes a row
    using ST = typename Op::Staged;
    constexpr int kRowPitch = BN * static_cast<int>(sizeof(ST)) + 16;   // a row of a staged result tile
    constexpr int kStagedBase = Op::kTransposed ? BN * kTilePitch * 4 : 0;   // behind the transposed tile
    constexpr int kPass = kTcThreads / 8;                   // rows the block requests in one pass: 8 lanes a row
    constexpr int kRowsA = 128 / kPass, kRowsB = BN / kPass;   // rows of a tile a thread requests
    extern __shared__ unsigned char dyn_raw[];
    __shared__ __align__(8) uint64_t bar[kStages];
    __shared__ uint32_t tmem_slot;
    __shared__ float bias_s[BN];
    if (!op.setup(blockIdx.x)) return;   // the same answer for the whole block
    const int m0 = blockIdx.y * 128, n0 = blockIdx.z * BN;
    if (m0 >= op.rows() || n0 >= op.cols()) return;
    const int tid = threadIdx.x, warp = tid >> 5;
    unsigned char* dyn = dyn_raw + ((1024u - (smem_addr(dyn_raw) & 1023u)) & 1023u);   // swizzle atoms are 1024 bytes
    if (tid == 0)
        for (int s = 0; s < kStages; ++s) mbar_init(&bar[s], 1);
    if (warp == 0) tmem_alloc(&tmem_slot, BN < 32 ? 32 : BN);
    if (tid < BN) {
        const float* bias = op.bias_row();
        bias_s[tid] = (bias && n0 + tid < op.cols()) ? bias[n0 + tid] : 0.0f;
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    const uint32_t idesc = umma_idesc_bf16(128, BN);
    const int K = op.depth();
    const int chunks = (K + kChunk - 1) / kChunk;
    const int unit = tid & 7, row0 = tid >> 3;   // this thread's unit of a row, and its row in each pass
    decltype(op.a_row(0)) a_rows[kRowsA];
    decltype(op.b_row(0)) b_rows[kRowsB];
#pragma unroll
    for (int j = 0; j < kRowsA; ++j) a_rows[j] = op.a_row(m0 + kPass * j + row0);
#pragma unroll
    for (int j = 0; j < kRowsB; ++j) b_rows[j] = op.b_row(n0 + kPass * j + row0);
    auto request = [&](int c) {   // K block c into stage c % kStages; one group per call, block or not
        if (c < chunks) {
            unsigned char* As = dyn + (c % kStages) * kStageBytes;
            unsigned char* Bs = As + 128 * 128;
            const int k = c * kChunk + 8 * unit;
            const bool in = k < K;
#pragma unroll
            for (int j = 0; j < kRowsA; ++j) {
                const int r = kPass * j + row0;
                copy16_or_zero(As + r * 128 + ((unit ^ (r & 7)) << 4), (in && a_rows[j]) ? a_rows[j] + k : nullptr, op.w1);
            }
#pragma unroll
            for (int j = 0; j < kRowsB; ++j) {
                const int r = kPass * j + row0;
                copy16_or_zero(Bs + r * 128 + ((unit ^ (r & 7)) << 4), (in && b_rows[j]) ? b_rows[j] + k : nullptr, op.w1);
            }
        }
        cp_async_commit();
    };
    for (int c = 0; c < kStages - 1; ++c) request(c);
    for (int c = 0; c < chunks; ++c) {
        cp_async_wait_but<kStages - 2>();   // the groups complete in order: block c has landed
        fence_async_smem();
        __syncthreads();
        if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
            const unsigned char* As = dyn + (c % kStages) * kStageBytes;
            const int steps = (min(kChunk, K - c * kChunk) + 15) >> 4;
            tcgen05_fence_after();
            umma_block_sw128<4>(taddr, umma_desc_sw128(As), umma_desc_sw128(As + 128 * 128), idesc, steps, c > 0);
            umma_commit(&bar[c % kStages]);
        }
        // block c + kStages - 1 goes where block c - 1 was: its products (issued an iteration ago) must have read it
        if (c >= 1 && c + kStages - 1 < chunks) mbar_wait(&bar[(c - 1) % kStages], ((c - 1) / kStages) & 1, status);
        request(c + kStages - 1);
    }
    mbar_wait(&bar[(chunks - 1) % kStages], ((chunks - 1) / kStages) & 1, status);   // the last commit covers every product before it
    tcgen05_fence_after();
    float x[32], second[8];
    uint32_t* tile = reinterpret_cast<uint32_t*>(dyn);   // [BN][128] words {result, second}, in the stages' memory (every product has read it)
    // warps w and w + 4 reach the same 32 rows of the accumulator: each takes half of the columns
    const int row = (warp & 3) * 32 + (tid & 31), half = (warp >> 2) * (BN / 2);
    for (int cb = half; cb < half + BN / 2; cb += 32) {   // 32 columns a wait on tensor memory
        uint4 held[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) held[j] = op.aux(m0 + row, n0 + cb + 8 * j);
        tmem_ld32(tmem_addr(taddr, (warp & 3) * 32, cb), x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const bool wrote = op.store(m0 + row, n0 + cb + 8 * j, x + 8 * j, bias_s + cb + 8 * j, second, held[j]);
            if constexpr (Op::kTransposed) {
#pragma unroll
                for (int i = 0; i < 8; ++i) tile[(cb + 8 * j + i) * kTilePitch + row] = wrote ? pack2(x[8 * j + i], second[i]) : 0u;
            }
            if constexpr (Op::kStagedTiles > 0) {   // row-major tiles, rows kRowPitch bytes apart (a quarter warp's 8 rows on 8 groups of banks)
                ST* at = reinterpret_cast<ST*>(dyn + kStagedBase + row * kRowPitch) + cb + 8 * j;
                store8(at, x + 8 * j);
                if constexpr (Op::kStagedTiles > 1) store8(reinterpret_cast<ST*>(reinterpret_cast<unsigned char*>(at) + 128 * kRowPitch), second);
            }
        }
    }
    if constexpr (Op::kTransposed) {
        __syncthreads();
        for (int e = tid; e < BN * 16; e += kTcThreads) op.store_unit(n0 + (e >> 4), m0, e & 15, tile + (e >> 4) * kTilePitch);
    }
    if constexpr (Op::kStagedTiles > 0) {   // consecutive threads write one row's 16-byte units: whole lines of global memory
        __syncthreads();
        constexpr int kPer = 16 / static_cast<int>(sizeof(ST)), kUnits = BN / kPer;   // elements a unit, units a row
        const int units = min(BN, op.cols() - n0) / kPer;
        for (int e = tid; e < 128 * kUnits; e += kTcThreads) {
            const int r = e / kUnits, u = e % kUnits;
            ST *first, *other;
            op.row_out(m0 + r, first, other);
            if (u < units && first) {
                const unsigned char* at = dyn + kStagedBase + r * kRowPitch + u * 16;
                *reinterpret_cast<uint4*>(first + n0 + kPer * u) = *reinterpret_cast<const uint4*>(at);
                if constexpr (Op::kStagedTiles > 1) *reinterpret_cast<uint4*>(other + n0 + kPer * u) = *reinterpret_cast<const uint4*>(at + 128 * kRowPitch);
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, BN < 32 ? 32 : BN);
}

// fp32 operands on the CUDA cores: block (x: tile or segment, y: 64 rows, z: 64 columns), a thread 2 x 8
// outputs, K in chunks of 16, every sum in K order.
template <class Op>
__global__ void __launch_bounds__(256) k_units_simt(Op op) {
    __shared__ float As[16][64], Bs[16][64];
    if (!op.setup(blockIdx.x)) return;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.z * 64;
    if (m0 >= op.rows() || n0 >= op.cols()) return;
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;
    const int K = op.depth();
    float acc[2][8] = {};
    float x[8];
    for (int k0 = 0; k0 < K; k0 += 16) {
        const int r = tid & 63, half = (tid >> 6) & 1;
        if (tid < 128) op.a(m0 + r, k0 + 8 * half, x);
        else op.b(n0 + r, k0 + 8 * half, x);
        float(*dst)[64] = tid < 128 ? As : Bs;
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[8 * half + i][r] = x[i];
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            const float a0 = As[kk][2 * ty], a1 = As[kk][2 * ty + 1];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float bv = Bs[kk][8 * tx + i];
                acc[0][i] = fmaf(a0, bv, acc[0][i]);
                acc[1][i] = fmaf(a1, bv, acc[1][i]);
            }
        }
        __syncthreads();
    }
    const float* bias = op.bias_row();
    float second[8];
    if (bias) bias += n0 + 8 * tx;   // read only where the store takes the columns
    op.store(m0 + 2 * ty, n0 + 8 * tx, acc[0], bias, second, make_uint4(0, 0, 0, 0));
    op.store(m0 + 2 * ty + 1, n0 + 8 * tx, acc[1], bias, second, make_uint4(0, 0, 0, 0));
}

// out[b][c][r] = bfloat16(src[b][row(r)][c]) for r < rows, c < cols: 32 x 32 tiles through shared memory. With
// `order`, row(r) = order[r] and a position that holds no pair (order < 0) becomes a column of zeros.
template <class S>
__global__ void __launch_bounds__(256) k_units_transpose(const S* src, int64_t src_batch, int rows, int cols, const int* order,
                                                         __nv_bfloat16* out, int64_t out_batch, int ld) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    src += static_cast<int64_t>(blockIdx.z) * src_batch;
    out += static_cast<int64_t>(blockIdx.z) * out_batch;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int r = r0 + ty + 8 * j, c = c0 + tx;
        float value = 0.0f;
        if (r < rows && c < cols) {
            const int64_t row = order ? order[r] : r;
            if (row >= 0) value = load1(src + row * cols + c);
        }
        tile[ty + 8 * j][tx] = value;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int c = c0 + ty + 8 * j, r = r0 + tx;
        if (c < cols && r < rows) out[static_cast<int64_t>(c) * ld + r] = __float2bfloat16_rn(tile[tx][ty + 8 * j]);
    }
}

// out[e] = bfloat16(src[e])
__global__ void __launch_bounds__(256) k_units_cast(const float* src, int64_t n8, __nv_bfloat16* out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    float x[8];
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; e < n8; e += stride) {
        load8(src + 8 * e, x);
        store8(out + 8 * e, x);
    }
}

// out[s] = bfloat16(v[order[s]]) for every sorted position that holds a pair: 8 elements a thread
__global__ void __launch_bounds__(256) k_units_gather(const float* v, int width8, int64_t n, const int* order, __nv_bfloat16* out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    float x[8];
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; e < n; e += stride) {
        const int64_t s = e / width8;
        const int k = static_cast<int>(e - s * width8) * 8;
        const int64_t row = order[s];
        if (row < 0) continue;
        load8(v + (row * width8) * 8 + k, x);
        store8(out + (s * width8) * 8 + k, x);
    }
}

// d_w[u][e] = round(sum over the unit's segments, in order, of partial[segment][e]); zero for a unit no pair chose
template <bool BF>
__global__ void __launch_bounds__(256) k_units_wgrad(const float* partial, int64_t elems, int M, Tables tb, float* dw) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; e < elems * M; e += stride) {
        const int u = static_cast<int>(e / elems);
        const int64_t at = e - static_cast<int64_t>(u) * elems;
        float sum = 0.0f;
        for (int s = tb.seg_first[u]; s < tb.seg_first[u + 1]; ++s) sum += partial[static_cast<int64_t>(s) * elems + at];
        dw[e] = rnd<BF>(sum);
    }
}

// d_b[u][c] = round(sum over the unit's pairs of x[row][c]): block (unit, 32 columns), 8 rows at a time
template <class E, bool BF, bool SORTED>
__global__ void __launch_bounds__(256) k_units_bgrad(const E* x, int width, Tables tb, float* db) {
    __shared__ float part[8][33];
    const int u = blockIdx.x, c = blockIdx.y * 32 + (threadIdx.x & 31), lane_row = threadIdx.x >> 5;
    const int begin = tb.unit_base[u], end = begin + tb.unit_count[u];
    float sum = 0.0f;
    if (c < width)
        for (int p = begin + lane_row; p < end; p += 8) {
            const int64_t row = SORTED ? p : tb.order[p];
            sum += load1(x + row * width + c);
        }
    part[lane_row][threadIdx.x & 31] = sum;
    __syncthreads();
    if (lane_row == 0 && c < width) {
        float total = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) total += part[r][threadIdx.x & 31];
        db[static_cast<int64_t>(u) * width + c] = rnd<BF>(total);
    }
}

// The same from a transposed operand [width, ld]: block (unit, column), the unit's positions are one contiguous
// run that starts on a multiple of 8 and is padded with zeros to one.
__global__ void __launch_bounds__(128) k_units_bgrad_t(const __nv_bfloat16* x_t, int ld, int width, Tables tb, float* db) {
    __shared__ float part[4];
    const int u = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
    const int units8 = (tb.unit_count[u] + 7) >> 3;
    const __nv_bfloat16* row = x_t + static_cast<int64_t>(c) * ld + tb.unit_base[u];
    float sum = 0.0f, x[8];
    for (int e = tid; e < units8; e += 128) {
        load8(row + 8 * e, x);
        sum += ((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]));
    }
    sum = warp_sum(sum);
    if ((tid & 31) == 0) part[tid >> 5] = sum;
    __syncthreads();
    if (tid == 0) db[static_cast<int64_t>(u) * width + c] = bf16r((part[0] + part[1]) + (part[2] + part[3]));
}

// ---- host ---------------------------------------------------------------------------------------------

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

constexpr int kTables = 13;

struct Plan {
    int blocks, max_tiles, seg, max_segs;
    int ld;   // sorted positions: the pairs and every unit's padding to a multiple of 8
    size_t bytes;
    size_t off_tables[kTables];
    size_t off_wa, off_wb;   // this call's two packed weights
    size_t off_vs, off_hids;   // forward: v and act(pre) in sorted order
    size_t off_dpre, off_partial1, off_partial2, off_vt, off_doutt, off_dpret, off_hidt;
};

Plan make_plan(const HsnwUnits* u, int64_t pairs, bool backward) {
    Plan p{};
    const int M = u->n_units;
    p.blocks = static_cast<int>((pairs + kSortBlock - 1) / kSortBlock);
    p.max_tiles = static_cast<int>((pairs + kTile - 1) / kTile) + M;
    int64_t seg = (pairs + 63) / 64;
    seg = (seg + kTile - 1) / kTile * kTile;
    p.seg = static_cast<int>(seg < 1024 ? 1024 : seg);
    p.max_segs = static_cast<int>((pairs + p.seg - 1) / p.seg) + M;
    p.ld = static_cast<int>(((pairs + 7) & ~static_cast<int64_t>(7)) + 8 * M);
    size_t at = 256;   // the status word
    const size_t sizes[kTables] = {
        static_cast<size_t>(p.ld), static_cast<size_t>(p.blocks) * M, static_cast<size_t>(M) + 1, static_cast<size_t>(M),
        static_cast<size_t>(M) + 1, static_cast<size_t>(M) + 1, static_cast<size_t>(p.max_tiles), static_cast<size_t>(p.max_tiles),
        static_cast<size_t>(p.max_tiles), static_cast<size_t>(p.max_segs), static_cast<size_t>(p.max_segs), static_cast<size_t>(p.max_segs), 2};
    for (int i = 0; i < kTables; ++i) {
        p.off_tables[i] = at;
        at += up256(sizes[i] * sizeof(int));
    }
    if (u->prod_bf16) {
        p.off_wa = at;
        at += up256(static_cast<size_t>(M) * u->d_in * u->hidden * 2);
        p.off_wb = at;
        at += up256(static_cast<size_t>(M) * u->hidden * u->d_out * 2);
    }
    if (!backward && u->prod_bf16) {
        p.off_vs = at;
        at += up256(static_cast<size_t>(p.ld) * u->d_in * 2);
        p.off_hids = at;
        at += up256(static_cast<size_t>(p.ld) * u->hidden * 2);
    }
    if (backward) {
        const size_t elem = u->prod_bf16 ? 2 : 4;
        p.off_dpre = at;
        at += up256(static_cast<size_t>(p.ld) * u->hidden * elem);
        p.off_partial1 = at;
        at += up256(static_cast<size_t>(p.max_segs) * u->d_in * u->hidden * sizeof(float));
        p.off_partial2 = at;
        at += up256(static_cast<size_t>(p.max_segs) * u->hidden * u->d_out * sizeof(float));
        if (u->prod_bf16) {
            p.off_vt = at;
            at += up256(static_cast<size_t>(p.ld) * u->d_in * 2);
            p.off_doutt = at;
            at += up256(static_cast<size_t>(p.ld) * u->d_out * 2);
            p.off_dpret = at;
            at += up256(static_cast<size_t>(p.ld) * u->hidden * 2);
            p.off_hidt = at;
            at += up256(static_cast<size_t>(p.ld) * u->hidden * 2);
        }
    }
    p.bytes = at;
    return p;
}

Tables make_tables(const Plan& p, void* scratch) {
    unsigned char* base = static_cast<unsigned char*>(scratch);
    auto at = [&](int i) { return reinterpret_cast<int*>(base + p.off_tables[i]); };
    return Tables{at(0), at(1), at(2), at(3), at(4), at(5), at(6), at(7), at(8), at(9), at(10), at(11), at(12)};
}

int check_units(const HsnwUnits* u, int64_t pairs, const char* what) {
    if (!u || pairs < 0) return hsnw_fail(HSNW_E_ARG, what);
    if (u->n_units < 1 || u->d_in < 1 || u->hidden < 1 || u->d_out < 1 || !u->w1 || !u->b1 || !u->w2 || !u->b2)
        return hsnw_fail(HSNW_E_ARG, "units: sizes or weights missing");
    if (u->n_units > kMaxUnits) return hsnw_fail(HSNW_E_UNSUPPORTED, "units: at most 256 units");
    if (u->d_in % 8 || u->hidden % 8 || u->d_out % 8) return hsnw_fail(HSNW_E_UNSUPPORTED, "units: the three widths in multiples of 8");
    if (pairs >= (static_cast<int64_t>(1) << 31) - kSortBlock - 8 * kMaxUnits) return hsnw_fail(HSNW_E_UNSUPPORTED, "units: fewer than 2^31 pairs");
    if ((reinterpret_cast<uintptr_t>(u->w1) | reinterpret_cast<uintptr_t>(u->w2)) & 15)
        return hsnw_fail(HSNW_E_ARG, "units: weights not 16-byte aligned");
    return HSNW_OK;
}

int sort_pairs(const HsnwUnits* u, const int64_t* unit_idx, int64_t pairs, const Plan& p, const Tables& tb, int* status, cudaStream_t stream) {
    const size_t shared = sizeof(int) * 32 * u->n_units;
    if (cudaMemsetAsync(tb.order, 0xff, sizeof(int) * static_cast<size_t>(p.ld), stream) != cudaSuccess) return hsnw_check_launch("units: sort");
    k_units_count<<<p.blocks, kSortBlock, shared, stream>>>(unit_idx, pairs, u->n_units, tb, status);
    k_units_scan<<<1, 256, 0, stream>>>(p.blocks, u->n_units, p.seg, tb);
    k_units_place<<<p.blocks, kSortBlock, shared, stream>>>(unit_idx, pairs, u->n_units, tb, status);
    return hsnw_check_launch("units: sort");
}

// the weights as bfloat16: as they are (k_units_cast) or with the last two dimensions exchanged
void pack_weights(const float* w, int M, int rows, int cols, bool transpose, __nv_bfloat16* out, cudaStream_t stream) {
    if (transpose) {
        k_units_transpose<float><<<dim3((rows + 31) / 32, (cols + 31) / 32, M), 256, 0, stream>>>(
            w, static_cast<int64_t>(rows) * cols, rows, cols, nullptr, out, static_cast<int64_t>(rows) * cols, rows);
    } else {
        const int64_t n8 = static_cast<int64_t>(M) * rows * cols / 8;
        k_units_cast<<<static_cast<unsigned>(std::min<int64_t>((n8 + 255) / 256, 1024)), 256, 0, stream>>>(w, n8, out);
    }
}

template <class Op>
void fill_base(Op& op, const HsnwUnits* u, const Tables& tb, const Plan& p, const __nv_bfloat16* packed) {
    op.Din = u->d_in, op.H = u->hidden, op.D = u->d_out, op.ld = p.ld;
    op.w1 = u->w1, op.b1 = u->b1, op.w2 = u->w2, op.b2 = u->b2;
    op.wp = packed;
    op.tb = tb;
}

template <class Op, int BN>
void launch_tc(const Op& op, int items, int rows, int cols, int* status, cudaStream_t stream) {
    size_t shared = static_cast<size_t>(kStages) * (128 + BN) * 128;
    shared = std::max(shared, (Op::kTransposed ? static_cast<size_t>(BN) * kTilePitch * 4 : 0)
                                  + static_cast<size_t>(Op::kStagedTiles) * 128 * (BN * sizeof(typename Op::Staged) + 16));   // the result tiles
    shared += 1024;   // the kernel starts its stages on a 1024-byte boundary
    k_units_tc<Op, BN><<<dim3(items, (rows + 127) / 128, (cols + BN - 1) / BN), kTcThreads, shared, stream>>>(op, status);
}
template <class Op>
void launch_simt(const Op& op, int items, int rows, int cols, cudaStream_t stream) {
    k_units_simt<Op><<<dim3(items, (rows + 63) / 64, (cols + 63) / 64), 256, 0, stream>>>(op);
}

template <class E, bool BF>
int forward_t(const HsnwUnits* u, const float* v, int64_t pairs, E* pre, E* out, const Plan& p, const Tables& tb, void* scratch,
              int* status, cudaStream_t stream) {
    unsigned char* base = static_cast<unsigned char*>(scratch);
    __nv_bfloat16* w1t = reinterpret_cast<__nv_bfloat16*>(base + p.off_wa);   // [M, H, Din]
    __nv_bfloat16* w2t = reinterpret_cast<__nv_bfloat16*>(base + p.off_wb);   // [M, D, H]
    First<E, BF> first;
    fill_base(first, u, tb, p, w1t);
    __nv_bfloat16* v_s = reinterpret_cast<__nv_bfloat16*>(base + p.off_vs);
    __nv_bfloat16* hid_s = reinterpret_cast<__nv_bfloat16*>(base + p.off_hids);
    first.v = v, first.pre = pre, first.v_s = v_s, first.hid_s = hid_s;
    Second<E, BF> second;
    fill_base(second, u, tb, p, w2t);
    second.pre = pre, second.out = out, second.hid_s = hid_s;
    if constexpr (BF) {
        const int64_t n = static_cast<int64_t>(p.ld) * (u->d_in / 8);
        k_units_gather<<<static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 148 * 16)), 256, 0, stream>>>(v, u->d_in / 8, n, tb.order, v_s);
        pack_weights(u->w1, u->n_units, u->d_in, u->hidden, true, w1t, stream);
        pack_weights(u->w2, u->n_units, u->hidden, u->d_out, true, w2t, stream);
        launch_tc<First<E, BF>, 128>(first, p.max_tiles, kTile, u->hidden, status, stream);
        if (u->d_out <= 64) launch_tc<Second<E, BF>, 64>(second, p.max_tiles, kTile, u->d_out, status, stream);
        else launch_tc<Second<E, BF>, 128>(second, p.max_tiles, kTile, u->d_out, status, stream);
    } else {
        launch_simt(first, p.max_tiles, kTile, u->hidden, stream);
        launch_simt(second, p.max_tiles, kTile, u->d_out, stream);
    }
    return hsnw_check_launch("units_forward");
}

template <class E, bool BF>
int backward_t(const HsnwUnits* u, const float* v, int64_t pairs, const E* pre, const E* dout, float* dv, float* dw1, float* db1, float* dw2,
               float* db2, const Plan& p, const Tables& tb, void* scratch, int* status, cudaStream_t stream) {
    unsigned char* base = static_cast<unsigned char*>(scratch);
    auto half = [&](size_t off) { return reinterpret_cast<__nv_bfloat16*>(base + off); };
    E* dpre = reinterpret_cast<E*>(base + p.off_dpre);
    float* partial1 = reinterpret_cast<float*>(base + p.off_partial1);
    float* partial2 = reinterpret_cast<float*>(base + p.off_partial2);
    __nv_bfloat16 *w1k = half(p.off_wa), *w2k = half(p.off_wb);   // [M, Din, H], [M, H, D]: the weights as they are
    __nv_bfloat16 *v_t = half(p.off_vt), *dout_t = half(p.off_doutt), *dpre_t = half(p.off_dpret), *hid_t = half(p.off_hidt);
    DPre<E, BF> dp;
    fill_base(dp, u, tb, p, w2k);
    dp.pre = pre, dp.dout = dout, dp.dpre = dpre, dp.dpre_t = dpre_t, dp.hid_t = hid_t;
    DInput<E, BF> di;
    fill_base(di, u, tb, p, w1k);
    di.dpre = dpre, di.dv = dv;
    DWeight1<E, BF> g1;
    fill_base(g1, u, tb, p, nullptr);
    g1.v = v, g1.dpre = dpre, g1.v_t = v_t, g1.dpre_t = dpre_t, g1.partial = partial1;
    DWeight2<E, BF> g2;
    fill_base(g2, u, tb, p, nullptr);
    g2.pre = pre, g2.dout = dout, g2.hid_t = hid_t, g2.dout_t = dout_t, g2.partial = partial2;
    const int M = u->n_units;
    if constexpr (BF) {
        pack_weights(u->w1, M, u->d_in, u->hidden, false, w1k, stream);
        pack_weights(u->w2, M, u->hidden, u->d_out, false, w2k, stream);
        k_units_transpose<float><<<dim3((p.ld + 31) / 32, (u->d_in + 31) / 32, 1), 256, 0, stream>>>(v, 0, p.ld, u->d_in, tb.order, v_t, 0, p.ld);
        k_units_transpose<E><<<dim3((p.ld + 31) / 32, (u->d_out + 31) / 32, 1), 256, 0, stream>>>(dout, 0, p.ld, u->d_out, tb.order, dout_t, 0, p.ld);
        launch_tc<DPre<E, BF>, 128>(dp, p.max_tiles, kTile, u->hidden, status, stream);
        launch_tc<DInput<E, BF>, 128>(di, p.max_tiles, kTile, u->d_in, status, stream);
        launch_tc<DWeight1<E, BF>, 128>(g1, p.max_segs, u->d_in, u->hidden, status, stream);
        if (u->d_out <= 64) launch_tc<DWeight2<E, BF>, 64>(g2, p.max_segs, u->hidden, u->d_out, status, stream);
        else launch_tc<DWeight2<E, BF>, 128>(g2, p.max_segs, u->hidden, u->d_out, status, stream);
        k_units_bgrad_t<<<dim3(M, u->hidden), 128, 0, stream>>>(dpre_t, p.ld, u->hidden, tb, db1);
        k_units_bgrad_t<<<dim3(M, u->d_out), 128, 0, stream>>>(dout_t, p.ld, u->d_out, tb, db2);
    } else {
        launch_simt(dp, p.max_tiles, kTile, u->hidden, stream);
        launch_simt(di, p.max_tiles, kTile, u->d_in, stream);
        launch_simt(g1, p.max_segs, u->d_in, u->hidden, stream);
        launch_simt(g2, p.max_segs, u->hidden, u->d_out, stream);
        k_units_bgrad<E, BF, true><<<dim3(M, (u->hidden + 31) / 32), 256, 0, stream>>>(dpre, u->hidden, tb, db1);
        k_units_bgrad<E, BF, false><<<dim3(M, (u->d_out + 31) / 32), 256, 0, stream>>>(dout, u->d_out, tb, db2);
    }
    const int64_t e1 = static_cast<int64_t>(u->d_in) * u->hidden, e2 = static_cast<int64_t>(u->hidden) * u->d_out;
    k_units_wgrad<BF><<<static_cast<unsigned>(std::min<int64_t>((e1 * M + 255) / 256, 4096)), 256, 0, stream>>>(partial1, e1, M, tb, dw1);
    k_units_wgrad<BF><<<static_cast<unsigned>(std::min<int64_t>((e2 * M + 255) / 256, 4096)), 256, 0, stream>>>(partial2, e2, M, tb, dw2);
    return hsnw_check_launch("units_backward");
}

int check_scratch(const Plan& p, void* scratch, int64_t bytes) {
    if (!scratch || bytes < static_cast<int64_t>(p.bytes) || (reinterpret_cast<uintptr_t>(scratch) & 255))
        return hsnw_fail(HSNW_E_ARG, "units: scratch too small or not 256-byte aligned (hsnw_units_scratch_bytes)");
    return HSNW_OK;
}

}  // namespace

extern "C" int64_t hsnw_units_scratch_bytes(const HsnwUnits* units, int64_t pairs, int backward) {
    if (!units || pairs < 0 || units->n_units < 1 || units->n_units > kMaxUnits) return 0;
    return static_cast<int64_t>(make_plan(units, pairs, backward != 0).bytes);
}

extern "C" int hsnw_units_forward(const HsnwUnits* units, const float* v, const int64_t* unit_idx, int64_t pairs, void* pre, void* out,
                                  void* scratch, int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check_units(units, pairs, "units_forward: null or negative")) return rc;
    const Plan p = make_plan(units, pairs, false);
    if (int rc = check_scratch(p, scratch, scratch_bytes)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int* status = static_cast<int*>(scratch);
    if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return hsnw_check_launch("units_forward");
    if (pairs == 0) return HSNW_OK;
    if (!v || !unit_idx || !pre || !out) return hsnw_fail(HSNW_E_ARG, "units_forward: null tensor");
    if ((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pre) | reinterpret_cast<uintptr_t>(out)) & 15)
        return hsnw_fail(HSNW_E_ARG, "units_forward: tensors not 16-byte aligned");
    const Tables tb = make_tables(p, scratch);
    hsnw_profile_mark(HSNW_K_UNITS_FWD, stream);
    if (int rc = sort_pairs(units, unit_idx, pairs, p, tb, status, stream)) return rc;
    if (units->prod_bf16)
        return forward_t<__nv_bfloat16, true>(units, v, pairs, static_cast<__nv_bfloat16*>(pre), static_cast<__nv_bfloat16*>(out), p, tb, scratch,
                                              status, stream);
    return forward_t<float, false>(units, v, pairs, static_cast<float*>(pre), static_cast<float*>(out), p, tb, scratch, status, stream);
}

extern "C" int hsnw_units_backward(const HsnwUnits* units, const float* v, const int64_t* unit_idx, int64_t pairs, const void* pre,
                                   const void* d_out, float* d_v, float* d_w1, float* d_b1, float* d_w2, float* d_b2, void* scratch,
                                   int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check_units(units, pairs, "units_backward: null or negative")) return rc;
    const Plan p = make_plan(units, pairs, true);
    if (int rc = check_scratch(p, scratch, scratch_bytes)) return rc;
    if (!d_w1 || !d_b1 || !d_w2 || !d_b2) return hsnw_fail(HSNW_E_ARG, "units_backward: null gradient");
    if (pairs > 0 && (!v || !unit_idx || !pre || !d_out || !d_v)) return hsnw_fail(HSNW_E_ARG, "units_backward: null tensor");
    if ((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(pre) | reinterpret_cast<uintptr_t>(d_out) | reinterpret_cast<uintptr_t>(d_v)
         | reinterpret_cast<uintptr_t>(d_w1) | reinterpret_cast<uintptr_t>(d_w2)) & 15)
        return hsnw_fail(HSNW_E_ARG, "units_backward: tensors not 16-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int* status = static_cast<int*>(scratch);
    if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return hsnw_check_launch("units_backward");
    if (pairs == 0) {   // no pair chose any unit: zero gradients
        const size_t m = static_cast<size_t>(units->n_units) * sizeof(float);
        if (cudaMemsetAsync(d_w1, 0, m * units->d_in * units->hidden, stream) != cudaSuccess
            || cudaMemsetAsync(d_b1, 0, m * units->hidden, stream) != cudaSuccess
            || cudaMemsetAsync(d_w2, 0, m * units->hidden * units->d_out, stream) != cudaSuccess
            || cudaMemsetAsync(d_b2, 0, m * units->d_out, stream) != cudaSuccess)
            return hsnw_check_launch("units_backward");
        return HSNW_OK;
    }
    const Tables tb = make_tables(p, scratch);
    hsnw_profile_mark(HSNW_K_UNITS_BWD, stream);
    if (int rc = sort_pairs(units, unit_idx, pairs, p, tb, status, stream)) return rc;
    if (units->prod_bf16)
        return backward_t<__nv_bfloat16, true>(units, v, pairs, static_cast<const __nv_bfloat16*>(pre), static_cast<const __nv_bfloat16*>(d_out),
                                               d_v, d_w1, d_b1, d_w2, d_b2, p, tb, scratch, status, stream);
    return backward_t<float, false>(units, v, pairs, static_cast<const float*>(pre), static_cast<const float*>(d_out), d_v, d_w1, d_b1, d_w2,
                                    d_b2, p, tb, scratch, status, stream);
}

void hsnw_units_set_attributes() {
    bool ok = true;
#define HSNW_UNITS_OPT(OP, BN) ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_units_tc<OP<__nv_bfloat16, true>, BN>), #OP)
    HSNW_UNITS_OPT(First, 128);
    HSNW_UNITS_OPT(Second, 64);
    HSNW_UNITS_OPT(Second, 128);
    HSNW_UNITS_OPT(DPre, 128);
    HSNW_UNITS_OPT(DInput, 128);
    HSNW_UNITS_OPT(DWeight1, 128);
    HSNW_UNITS_OPT(DWeight2, 64);
    HSNW_UNITS_OPT(DWeight2, 128);
#undef HSNW_UNITS_OPT
    if (!ok) hsnw_attribute_failed();
}
