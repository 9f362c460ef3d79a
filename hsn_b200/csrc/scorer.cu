// The replay's scorer logits over every cell of every window position, and the gradients of the scorer's
// weight and bias (reference python/hsn/train/split.py:305-342, _scorer_logits, and autograd's backward of
// it; the features are constants of the replay).
//
//   logits[r, n, :] = (W_h h[r, n] + (W_t [age[r, n] / age_max; scalars[r, n]] + b)) + W_row [u[r]; eps[r]]
//   d W_h = sum_{r, n} g[r, n]^T h[r, n],  d W_t, d b likewise,  d W_row = sum_r (sum_n g[r, n])^T [u[r]; eps[r]]
//
// Both passes are one read of the recorded state h (R N d floats: 0.5 GB for a B32 T256 N256 d64 window) and are
// bound by it. A persistent block takes tiles of 128 cells of one position: the tile of h (contiguous, 32 KB at
// d = 64) arrives by one bulk copy into one of three stages, two tiles ahead of the one the block works on; age and scalars
// (a few KB) go through registers into shared memory. Eight lanes share a cell, one per unit, and a warp works
// on four cells at a time: the eight lanes read the same 16 bytes of the cell's row (a broadcast), and the four
// cells read different quarters of their rows in the same instruction (cell c starts 2 c float4s further on and
// wraps around), so a warp's load touches every bank once; a lane keeps its unit's weights in registers in the
// order it meets them. The backward keeps a lane's gradient sums in registers over all of its block's tiles and
// reduces them once at the end: lanes of a warp in turn into shared memory, warps and then blocks in order, so
// two runs give the same bits.
#include "../../include/hsn_scorer_b200.h"
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "stage.cuh"
#include "host_util.h"
#include "umma.cuh"

#include <algorithm>

using namespace hsnw;

namespace {

constexpr int kCells = 128;    // cells of a tile
constexpr int kThreads = 256;  // 8 warps x 4 cells x 8 units
constexpr int kMaxTail = 16;   // 1 + scalars
constexpr int kRowChunks = 128; // partial sums of the row block's gradient
constexpr int kStages = 3;     // tiles of h in shared memory: the block works on one, two are on their way

struct Ctx {
    int d, N, M, S, F, tiles;
    float age_max;
    int64_t rows, items;
    const float *weight, *bias, *u, *eps, *h, *scalars;
    const int64_t* age;
    float* rowterm;         // [rows, M]
    float* logits;
    const float* dlogits;
    float* partial;         // [blocks][M][d + 1 + S + 1]: the state block, the tail block, the bias
    float* rowsum;          // [rows][tiles][M] sums of the cotangent over a tile's cells
    float* partial_row;     // [kRowChunks][M][2 d]
    int* status;
};

template <bool BF>
__device__ __forceinline__ float rnd(float x) {
    return BF ? bf16r(x) : x;
}

// rowterm[r, j] = [u[r]; eps[r]] . W[j, :2d]
template <bool BF>
__global__ void __launch_bounds__(256) k_scorer_row(Ctx c) {
    const int64_t e = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (e >= c.rows * c.M) return;
    const int64_t r = e / c.M;
    const int j = static_cast<int>(e - r * c.M);
    const float* w = c.weight + static_cast<int64_t>(j) * c.F;
    float sum = 0.0f;
    for (int x = 0; x < c.d; ++x) sum = fmaf(rnd<BF>(c.u[r * c.d + x]), rnd<BF>(w[x]), sum);
    for (int x = 0; x < c.d; ++x) sum = fmaf(rnd<BF>(c.eps[r * c.d + x]), rnd<BF>(w[c.d + x]), sum);
    c.rowterm[e] = rnd<BF>(sum);
}

// What the two passes share: the stages, the requests, a lane's place.
template <int D4, bool BF, int NS = kStages>
struct Tiles {
    static constexpr int d = 4 * D4;
    float* h_s;      // [NS][kCells * d]
    float* tail_s;   // [2][kCells * kMaxTail], a cell's [age / age_max, scalars] at pitch T1
    uint64_t* bar;
    const Ctx& c;
    int T1;
    float held[(kCells * (kMaxTail - 1) + kThreads - 1) / kThreads];   // the next tile's scalars and ages on their way to shared
    long long held_age;                                               // memory: loaded before the tile's work, stored after it

    __device__ Tiles(unsigned char* dyn, uint64_t* bars, const Ctx& ctx) : bar(bars), c(ctx) {
        h_s = reinterpret_cast<float*>(dyn);
        tail_s = h_s + NS * kCells * d;
        T1 = c.S + 1;
    }
    __device__ int cells_of(int64_t item) const { return min(kCells, c.N - static_cast<int>(item % c.tiles) * kCells); }
    __device__ int64_t first_cell(int64_t item) const { return (item / c.tiles) * c.N + (item % c.tiles) * kCells; }
    // thread 0: the tile of h into stage s
    __device__ void request(int64_t item, int s) const {
        const uint32_t bytes = static_cast<uint32_t>(cells_of(item)) * d * sizeof(float);
        mbar_expect_tx(&bar[s], bytes);
        bulk_g2s(h_s + s * kCells * d, c.h + first_cell(item) * d, bytes, &bar[s]);
    }
    __device__ void tail_load(int64_t item) {   // contiguous reads: a tile's scalars are one run, its ages another
        const int cells = cells_of(item);
        const int64_t cell0 = first_cell(item);
        held_age = static_cast<int>(threadIdx.x) < cells ? c.age[cell0 + threadIdx.x] : 0;
#pragma unroll
        for (int q = 0; q < static_cast<int>(sizeof(held) / sizeof(float)); ++q) {
            const int e = threadIdx.x + q * kThreads;
            held[q] = e < cells * c.S ? c.scalars[cell0 * c.S + e] : 0.0f;
        }
    }
    __device__ void tail_store(int s) const {
        float* t = tail_s + s * kCells * kMaxTail;
        if (threadIdx.x < kCells) t[threadIdx.x * T1] = rnd<BF>(static_cast<float>(held_age) / c.age_max);
#pragma unroll
        for (int q = 0; q < static_cast<int>(sizeof(held) / sizeof(float)); ++q) {
            const int e = threadIdx.x + q * kThreads;
            if (e < kCells * c.S) {
                const int cell = e / c.S;
                t[cell * T1 + 1 + (e - cell * c.S)] = rnd<BF>(held[q]);
            }
        }
    }
    // the bf16 pass reads h as bfloat16 values: round the landed tile in place, once for its eight readers
    __device__ void round_tile(int s, int cells) const {
        if (!BF) return;
        float4* t = reinterpret_cast<float4*>(h_s + s * kCells * d);
        for (int e = threadIdx.x; e < cells * D4; e += kThreads) {
            float4 v = t[e];
            v.x = bf16r(v.x), v.y = bf16r(v.y), v.z = bf16r(v.z), v.w = bf16r(v.w);
            t[e] = v;
        }
    }
};

// a lane's float4 number i of its cell's row: cell c of the warp's four starts 2 c further on (d = 16: c / 2)
template <int D4>
__device__ __forceinline__ int quarter(int i, int cc) {
    return (i + (D4 >= 8 ? 2 * cc : cc >> 1)) & (D4 - 1);
}

template <int D4, bool BF>
__global__ void __launch_bounds__(kThreads, D4 <= 16 ? 2 : 1) k_scorer_fwd(Ctx c) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t bar[kStages];
    constexpr int d = 4 * D4;
    Tiles<D4, BF> tl(dyn, bar, c);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cc = lane >> 3, j = lane & 7;
    const int T1 = tl.T1;
    if (tid == 0)
        for (int st = 0; st < kStages; ++st) mbar_init(&bar[st], 1);
    float4 wh[D4];
    float wt[kMaxTail], bj = 0.0f;
    {
        const float* w = c.weight + static_cast<int64_t>(min(j, c.M - 1)) * c.F;
#pragma unroll
        for (int i = 0; i < D4; ++i) {
            const float* p = w + 2 * d + 4 * quarter<D4>(i, cc);
            wh[i] = make_float4(rnd<BF>(p[0]), rnd<BF>(p[1]), rnd<BF>(p[2]), rnd<BF>(p[3]));
        }
#pragma unroll
        for (int s = 0; s < kMaxTail; ++s) wt[s] = s < T1 ? rnd<BF>(w[3 * d + s]) : 0.0f;
        bj = rnd<BF>(c.bias[min(j, c.M - 1)]);
    }
    int64_t item = blockIdx.x;
    if (item < c.items) {
        tl.tail_load(item);
        tl.tail_store(0);
    }
    __syncthreads();   // the barriers are initialised
    if (tid == 0)
        for (int k = 0; k < kStages - 1; ++k)
            if (item + k * static_cast<int64_t>(gridDim.x) < c.items) tl.request(item + k * static_cast<int64_t>(gridDim.x), k);
    for (int n_it = 0; item < c.items; item += gridDim.x, ++n_it) {
        const int s = n_it % kStages, ts = n_it & 1;
        const int64_t next = item + gridDim.x, ahead = item + (kStages - 1) * static_cast<int64_t>(gridDim.x);
        const int cells = tl.cells_of(item);
        mbar_wait(&bar[s], (n_it / kStages) & 1, c.status);
        tl.round_tile(s, cells);
        __syncthreads();   // tile s and its tail are complete; everyone is done with the stage of the tile before
        if (tid == 0 && ahead < c.items) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // that stage was read (and rounded) by ordinary accesses
            tl.request(ahead, (n_it + kStages - 1) % kStages);
        }
        if (next < c.items) tl.tail_load(next);
        const float* ht = tl.h_s + s * kCells * d;
        const float* tt = tl.tail_s + ts * kCells * kMaxTail;
        const int64_t r = item / c.tiles;
        const float row = j < c.M ? c.rowterm[r * c.M + j] : 0.0f;
        const int64_t cell0 = tl.first_cell(item);
#pragma unroll
        for (int round = 0; round < 4; ++round) {
            const int cell = warp * 16 + round * 4 + cc;
            if (cell < cells) {   // (a whole group of eight lanes at once)
                const float4* hp = reinterpret_cast<const float4*>(ht + cell * d);
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f, t0 = 0.0f, t1 = 0.0f;   // independent sums: no chain of 4 d additions
#pragma unroll
                for (int i = 0; i < D4; ++i) {
                    const float4 x = hp[quarter<D4>(i, cc)];
                    a0 = fmaf(x.x, wh[i].x, a0);
                    a1 = fmaf(x.y, wh[i].y, a1);
                    a2 = fmaf(x.z, wh[i].z, a2);
                    a3 = fmaf(x.w, wh[i].w, a3);
                }
#pragma unroll
                for (int sI = 0; sI < kMaxTail; sI += 2) {
                    if (sI < T1) t0 = fmaf(tt[cell * T1 + sI], wt[sI], t0);
                    if (sI + 1 < T1) t1 = fmaf(tt[cell * T1 + sI + 1], wt[sI + 1], t1);
                }
                if (j < c.M) c.logits[(cell0 + cell) * c.M + j] = (rnd<BF>((a0 + a1) + (a2 + a3)) + rnd<BF>((t0 + t1) + bj)) + row;
            }
        }
        if (next < c.items) tl.tail_store(ts ^ 1);
    }
}

// ---- bf16 products on the tensor cores (d = 64) ------------------------------------------------------------
// The state block's product of a tile is [128 cells, d] x [d, units]: one tcgen05.mma chain with the cells as
// the rows of A. The landed float32 tile is converted once to bfloat16 in the 128-byte swizzle (rows of 64
// elements, unit u of row r at u ^ (r % 8); d = 128: two such K blocks), which is at once A K-major for this
// product and, read the other way, B MN-major for the gradient's product [units, cells] x [cells, d].

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

// all threads: the float32 tile in stage memory -> the bfloat16 operand tile; rows past `cells` become zeros
template <int KB>
__device__ __forceinline__ void convert_tile(const float* h_tile, unsigned char* a_tile, int cells) {
    constexpr int d = 64 * KB;
    for (int e = threadIdx.x; e < kCells * 8 * KB; e += kThreads) {
        const int row = e / (8 * KB), u = e - row * (8 * KB), kb = u >> 3, uu = u & 7;
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (row < cells) {
            const float4 a = *reinterpret_cast<const float4*>(h_tile + row * d + 8 * u);
            const float4 b = *reinterpret_cast<const float4*>(h_tile + row * d + 8 * u + 4);
            packed = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
        }
        *reinterpret_cast<uint4*>(a_tile + kb * (kCells * 128) + row * 128 + ((uu ^ (row & 7)) << 4)) = packed;
    }
}

constexpr int kTcStages = 2;   // two blocks an SM take turns on the tensor cores; each has two tiles on their way (a stage is
                               // free as soon as its tile is converted)

// a tile's tail operand: thread (cell, half) holds [age / age_max, scalars] numbers 8 half .. 8 half + 7 of its cell
struct TailRegs {
    float v[8];
    long long age;
    __device__ void load(const Ctx& c, int64_t cell0, int cells) {
        const int cell = threadIdx.x >> 1, half = threadIdx.x & 1;
        age = -1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int k = 8 * half + i;   // 0: the age, k > 0: scalar k - 1
            v[i] = 0.0f;
            if (cell < cells) {
                if (k == 0) age = c.age[cell0 + cell];
                else if (k - 1 < c.S) v[i] = c.scalars[(cell0 + cell) * c.S + k - 1];
            }
        }
    }
    // as bfloat16 into the unswizzled K-major operand tile [2 planes][128 rows][16 bytes]
    __device__ void store(const Ctx& c, unsigned char* tile) const {
        const int cell = threadIdx.x >> 1, half = threadIdx.x & 1;
        const float first = age >= 0 ? static_cast<float>(age) / c.age_max : v[0];
        *reinterpret_cast<uint4*>(tile + half * (kCells * 16) + cell * 16) =
            make_uint4(pack_bf16x2(first, v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    }
};

template <int KB>
__global__ void __launch_bounds__(kThreads, 2) k_scorer_fwd_tc(Ctx c) {
    extern __shared__ unsigned char dyn_raw[];
    __shared__ __align__(8) uint64_t bar[kTcStages];
    __shared__ __align__(8) uint64_t bar_mma;
    __shared__ uint32_t tmem_slot;
    __shared__ float bias_s[8];
    constexpr int d = 64 * KB, D4 = d / 4;
    // (1024-aligned) the state operand tile | the state weights' tile | the tail operand tile | the tail weights' tile | float32 stages
    unsigned char* dyn = dyn_raw + ((1024u - (smem_addr(dyn_raw) & 1023u)) & 1023u);
    unsigned char* a_tile = dyn;                           // KB x [128 rows x 128 bytes], 128-byte swizzle
    unsigned char* b_tile = a_tile + KB * kCells * 128;    // KB x [16 rows x 128 bytes]: the units, padded with zero rows
    unsigned char* a2_tile = b_tile + KB * 16 * 128;       // [2 planes][128 rows][16 bytes], unswizzled: a cell's 16 tail numbers
    unsigned char* b2_tile = a2_tile + 2 * kCells * 16;    // [2 planes][16 rows][16 bytes]
    Tiles<D4, true, kTcStages> tl(b2_tile + 2 * 16 * 16, bar, c);
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        for (int st = 0; st < kTcStages; ++st) mbar_init(&bar[st], 1);
        mbar_init(&bar_mma, 1);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 32);
    for (int e = tid; e < 16 * 8 * KB; e += kThreads) {   // W[:, 2d:3d] as the B operand: row = unit, K = d
        const int row = e / (8 * KB), u = e - row * (8 * KB), kb = u >> 3, uu = u & 7;
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (row < c.M) {
            const float* w = c.weight + static_cast<int64_t>(row) * c.F + 2 * d + 8 * u;
            packed = make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]), pack_bf16x2(w[4], w[5]), pack_bf16x2(w[6], w[7]));
        }
        *reinterpret_cast<uint4*>(b_tile + kb * (16 * 128) + row * 128 + ((uu ^ (row & 7)) << 4)) = packed;
    }
    if (tid < 32) {   // W[:, 3d:] as the tail product's B operand: (plane, unit) -> 8 weights
        const int plane = tid >> 4, unit = tid & 15;
        float w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int k = 8 * plane + i;
            w[i] = (unit < c.M && k <= c.S) ? c.weight[static_cast<int64_t>(unit) * c.F + 3 * d + k] : 0.0f;
        }
        *reinterpret_cast<uint4*>(b2_tile + plane * (16 * 16) + unit * 16) =
            make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]), pack_bf16x2(w[4], w[5]), pack_bf16x2(w[6], w[7]));
    }
    if (tid < 8) bias_s[tid] = tid < c.M ? bf16r(c.bias[tid]) : 0.0f;
    TailRegs tail;
    int64_t item = blockIdx.x;
    if (item < c.items) {
        tail.load(c, tl.first_cell(item), tl.cells_of(item));
        tail.store(c, a2_tile);
    }
    tcgen05_fence_before();
    __syncthreads();   // the barriers, tensor memory and the weights' tiles are in place
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    const uint32_t idesc = umma_idesc_bf16(128, 16);
    if (tid == 0)
        for (int k = 0; k < kTcStages; ++k)
            if (item + k * static_cast<int64_t>(gridDim.x) < c.items) tl.request(item + k * static_cast<int64_t>(gridDim.x), k);
    for (int n_it = 0; item < c.items; item += gridDim.x, ++n_it) {
        const int s = n_it % kTcStages;
        const int64_t next = item + gridDim.x, ahead = item + kTcStages * static_cast<int64_t>(gridDim.x);
        const int cells = tl.cells_of(item);
        mbar_wait(&bar[s], (n_it / kTcStages) & 1, c.status);
        convert_tile<KB>(tl.h_s + s * kCells * d, a_tile, cells);   // (the last tile's products were waited for before its epilogue)
        fence_async_smem();
        __syncthreads();   // both operand tiles are complete; the float32 stage has been read: it is free again
        if (tid < 32) {    // the whole first warp, converged after the barrier: one elected lane issues
            tcgen05_fence_after();
            __syncwarp();
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {   // a K block of 64 is one 128-byte row: a K = 16 step moves both operands by 32 bytes
                const uint64_t da = umma_desc_sw128(a_tile + kb * (kCells * 128)), db = umma_desc_sw128(b_tile + kb * (16 * 128));
#pragma unroll
                for (int st = 0; st < 4; ++st) umma_bf16(taddr, da + 2 * st, db + 2 * st, idesc, kb > 0 || st > 0);
            }
            umma_bf16(taddr + 16, umma_desc(a2_tile, kCells), umma_desc(b2_tile, 16), idesc, false);   // the tail block: its own sum
            umma_commit(&bar_mma);
        }
        if (tid == 0 && ahead < c.items) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the stage was read by ordinary loads
            tl.request(ahead, s);
        }
        if (next < c.items) tail.load(c, tl.first_cell(next), tl.cells_of(next));
        mbar_wait(&bar_mma, n_it & 1, c.status);
        tcgen05_fence_after();
        if (warp < 4) {   // a thread a cell: the two sums' 8 units, the bias, the row term
            float state[8], rest[8];
            tmem_ld8(tmem_addr(taddr, warp * 32, 0), state);
            tmem_ld8(tmem_addr(taddr, warp * 32, 16), rest);
            const int cell = tid;
            if (cell < cells) {
                const int64_t r = item / c.tiles;
                float out[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    out[j] = (bf16r(state[j]) + bf16r(rest[j] + bias_s[j])) + (j < c.M ? c.rowterm[r * c.M + j] : 0.0f);
                float* dst = c.logits + (tl.first_cell(item) + cell) * c.M;
                if (c.M == 8) {
                    *reinterpret_cast<float4*>(dst) = make_float4(out[0], out[1], out[2], out[3]);
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(out[4], out[5], out[6], out[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (j < c.M) dst[j] = out[j];
                }
            }
        }
        tcgen05_fence_before();
        if (next < c.items) tail.store(c, a2_tile);   // (this tile's products have read the tile: waited for above)
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, 32);
}

// The gradients of the state block and of the tail block (with the bias as a column of ones) as two accumulating
// products over all of a block's tiles: D1 [units, d] += g^T [units, cells] x h [cells, d], D2 [units, 16] += g^T x
// [tail, 1] [cells, 16]. g^T is the A operand (K = the cells; 8 rows in the 128-byte swizzle, which every row group
// of the product's 128 rows reads again), h is the forward's bfloat16 tile read as B MN-major (a K row = a cell's 64 elements =
// one 128-byte swizzled row), the tail is written transposed as B K-major. Nothing is read back per tile: the
// accumulators stay in tensor memory until the block's last tile.
constexpr int kBwdStages = 2;
__global__ void __launch_bounds__(kThreads, 2) k_scorer_bwd_tc(Ctx c) {
    extern __shared__ unsigned char dyn_raw[];
    __shared__ __align__(8) uint64_t bar[kBwdStages];
    __shared__ __align__(8) uint64_t bar_mma[2];   // the products of a tile have read operand set (tile & 1)
    __shared__ uint32_t tmem_slot;
    __shared__ float part_s[2][16][8];   // a tile's raw cotangent summed over 8 cells, per plane and unit
    constexpr int d = 64, D4 = 16;
    unsigned char* dyn = dyn_raw + ((1024u - (smem_addr(dyn_raw) & 1023u)) & 1023u);
    constexpr int kSet = kCells * 128 + 2 * 8 * 128 + 16 * 16 * 16;   // two sets of the three operand tiles: a tile is staged
    unsigned char* h_tile = dyn;                        // beside the products of the one before. [128 cells x 128 bytes], 128-byte swizzle
    unsigned char* g_tile = h_tile + kCells * 128;      // [2 K blocks of 64 cells][8 rows x 128 bytes], 128-byte swizzle: g^T; the
                                                        // descriptor's stride between row groups is zero, so the product's rows
                                                        // 8 .. 127 repeat rows 0 .. 7 (never read)
    unsigned char* t_tile = g_tile + 2 * 8 * 128;       // [16 planes][16 rows][16 bytes]: the tail and the ones, transposed
    Tiles<D4, true, kBwdStages> tl(dyn + 2 * kSet, bar, c);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int T1 = tl.T1;
    if (tid == 0) {
        for (int st = 0; st < kBwdStages; ++st) mbar_init(&bar[st], 1);
        mbar_init(&bar_mma[0], 1);
        mbar_init(&bar_mma[1], 1);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 128);
    for (int e = tid; e < 16 * 16; e += kThreads) {
        reinterpret_cast<uint4*>(t_tile)[e] = make_uint4(0u, 0u, 0u, 0u);
        reinterpret_cast<uint4*>(t_tile + kSet)[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    TailRegs tail;
    // thread (cell, half) writes its 8 tail numbers (and the one) into rows 8 half .. of column `cell`
    auto tail_store = [&](int cells, int set) {
        const int cell = tid >> 1, half = tid & 1;
        __nv_bfloat16* col = reinterpret_cast<__nv_bfloat16*>(t_tile + set * kSet + (cell >> 3) * (16 * 16)) + (cell & 7);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int k = 8 * half + i;
            float v = k == 0 ? (tail.age >= 0 ? static_cast<float>(tail.age) / c.age_max : 0.0f) : tail.v[i];
            if (k == T1) v = 1.0f;   // the bias: a column of ones
            if (cell >= cells) v = 0.0f;
            col[k * 8] = __float2bfloat16_rn(v);
        }
    };
    int64_t item = blockIdx.x;
    if (item < c.items) tail.load(c, tl.first_cell(item), tl.cells_of(item));
    tcgen05_fence_before();
    __syncthreads();   // the barriers, tensor memory and the zeroed tiles are in place
    tcgen05_fence_after();
    if (item < c.items) tail_store(tl.cells_of(item), 0);
    const uint32_t taddr = tmem_slot;
    const uint32_t idesc_state = umma_idesc_bf16(128, 64) | (1u << 16);   // B MN-major
    const uint32_t idesc_tail = umma_idesc_bf16(128, 16);
    if (tid == 0)
        for (int k = 0; k < kBwdStages; ++k)
            if (item + k * static_cast<int64_t>(gridDim.x) < c.items) tl.request(item + k * static_cast<int64_t>(gridDim.x), k);
    int n_it = 0;
    int64_t last_item = -1;
    float g[8];   // threads 0..127: the tile's cotangent for 8 cells of one unit, requested a tile ahead
    auto g_load = [&](int64_t it) {
        const int n = tl.cells_of(it);
        const int64_t first = tl.first_cell(it);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int cell = 8 * (tid >> 3) + i;
            g[i] = (tid < 128 && cell < n && (tid & 7) < c.M) ? c.dlogits[(first + cell) * c.M + (tid & 7)] : 0.0f;
        }
    };
    if (item < c.items) g_load(item);
    for (; item < c.items; item += gridDim.x, ++n_it) {
        const int s = n_it % kBwdStages, ts = n_it & 1;
        const int64_t next = item + gridDim.x, ahead = item + kBwdStages * static_cast<int64_t>(gridDim.x);
        const int cells = tl.cells_of(item);
        const int unit = tid & 7, plane = tid >> 3;   // threads 0..127: 8 cells of one unit
        mbar_wait(&bar[s], (n_it / kBwdStages) & 1, c.status);
        const int set = n_it & 1;
        if (n_it > 1) mbar_wait(&bar_mma[set], ((n_it >> 1) - 1) & 1, c.status);   // the products of two tiles ago have read this set
        convert_tile<1>(tl.h_s + s * kCells * d, h_tile + set * kSet, cells);
        if (tid < 128) {
            *reinterpret_cast<uint4*>(g_tile + set * kSet + (plane >> 3) * (8 * 128) + unit * 128 + (((plane & 7) ^ unit) << 4)) =
                make_uint4(pack_bf16x2(g[0], g[1]), pack_bf16x2(g[2], g[3]), pack_bf16x2(g[4], g[5]), pack_bf16x2(g[6], g[7]));
            part_s[ts][plane][unit] = ((g[0] + g[1]) + (g[2] + g[3])) + ((g[4] + g[5]) + (g[6] + g[7]));
        }
        if (n_it > 0) tail_store(cells, set);   // (the first tile's went in before the loop)
        fence_async_smem();
        __syncthreads();   // the operand tiles are complete; the float32 stage has been read: it is free again
        if (tid < 32) {
            tcgen05_fence_after();
            __syncwarp();
            const uint64_t no_stride = ~(static_cast<uint64_t>(0x3fffu) << 32);   // the row groups of g^T all start at its first
            const uint64_t db = umma_desc_sw128(h_tile + set * kSet), dt = umma_desc(t_tile + set * kSet, 16);
#pragma unroll
            for (int st = 0; st < 8; ++st) {   // 16 cells a step
                const uint64_t da = (umma_desc_sw128(g_tile + set * kSet + (st >> 2) * (8 * 128)) & no_stride) + 2u * (st & 3);
                umma_bf16(taddr, da, db + st * 128u, idesc_state, n_it > 0 || st > 0);
                umma_bf16(taddr + 64, da, dt + st * umma_kstep(16), idesc_tail, n_it > 0 || st > 0);
            }
            umma_commit(&bar_mma[set]);
        }
        if (tid < 8 && tid < c.M) {   // the tile's raw cotangent summed over its cells, planes in order
            float total = 0.0f;
#pragma unroll
            for (int p = 0; p < 16; ++p) total += part_s[ts][p][tid];
            c.rowsum[item * c.M + tid] = total;
        }
        if (tid == 0 && ahead < c.items) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            tl.request(ahead, s);
        }
        if (next < c.items) {
            tail.load(c, tl.first_cell(next), tl.cells_of(next));
            g_load(next);   // (this tile's were packed into the operand tile before the barrier)
        }
        last_item = item;
    }
    if (n_it > 0) mbar_wait(&bar_mma[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, c.status);   // the last commit covers every product before it
    tcgen05_fence_after();
    const int width = d + T1 + 1;
    if (warp == 0) {   // lanes = units: the block's sums out of tensor memory
        const int lane = tid;
        float* dst = c.partial + (static_cast<int64_t>(blockIdx.x) * c.M + lane) * width;
        float x[8];
#pragma unroll
        for (int cb = 0; cb < 64; cb += 8) {
            tmem_ld8(tmem_addr(taddr, 0, cb), x);
            if (lane < c.M && last_item >= 0)
#pragma unroll
                for (int i = 0; i < 8; ++i) dst[cb + i] = x[i];
        }
#pragma unroll
        for (int cb = 0; cb < 16; cb += 8) {
            tmem_ld8(tmem_addr(taddr, 0, 64 + cb), x);
            if (lane < c.M && last_item >= 0)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (cb + i <= T1) dst[d + cb + i] = x[i];   // the tail block, then the bias at d + T1
        }
        if (lane < c.M && last_item < 0)
            for (int e = 0; e < width; ++e) dst[e] = 0.0f;
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, 128);
}

template <int D4, bool BF>
__global__ void __launch_bounds__(kThreads, D4 <= 16 ? 2 : 1) k_scorer_bwd(Ctx c) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t bar[kStages];
    __shared__ float warp_sum_s[2][8][8];   // a tile's cotangent summed over a warp's cells, per unit
    constexpr int d = 4 * D4;
    Tiles<D4, BF> tl(dyn, bar, c);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cc = lane >> 3, j = lane & 7;
    const int T1 = tl.T1;
    if (tid == 0)
        for (int st = 0; st < kStages; ++st) mbar_init(&bar[st], 1);
    float4 ah[D4];
    float at[kMaxTail], ab = 0.0f;
#pragma unroll
    for (int i = 0; i < D4; ++i) ah[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int s = 0; s < kMaxTail; ++s) at[s] = 0.0f;
    int64_t item = blockIdx.x, last_item = -1;
    if (item < c.items) {
        tl.tail_load(item);
        tl.tail_store(0);
    }
    __syncthreads();
    if (tid == 0)
        for (int k = 0; k < kStages - 1; ++k)
            if (item + k * static_cast<int64_t>(gridDim.x) < c.items) tl.request(item + k * static_cast<int64_t>(gridDim.x), k);
    int n_it = 0;
    for (; item < c.items; item += gridDim.x, ++n_it) {
        const int s = n_it % kStages, ts = n_it & 1;
        const int64_t next = item + gridDim.x, ahead = item + (kStages - 1) * static_cast<int64_t>(gridDim.x);
        const int cells = tl.cells_of(item);
        const int64_t cell0 = tl.first_cell(item);
        float g[4];
#pragma unroll
        for (int round = 0; round < 4; ++round) {   // the tile's cotangent: 128 contiguous bytes a warp load
            const int cell = warp * 16 + round * 4 + cc;
            g[round] = (cell < cells && j < c.M) ? c.dlogits[(cell0 + cell) * c.M + j] : 0.0f;
        }
        mbar_wait(&bar[s], (n_it / kStages) & 1, c.status);
        tl.round_tile(s, cells);
        __syncthreads();   // tile s and its tail are complete; everyone is done with the tile before and its sums are written
        if (last_item >= 0 && tid < 8 && tid < c.M) {   // the last tile's cotangent summed over its cells, warps in order
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) total += warp_sum_s[ts ^ 1][w][tid];
            c.rowsum[last_item * c.M + tid] = total;
        }
        if (tid == 0 && ahead < c.items) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            tl.request(ahead, (n_it + kStages - 1) % kStages);
        }
        if (next < c.items) tl.tail_load(next);
        const float* ht = tl.h_s + s * kCells * d;
        const float* tt = tl.tail_s + ts * kCells * kMaxTail;
        float raw = 0.0f;
#pragma unroll
        for (int round = 0; round < 4; ++round) {
            const int cell = warp * 16 + round * 4 + cc;
            raw += g[round];
            if (cell < cells) {
                const float gr = rnd<BF>(g[round]);
                const float4* hp = reinterpret_cast<const float4*>(ht + cell * d);
#pragma unroll
                for (int i = 0; i < D4; ++i) {
                    const float4 x = hp[quarter<D4>(i, cc)];
                    ah[i].x = fmaf(gr, x.x, ah[i].x);
                    ah[i].y = fmaf(gr, x.y, ah[i].y);
                    ah[i].z = fmaf(gr, x.z, ah[i].z);
                    ah[i].w = fmaf(gr, x.w, ah[i].w);
                }
#pragma unroll
                for (int sI = 0; sI < kMaxTail; ++sI)
                    if (sI < T1) at[sI] = fmaf(gr, tt[cell * T1 + sI], at[sI]);
                ab += gr;
            }
        }
        raw += __shfl_xor_sync(0xffffffffu, raw, 8);
        raw += __shfl_xor_sync(0xffffffffu, raw, 16);
        if (cc == 0) warp_sum_s[ts][warp][j] = raw;
        last_item = item;
        if (next < c.items) tl.tail_store(ts ^ 1);
    }
    __syncthreads();
    if (last_item >= 0 && tid < 8 && tid < c.M) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += warp_sum_s[(n_it - 1) & 1][w][tid];
        c.rowsum[last_item * c.M + tid] = total;
    }
    // a block's sums: the four cells' lanes of a warp in turn into the warp's slice of shared memory (the stages
    // are free now), then the warps in order
    const int width = d + T1 + 1;
    float* red = reinterpret_cast<float*>(dyn);   // [8 warps][8 units][width]
    float* mine = red + (warp * 8 + j) * width;
    for (int turn = 0; turn < 4; ++turn) {
        if (cc == turn) {
#pragma unroll
            for (int i = 0; i < D4; ++i) {
                float* at4 = mine + 4 * quarter<D4>(i, cc);
                if (turn == 0) at4[0] = ah[i].x, at4[1] = ah[i].y, at4[2] = ah[i].z, at4[3] = ah[i].w;
                else at4[0] += ah[i].x, at4[1] += ah[i].y, at4[2] += ah[i].z, at4[3] += ah[i].w;
            }
#pragma unroll
            for (int sI = 0; sI < kMaxTail; ++sI)
                if (sI < T1) mine[d + sI] = turn == 0 ? at[sI] : mine[d + sI] + at[sI];
            mine[d + T1] = turn == 0 ? ab : mine[d + T1] + ab;
        }
        __syncwarp();
    }
    __syncthreads();
    for (int e = tid; e < c.M * width; e += kThreads) {
        const int unit = e / width, col = e - unit * width;
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) total += red[(w * 8 + unit) * width + col];
        c.partial[static_cast<int64_t>(blockIdx.x) * c.M * width + e] = total;
    }
}

// the row block's gradient: a chunk of positions -> partial_row[chunk][unit][input]. The chunk's cotangents
// (a position's, summed over its tiles, rounded as the row map's cotangent is) go to shared memory; a thread
// then owns an input column and four units and walks the chunk's rows, whose loads do not depend on one another.
template <bool BF>
__global__ void __launch_bounds__(256) k_scorer_rowgrad(Ctx c) {
    __shared__ float g_s[64][8];
    const int64_t per = (c.rows + kRowChunks - 1) / kRowChunks;   // at most 64 a block: the host splits the chunks so
    const int64_t r0 = blockIdx.x * per, r1 = min(c.rows, r0 + per);
    const int n = static_cast<int>(max(static_cast<int64_t>(0), r1 - r0)), two_d = 2 * c.d, tid = threadIdx.x;
    float* out = c.partial_row + static_cast<int64_t>(blockIdx.x) * c.M * two_d;
    for (int base = 0; base < max(n, 1); base += 64) {   // (n <= 64 with the host's chunks; the loop keeps any n right)
        const int m = min(64, n - base);
        __syncthreads();
        for (int e = tid; e < 64 * 8; e += 256) {
            const int rr = e >> 3, unit = e & 7;
            float g = 0.0f;
            if (rr < m && unit < c.M)
                for (int t = 0; t < c.tiles; ++t) g += c.rowsum[((r0 + base + rr) * c.tiles + t) * c.M + unit];
            g_s[rr][unit] = rnd<BF>(g);
        }
        __syncthreads();
        for (int x = tid & 127; x < two_d; x += 128) {
            const int u0 = 4 * (tid >> 7);
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 8
            for (int rr = 0; rr < m; ++rr) {
                const int64_t r = r0 + base + rr;
                const float in = rnd<BF>(x < c.d ? c.u[r * c.d + x] : c.eps[r * c.d + x - c.d]);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = fmaf(g_s[rr][u0 + k], in, acc[k]);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (u0 + k < c.M) out[(u0 + k) * two_d + x] = (base == 0 ? 0.0f : out[(u0 + k) * two_d + x]) + acc[k];
        }
    }
}

// d_weight and d_bias from the blocks' and the row chunks' partial sums: a warp an output, a lane every 32nd
// partial in order, then a fixed tree over the lanes (the same bits every run)
template <bool BF>
__global__ void __launch_bounds__(256) k_scorer_wgrad(Ctx c, int blocks, float* d_weight, float* d_bias) {
    const int width = c.d + c.S + 2, two_d = 2 * c.d;
    const int e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= c.M * (c.F + 1)) return;
    const int unit = e / (c.F + 1), col = e - unit * (c.F + 1);   // col F: the bias
    float total = 0.0f;
    if (col < two_d) {
        for (int k = lane; k < kRowChunks; k += 32) total += c.partial_row[(static_cast<int64_t>(k) * c.M + unit) * two_d + col];
    } else {
        const int at = col - two_d;   // the state block, the tail block, the bias: the blocks' layout
        for (int b = lane; b < blocks; b += 32) total += c.partial[(static_cast<int64_t>(b) * c.M + unit) * width + at];
    }
    total = warp_sum(total);
    if (lane == 0) {
        if (col < c.F) d_weight[unit * c.F + col] = rnd<BF>(total);
        else d_bias[unit] = rnd<BF>(total);
    }
}

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct Plan {
    int tiles, blocks, blocks_tc, blocks_bwd;
    size_t shared;
    size_t off_rowterm, off_partial, off_rowsum, off_partial_row, bytes;
};

Plan make_plan(const HsnwScorer* s, int64_t rows, bool backward) {
    Plan p{};
    p.tiles = (s->n_cells + kCells - 1) / kCells;
    p.shared = sizeof(float) * (kStages * kCells * static_cast<size_t>(s->d) + 2 * kCells * kMaxTail);
    const int sms = std::max(1, hsnw_sm_count_current());
    const int per_sm = static_cast<int>(std::max<size_t>(1, std::min<size_t>(2, (226 * 1024) / (p.shared + 1024))));   // (128 registers a thread: two blocks)
    p.blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(rows * p.tiles, static_cast<int64_t>(sms) * per_sm)));
    p.blocks_tc = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(rows * p.tiles, 2 * static_cast<int64_t>(sms))));   // two blocks an SM
    p.blocks_bwd = (s->prod_bf16 && s->d == 64 && s->n_scalars + 2 <= kMaxTail) ? p.blocks_tc : p.blocks;
    size_t at = 256;
    p.off_rowterm = at;
    at += up256(sizeof(float) * static_cast<size_t>(rows) * s->n_units);
    if (backward) {
        p.off_partial = at;
        at += up256(sizeof(float) * static_cast<size_t>(p.blocks_bwd) * s->n_units * (s->d + s->n_scalars + 2));
        p.off_rowsum = at;
        at += up256(sizeof(float) * static_cast<size_t>(rows) * p.tiles * s->n_units);
        p.off_partial_row = at;
        at += up256(sizeof(float) * kRowChunks * s->n_units * 2 * s->d);
    }
    p.bytes = at;
    return p;
}

int check(const HsnwScorer* s, int64_t rows, const char* what) {
    if (!s || rows < 0) return hsnw_fail(HSNW_E_ARG, what);
    if (s->d < 4 || s->n_cells < 1 || s->n_units < 1 || s->n_scalars < 0 || !s->weight || !s->bias || !(s->age_max > 0.0f))
        return hsnw_fail(HSNW_E_ARG, "scorer: sizes, age_max or weights missing");
    if ((s->d != 16 && s->d != 32 && s->d != 64 && s->d != 128) || s->n_units > 8 || s->n_scalars + 1 > kMaxTail)
        return hsnw_fail(HSNW_E_UNSUPPORTED, "scorer: d in {16, 32, 64, 128}, at most 8 units, at most 15 scalars");
    return HSNW_OK;
}

Ctx make_ctx(const HsnwScorer* s, const Plan& p, const float* u, const float* eps, const float* h, const int64_t* age, const float* scalars,
             int64_t rows, void* scratch) {
    unsigned char* base = static_cast<unsigned char*>(scratch);
    Ctx c{};
    c.d = s->d, c.N = s->n_cells, c.M = s->n_units, c.S = s->n_scalars, c.F = 3 * s->d + 1 + s->n_scalars, c.tiles = p.tiles;
    c.age_max = s->age_max;
    c.rows = rows, c.items = rows * p.tiles;
    c.weight = s->weight, c.bias = s->bias, c.u = u, c.eps = eps, c.h = h, c.scalars = scalars, c.age = age;
    c.rowterm = reinterpret_cast<float*>(base + p.off_rowterm);
    c.partial = reinterpret_cast<float*>(base + p.off_partial);
    c.rowsum = reinterpret_cast<float*>(base + p.off_rowsum);
    c.partial_row = reinterpret_cast<float*>(base + p.off_partial_row);
    c.status = reinterpret_cast<int*>(base);
    return c;
}

size_t tc_shared(int d) {   // 1024 of slack for the alignment, the two operand tiles, then the stages and the tail tiles
    const int KB = d / 64;
    return 1024 + static_cast<size_t>(KB) * (kCells + 16) * 128 + 2 * (kCells + 16) * 16 + sizeof(float) * (kTcStages * kCells * static_cast<size_t>(d) + 2 * kCells * kMaxTail);
}

template <bool BF>
void launch_fwd(const Ctx& c, const Plan& p, cudaStream_t stream) {
    if (BF && c.d == 64) {
        k_scorer_fwd_tc<1><<<p.blocks_tc, kThreads, tc_shared(64), stream>>>(c);
        return;
    }
    switch (c.d) {
        case 16: k_scorer_fwd<4, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
        case 32: k_scorer_fwd<8, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
        case 64: k_scorer_fwd<16, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
        default: k_scorer_fwd<32, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
    }
}
size_t tc_shared_bwd() {   // the alignment's slack, the three operand tiles, the stages (and the tail tiles the stage helper lays out)
    return 1024 + 2 * (kCells * 128 + 2 * 8 * 128 + 16 * 16 * 16) + sizeof(float) * (kBwdStages * kCells * 64);
}

template <bool BF>
void launch_bwd(const Ctx& c, const Plan& p, cudaStream_t stream) {
    if (BF && c.d == 64 && c.S + 2 <= kMaxTail) {   // (make_plan's condition for blocks_bwd)
        k_scorer_bwd_tc<<<p.blocks_bwd, kThreads, tc_shared_bwd(), stream>>>(c);
        return;
    }
    switch (c.d) {
        case 16: k_scorer_bwd<4, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
        case 32: k_scorer_bwd<8, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
        case 64: k_scorer_bwd<16, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
        default: k_scorer_bwd<32, BF><<<p.blocks, kThreads, p.shared, stream>>>(c); break;
    }
}

int check_call(const Plan& p, const void* u, const void* eps, const void* h, const void* age, const void* scalars, int n_scalars,
               void* scratch, int64_t bytes) {
    if (!u || !eps || !h || !age || (n_scalars > 0 && !scalars)) return hsnw_fail(HSNW_E_ARG, "scorer: null tensor");
    if (reinterpret_cast<uintptr_t>(h) & 15) return hsnw_fail(HSNW_E_ARG, "scorer: h not 16-byte aligned");
    if (!scratch || bytes < static_cast<int64_t>(p.bytes) || (reinterpret_cast<uintptr_t>(scratch) & 255))
        return hsnw_fail(HSNW_E_ARG, "scorer: scratch too small or not 256-byte aligned (hsnw_scorer_scratch_bytes)");
    return HSNW_OK;
}

}  // namespace

extern "C" int64_t hsnw_scorer_scratch_bytes(const HsnwScorer* scorer, int64_t rows, int backward) {
    if (!scorer || rows < 0 || scorer->n_units < 1 || scorer->d < 4 || scorer->n_cells < 1) return 0;
    return static_cast<int64_t>(make_plan(scorer, rows, backward != 0).bytes);
}

extern "C" int hsnw_scorer_logits(const HsnwScorer* scorer, const float* u, const float* eps, const float* h, const int64_t* age,
                                  const float* scalars, int64_t rows, float* logits, void* scratch, int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(scorer, rows, "scorer_logits: null or negative")) return rc;
    const Plan p = make_plan(scorer, rows, false);
    if (rows == 0) return HSNW_OK;
    if (int rc = check_call(p, u, eps, h, age, scalars, scorer->n_scalars, scratch, scratch_bytes)) return rc;
    if (!logits) return hsnw_fail(HSNW_E_ARG, "scorer_logits: null output");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    Ctx c = make_ctx(scorer, p, u, eps, h, age, scalars, rows, scratch);
    c.logits = logits;
    if (cudaMemsetAsync(c.status, 0, sizeof(int), stream) != cudaSuccess) return hsnw_check_launch("scorer_logits");
    hsnw_profile_mark(HSNW_K_SCORER_FWD, stream);
    const unsigned row_blocks = static_cast<unsigned>((rows * c.M + 255) / 256);
    if (scorer->prod_bf16) {
        k_scorer_row<true><<<row_blocks, 256, 0, stream>>>(c);
        launch_fwd<true>(c, p, stream);
    } else {
        k_scorer_row<false><<<row_blocks, 256, 0, stream>>>(c);
        launch_fwd<false>(c, p, stream);
    }
    return hsnw_check_launch("scorer_logits");
}

extern "C" int hsnw_scorer_logits_backward(const HsnwScorer* scorer, const float* u, const float* eps, const float* h, const int64_t* age,
                                           const float* scalars, int64_t rows, const float* d_logits, float* d_weight, float* d_bias,
                                           void* scratch, int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check(scorer, rows, "scorer_logits_backward: null or negative")) return rc;
    if (!d_weight || !d_bias) return hsnw_fail(HSNW_E_ARG, "scorer_logits_backward: null gradient");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int F = 3 * scorer->d + 1 + scorer->n_scalars;
    if (rows == 0) {
        if (cudaMemsetAsync(d_weight, 0, sizeof(float) * scorer->n_units * F, stream) != cudaSuccess
            || cudaMemsetAsync(d_bias, 0, sizeof(float) * scorer->n_units, stream) != cudaSuccess)
            return hsnw_check_launch("scorer_logits_backward");
        return HSNW_OK;
    }
    const Plan p = make_plan(scorer, rows, true);
    if (int rc = check_call(p, u, eps, h, age, scalars, scorer->n_scalars, scratch, scratch_bytes)) return rc;
    if (!d_logits) return hsnw_fail(HSNW_E_ARG, "scorer_logits_backward: null cotangent");
    Ctx c = make_ctx(scorer, p, u, eps, h, age, scalars, rows, scratch);
    c.dlogits = d_logits;
    if (cudaMemsetAsync(c.status, 0, sizeof(int), stream) != cudaSuccess) return hsnw_check_launch("scorer_logits_backward");
    hsnw_profile_mark(HSNW_K_SCORER_BWD, stream);
    const unsigned out_blocks = static_cast<unsigned>((c.M * (F + 1) + 7) / 8);   // a warp an output
    if (scorer->prod_bf16) {
        launch_bwd<true>(c, p, stream);
        k_scorer_rowgrad<true><<<kRowChunks, 256, 0, stream>>>(c);
        k_scorer_wgrad<true><<<out_blocks, 256, 0, stream>>>(c, p.blocks_bwd, d_weight, d_bias);
    } else {
        launch_bwd<false>(c, p, stream);
        k_scorer_rowgrad<false><<<kRowChunks, 256, 0, stream>>>(c);
        k_scorer_wgrad<false><<<out_blocks, 256, 0, stream>>>(c, p.blocks_bwd, d_weight, d_bias);
    }
    return hsnw_check_launch("scorer_logits_backward");
}

void hsnw_scorer_set_attributes() {
    bool ok = true;
#define HSNW_SCORER_OPT(D4) \
    ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_scorer_fwd<D4, true>), "scorer_fwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_scorer_fwd<D4, false>), "scorer_fwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_scorer_bwd<D4, true>), "scorer_bwd") \
         && hsnw_opt_in(reinterpret_cast<const void*>(k_scorer_bwd<D4, false>), "scorer_bwd")
    HSNW_SCORER_OPT(4);
    HSNW_SCORER_OPT(8);
    HSNW_SCORER_OPT(16);
    HSNW_SCORER_OPT(32);
#undef HSNW_SCORER_OPT
    ok = ok && hsnw_opt_in(reinterpret_cast<const void*>(k_scorer_fwd_tc<1>), "scorer_fwd_tc")
         && hsnw_opt_in(reinterpret_cast<const void*>(k_scorer_bwd_tc), "scorer_bwd_tc");
    if (!ok) hsnw_attribute_failed();
}
