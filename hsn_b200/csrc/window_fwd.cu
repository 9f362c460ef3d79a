// The forward sweep of a window as batch-synchronous phases: every row advances one position per
// round of four phases, and the phases' work is laid out for the hardware rather than per row:
//
//   front   weight-stationary: a block holds a 64-column slice of the shared path's first layer
//           ([q -> 2H], S and P merged) and the matching rows of its second layer in shared
//           memory and serves every row; the rows' partial sums are reduced in slice order later.
//   row     one block per row: reduce the partials to (u, z_hat), the scorer's logits for every
//           cell, the router's decision (select.cuh), the gather of the selected cells and of
//           their message sources, the messages, the cell norm -> the pairs' inputs v. What the
//           scorer and the messages read of the state is kept as derived state that only the K
//           written cells change per position (the state's part of every cell's logits, V h of
//           every cell, every cell's max |h|), so no position walks the whole state; the row's
//           inputs are staged into shared memory by the TMA's bulk copies on an mbarrier.
//   unit    weight-stationary: a block holds a 64-column slice of ONE unit's first layer and the
//           matching rows of its second layer and serves the pairs (row, slot) routed to that
//           unit, found by a ballot compaction of the pair list: no unit runs for a pair that did
//           not choose it (the reference multiplies every pair by all M units,
//           python/hsn/model/units.py:566-572). The gate's linear rides as extra jobs.
//   update  one block per row: reduce the second layer's partials, W_out, candidate norm, tanh,
//           sigmoid, the gated write-back, summary, ages, the tape's records and the next
//           position's reset.
//
// What it computes per position is the reference's folded sweep (python/hsn/train/compile.py:
// 1117-1193; per position python/hsn/model/hsn.py:1903-1980 and python/hsn/model/cell.py:349-505)
// and it writes the reference's tape (compile.py:1196-1213). With prod_bf16 every product rounds
// its operands and its output to bfloat16 and sums in fp32, the state and the norms stay fp32.
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "select.cuh"
#include "stage.cuh"
#include "umma.cuh"
#include "host_util.h"

using namespace hsnw;

namespace {

constexpr int kSlice = 64;       // tile edge of the window-invariant projection (k_pre)
constexpr int kFS = 32;          // columns of a front slice
constexpr int kFR = 8;           // rows a front block serves (kFRBig of them where the batch has hundreds of rows)
constexpr int kFRBig = 32;
constexpr int kUS = 32;          // columns of a unit slice
constexpr int kPB = 32;          // pairs a unit block multiplies at a time
constexpr int kPairTile = 256;   // pairs a unit block scans
constexpr int kCopyFloats = 4096;  // floats of the state a copy block moves
constexpr int kInitCells = 32;   // cells of a block of the derived-state kernel
constexpr int kMaxM = 16;        // units (registers of the scorer's thread)

// Optional phase timestamps for tuning (compiled in with -DHSNW_TRACE): event i of block b of a
// kernel lands at trace[(kernel * 512 + b) * 16 + i] (nanoseconds of the global timer).
#ifdef HSNW_TRACE
#define HSNW_MARK(kernel, i)                                                                     \
    do {                                                                                         \
        if (threadIdx.x == 0 && blockIdx.y == 0 && blockIdx.x < 512) {                           \
            unsigned long long now;                                                              \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));                              \
            c.trace[((kernel) * 512 + blockIdx.x) * 16 + (i)] = now;                             \
        }                                                                                        \
    } while (0)
#else
#define HSNW_MARK(kernel, i) do { } while (0)
#endif

struct FwdCtx {
    HsnwModel m;
    HsnwForward io;
    int nF;      // slices of one front MLP's hidden layer
    int nU;      // slices of a unit's hidden layer
    int nG;      // slices of the gate's outputs
    int n_front; // blocks of k_front that run the front (the rest copy the state tape)
    int copy_per_row;
    int stage_cells;    // 1: the row phase stages the per-cell logit parts and scalars in shared memory
    int carried;        // 1: the derived state in the scratch is current (a resident state's next call)
    int pair_tile;      // pairs a tensor-core unit block scans for its unit's
    int front_rows;     // rows a front block serves: kFR, or kFRBig for large batches (a weight slice is loaded once for them)
    int marker;         // status[4] holds it while the scratch's derived state is current for this B, T, resident
    int* status;        // [1] 0, or 1 when a bounded wait ran out
    unsigned long long* trace;  // phase timestamps (HSNW_TRACE builds)
    float* pre_s;       // [B*T, H]
    float* part_front;  // [B, 2 nF, d]
    float* v;           // [B*K, 4d]
    int* pair_unit;     // [B*K] the pair's unit, -1 on a padded slot
    float* part_f;      // [nU, B*K, d]
    float* gate_pre;    // [B*K, d]
    int* hmax_part;     // [B] bits of max |h| over the cells the position does not write
    float* lh;          // [B, N, M] derived: the state's part of every cell's logits
    float* vh;          // [B, N, d] derived: V h of every cell
    int* cmax;          // [B, N]    derived: bits of every cell's max |h|
};

__device__ __forceinline__ const float* state_h(const FwdCtx& c, int row, int t) {
    return c.io.tape_state ? c.io.tape_h + (static_cast<int64_t>(row) * (c.io.T + 1) + t) * c.m.N * c.m.d
                           : c.io.h0 + static_cast<int64_t>(row) * c.m.N * c.m.d;
}
__device__ __forceinline__ const float* state_q(const FwdCtx& c, int row, int t) {
    return c.io.tape_state ? c.io.tape_q + (static_cast<int64_t>(row) * (c.io.T + 1) + t) * c.m.d
                           : c.io.q0 + static_cast<int64_t>(row) * c.m.d;
}
__device__ __forceinline__ const int64_t* state_age(const FwdCtx& c, int row, int t) {
    return c.io.tape_state ? c.io.tape_age + (static_cast<int64_t>(row) * (c.io.T + 1) + t) * c.m.N
                           : c.io.age0 + static_cast<int64_t>(row) * c.m.N;
}
__host__ __device__ __forceinline__ int pad4(int n) { return (n + 3) & ~3; }

// The derived state of one cell from its state row hrow [d] (shared memory, already rounded to the
// products' operand precision): thread `first` of a group of `stride` threads computes outputs
// first, first + stride, ... of [M logit parts | d of V h].
__device__ __forceinline__ void derive_outputs(const FwdCtx& c, const float* hrow, const float* swh,
                                               const float* vt, float* lh_out, float* vh_out, int first,
                                               int stride) {
    const int d = c.m.d, M = c.m.M;
    const bool bf = c.m.prod_bf16 != 0;
    for (int o = first; o < M + d; o += stride) {
        if (o < M) lh_out[o] = dot4(hrow, 1, swh + o, M, d);
        else vh_out[o - M] = maybe_bf16(dot4(hrow, 1, vt + (o - M), d, d), bf);
    }
}

// ------------------------------------------------------------------------------------------------
// init: record 0 of the tape is the start state with column 0's reset applied (resident: the
// reset is applied in place), and the derived state of every cell. blockIdx.x = row,
// blockIdx.y = tile of 32 cells. Shared: hs [32][d], swh [d M], vt [d d].
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_init(FwdCtx c) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int N = c.m.N, d = c.m.d, M = c.m.M, T = c.io.T;
    float* hs = reinterpret_cast<float*>(dyn);
    float* hb = hs + kInitCells * d;     // the same rows at the products' operand precision
    float* swh = hb + kInitCells * d;
    float* vt = swh + d * M;
    const bool bf = c.m.prod_bf16 != 0;
    const bool cut = c.io.reset[static_cast<int64_t>(row) * T] != 0;
    float* h0 = c.io.h0 + static_cast<int64_t>(row) * N * d;
    if (row == 0 && blockIdx.y == 0 && tid == 0) *c.status = 0;
    // carried: the previous call on this state left every cell's derived values, if it was one of the
    // batch-synchronous kind with the same sizes (its last kernel then wrote the marker)
    if (c.carried && c.status[4] == c.marker && !cut) return;
    for (int e = tid; e < d * M; e += nt) swh[e] = c.m.score_w_t[2 * d * M + e];
    for (int e = tid; e < d * d; e += nt) vt[e] = c.m.v_t[e];
    // (a carried call launches at most 8 blocks a row: they walk the row's tiles themselves on the rare row that was reset)
    for (int tile = blockIdx.y; tile * kInitCells < N; tile += gridDim.y) {
    const int cell0 = tile * kInitCells;
    const int ncell = min(kInitCells, N - cell0);
    __syncthreads();   // the last tile's rows have been read
    for (int e = tid; e < ncell * d; e += nt) {
        const float v = cut ? 0.0f : h0[static_cast<int64_t>(cell0) * d + e];
        hs[e] = v;
        hb[e] = maybe_bf16(v, bf);
        if (c.io.tape_state) c.io.tape_h[(static_cast<int64_t>(row) * (T + 1)) * N * d + static_cast<int64_t>(cell0) * d + e] = v;
        else if (cut) h0[static_cast<int64_t>(cell0) * d + e] = 0.0f;
    }
    for (int n = tid; n < ncell; n += nt) {
        int64_t* a0 = c.io.age0 + static_cast<int64_t>(row) * N + cell0;
        if (c.io.tape_state) c.io.tape_age[(static_cast<int64_t>(row) * (T + 1)) * N + cell0 + n] = cut ? 0 : a0[n];
        else if (cut) a0[n] = 0;
    }
    if (tile == 0) {
        float* q0 = c.io.q0 + static_cast<int64_t>(row) * d;
        for (int x = tid; x < d; x += nt) {
            if (c.io.tape_state) c.io.tape_q[(static_cast<int64_t>(row) * (T + 1)) * d + x] = cut ? 0.0f : q0[x];
            else if (cut) q0[x] = 0.0f;
        }
    }
    __syncthreads();
    // 8 threads per cell
    const int cl = tid >> 3, sub = tid & 7;
    if (cl < ncell) {
        const int64_t cell = static_cast<int64_t>(row) * N + cell0 + cl;
        derive_outputs(c, hb + cl * d, swh, vt, c.lh + cell * M, c.vh + cell * d, sub, 8);
        if (sub == 0) {
            int top = 0;
            for (int x = 0; x < d; ++x) top = max(top, __float_as_int(fabsf(hs[cl * d + x])));
            c.cmax[cell] = top;
        }
    }
    }
}

// ------------------------------------------------------------------------------------------------
// pre: the window-invariant part of S's first layer for every (row, position):
// pre_s[r, j] = b1[j] + sum_x [z; ctx][r, x] W[x, j]. A 64 x 64 tile per block, 16 deep.
// ------------------------------------------------------------------------------------------------
__global__ void k_pre(HsnwModel m, const float* z, const float* ctx, int64_t rows, float* out) {
    __shared__ float xs[16][kSlice + 1];
    __shared__ float ws[16][kSlice];
    const int d = m.d, dc = m.dc, H = m.H, in = d + dc;
    const bool bf = m.prod_bf16 != 0;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * kSlice;
    const int c0 = blockIdx.y * kSlice;
    const int tid = threadIdx.x;           // 256 threads: 16 x 16, a 4 x 4 register tile each
    const int tr = tid >> 4, tc = tid & 15;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < in; k0 += 16) {
        for (int e = tid; e < 16 * kSlice; e += 256) {
            const int kk = e & 15, r = e >> 4;
            const int64_t rr = r0 + r;
            const int x = k0 + kk;
            float v = 0.0f;
            if (rr < rows && x < in) v = x < d ? z[rr * d + x] : ctx[rr * dc + (x - d)];
            xs[kk][r] = maybe_bf16(v, bf);
        }
        for (int e = tid; e < 16 * kSlice; e += 256) {
            const int cc = e & (kSlice - 1), kk = e >> 6;
            const int x = k0 + kk, col = c0 + cc;
            ws[kk][cc] = (x < in && col < H) ? m.s_w1zc_t[static_cast<int64_t>(x) * H + col] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[kk][tr * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[kk][tc * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += xv[i] * wv[j];
        }
        __syncthreads();
    }
    for (int i = 0; i < 4; ++i) {
        const int64_t rr = r0 + tr * 4 + i;
        if (rr >= rows) continue;
        for (int j = 0; j < 4; ++j) {
            const int col = c0 + tc * 4 + j;
            if (col < H) out[rr * H + col] = acc[i][j] + m.f_b1[col];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// pre on the tensor cores (bf16 products): a 128 x 128 tile of pre_s per block, K = d + dc.
// Both operands are converted to bf16 while they are staged into the K-major core-matrix layout of
// umma.cuh; one thread issues the tcgen05.mma chain into a 128-column TMEM accumulator and commits
// it to an mbarrier; the four warps read their 32 lanes back (tcgen05.ld) and add the bias.
// Shared (dynamic): A [Kp/8][128][8] bf16, B [Kp/8][128][8] bf16.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);   // one conversion for both halves
    return *reinterpret_cast<const uint32_t*>(&pair);
}

// BN: the columns of a block's tile (128; 32 for few rows, so that a serving step's 512 rows still give 64 blocks)
template <int BN>
__global__ void __launch_bounds__(128) k_pre_tc(HsnwModel m, const float* z, const float* ctx, int64_t rows, float* out,
                                                int* status) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int d = m.d, dc = m.dc, H = m.H, K = d + dc, Kp = (K + 15) & ~15, planes = Kp >> 3;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * 128;
    const int c0 = blockIdx.y * BN;
    uint4* As = reinterpret_cast<uint4*>(dyn);
    uint4* Bs = As + planes * 128;
    if (tid == 0) mbar_init(&bar, 1);
    // eight consecutive inputs of a row are 32 contiguous bytes of z or of ctx when both widths are multiples of 8
    const bool vec = ((d | dc) & 7) == 0 && ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(ctx)) & 15) == 0;
    for (int idx = tid; idx < planes * 128; idx += 128) {
        const int r = idx & 127, kc = idx >> 7;
        const int64_t row = r0 + r;
        float v[8];
        const int k0 = kc * 8;
        if (vec && row < rows && k0 < K) {
            const float* src = k0 < d ? z + row * d + k0 : ctx + row * dc + (k0 - d);
            const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int k = k0 + j;
                v[j] = (row < rows && k < K) ? (k < d ? z[row * d + k] : ctx[row * dc + (k - d)]) : 0.0f;
            }
        }
        As[idx] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    }
    for (int idx = tid; idx < planes * BN; idx += 128) {
        const int r = idx % BN, kc = idx / BN;
        const int col = c0 + r;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = kc * 8 + j;
            v[j] = (col < H && k < K) ? m.s_w1zc_t[static_cast<int64_t>(k) * H + col] : 0.0f;
        }
        Bs[idx] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
    }
    fence_async_smem();
    if (warp == 0) tmem_alloc(&tmem_slot, BN);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
        const uint32_t idesc = umma_idesc_bf16(128, BN);
        const uint64_t da = umma_desc(As, 128), db = umma_desc(Bs, BN);
        umma_chain(taddr, da, db, idesc, Kp >> 4, umma_kstep(128), umma_kstep(BN));  // two planes per K = 16
        umma_commit(&bar);
    }
    mbar_wait(&bar, 0, status);
    tcgen05_fence_after();
    const int64_t row = r0 + warp * 32 + lane;
    for (int cb = 0; cb < BN; cb += 8) {
        float acc[8];
        tmem_ld8(tmem_addr(taddr, warp * 32, cb), acc);
        if (row < rows) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int col = c0 + cb + i;
                if (col < H) out[row * H + col] = acc[i] + m.f_b1[col];
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, BN);
}

// ------------------------------------------------------------------------------------------------
// front: blocks [0, n_front): (slice, row tile) of the shared path, slices 0..nF-1: S, nF..2nF-1: P;
// 256 threads: thread (row r, column cc) for the first layer, strided outputs for the second.
// Shared: w1 [d][32], w2 [32][d], q [8][d], act [8][32].
// Blocks [n_front, ...): the state tape's next record as a copy of this one, 16 KB a block (zeros
// when the next position resets; the ages one older): off the critical path of the row phase,
// which then only overwrites the K written cells.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_front(FwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const int d = c.m.d, H = c.m.H, B = c.io.B, T = c.io.T, N = c.m.N;
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const bool bf = c.m.prod_bf16 != 0;
    const int tid = threadIdx.x;
    if (static_cast<int>(blockIdx.x) >= c.n_front) {
        const int job = blockIdx.x - c.n_front;
        const int row = job / c.copy_per_row, chunk = job - row * c.copy_per_row;
        const bool clear = t + 1 < T && c.io.reset[static_cast<int64_t>(row) * T + t + 1] != 0;
        const int64_t rec = (static_cast<int64_t>(row) * (T + 1) + t) * N;
        const float4* src = reinterpret_cast<const float4*>(c.io.tape_h + rec * d);
        float4* dst = reinterpret_cast<float4*>(c.io.tape_h + (rec + N) * d);
        const int total4 = (N * d) >> 2;
        const int lo = chunk * (kCopyFloats >> 2), hi = min(total4, lo + (kCopyFloats >> 2));
        for (int e = lo + tid; e < hi; e += 256) dst[e] = clear ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : src[e];
        if (chunk == 0) {
            const int64_t* age = c.io.tape_age + rec;
            int64_t* age_next = c.io.tape_age + rec + N;
            for (int n = tid; n < N; n += 256) age_next[n] = clear ? 0 : age[n] + 1;
        }
        return;
    }
    const int nF = c.nF;
    const int slice = blockIdx.x % (2 * nF), tile = blockIdx.x / (2 * nF);
    const bool is_p = slice >= nF;
    const int c0 = (is_p ? slice - nF : slice) * kFS;
    const int cols = min(kFS, H - c0);
    const int col_base = (is_p ? H : 0) + c0;   // column in the merged [d, 2H] first layer
    const int FR = c.front_rows;
    const int r0 = tile * FR;
    const int rows = min(FR, B - r0);
    float* w1 = reinterpret_cast<float*>(dyn);          // [d][32]
    float* w2 = w1 + d * kFS;                           // [32][d]
    float* qs = w2 + kFS * d;                           // [8][d]
    float* act = qs + FR * d;                           // [rows][32]
    if (cols == kFS) {
        // 16 bytes per request, every request in flight at once
        for (int e = tid; e < d * (kFS >> 2); e += 256) {
            const int x = e >> 3, c4 = e & 7;
            cp_async16(w1 + x * kFS + c4 * 4, c.m.f_w1q_t + static_cast<int64_t>(x) * 2 * H + col_base + c4 * 4);
        }
        cp_async_floats(w2, c.m.f_w2_t + static_cast<int64_t>(col_base) * d, kFS * d);
        cp_async_commit();
    } else {
        for (int e = tid; e < d * kFS; e += 256) {
            const int x = e >> 5, cc = e & 31;
            w1[e] = cc < cols ? c.m.f_w1q_t[static_cast<int64_t>(x) * 2 * H + col_base + cc] : 0.0f;
        }
        for (int e = tid; e < kFS * d; e += 256) {
            const int cc = div_magic(e, dmag), x = e - cc * d;
            w2[e] = cc < cols ? c.m.f_w2_t[static_cast<int64_t>(col_base + cc) * d + x] : 0.0f;
        }
    }
    for (int e = tid; e < rows * d; e += 256) {
        const int r = div_magic(e, dmag), x = e - r * d;
        qs[e] = maybe_bf16(state_q(c, r0 + r, t)[x], bf);
    }
    // thread (r, cc) serves rows r, r + 8, ... of the tile: a weight is read once for them
    constexpr int kRI = kFRBig / 8;
    float pre[kRI];
    {
        const int r = tid >> 5, cc = tid & 31;
#pragma unroll
        for (int i = 0; i < kRI; ++i) {
            const int rr = r + 8 * i;
            pre[i] = 0.0f;
            if (rr < rows && cc < cols)
                pre[i] = is_p ? c.m.f_b1[H + c0 + cc] : c.pre_s[(static_cast<int64_t>(r0 + rr) * T + t) * H + c0 + cc];
        }
    }
    cp_async_wait_all();
    __syncthreads();
    {
        const int r = tid >> 5, cc = tid & 31;
        float sum[kRI] = {};
        if (rows <= 8) {
            if (r < rows)
                for (int x = 0; x < d; ++x) sum[0] += qs[r * d + x] * w1[x * kFS + cc];
        } else {
            for (int x = 0; x < d; ++x) {
                const float w = w1[x * kFS + cc];
#pragma unroll
                for (int i = 0; i < kRI; ++i) sum[i] += qs[min(r + 8 * i, rows - 1) * d + x] * w;
            }
        }
#pragma unroll
        for (int i = 0; i < kRI; ++i) {
            const int rr = r + 8 * i;
            if (rr < FR) act[rr * kFS + cc] = rr < rows && cc < cols ? maybe_bf16(gelu_erf(maybe_bf16(sum[i] + pre[i], bf)), bf) : 0.0f;
        }
    }
    __syncthreads();
    if (rows <= 8) {
        for (int e = tid; e < rows * d; e += 256) {
            const int r = div_magic(e, dmag), x = e - r * d;
            float sum = 0.0f;
#pragma unroll 8
            for (int cc = 0; cc < kFS; ++cc) sum += act[r * kFS + cc] * w2[cc * d + x];
            c.part_front[(static_cast<int64_t>(r0 + r) * 2 * nF + slice) * d + x] = sum;
        }
    } else {
        // four rows a thread (r4, r4 + 1, .. of a group of four): a weight is read once for them
        for (int e = tid; e < ((rows + 3) / 4) * d; e += 256) {
            const int g = div_magic(e, dmag), x = e - g * d;
            float sum[4] = {};
#pragma unroll 8
            for (int cc = 0; cc < kFS; ++cc) {
                const float w = w2[cc * d + x];
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[i] += act[min(g * 4 + i, FR - 1) * kFS + cc] * w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (g * 4 + i < rows) c.part_front[(static_cast<int64_t>(r0 + g * 4 + i) * 2 * nF + slice) * d + x] = sum[i];
        }
    }
}

// The scorer on a row's cells, a thread per cell: logits = the cell's derived part + the age term +
// the scalars' terms (in that order) + the row's term + the bias, rounded; the cell's score is its
// best logit (less the unit's cost) and its unit the first maximiser. MM bounds the units (8 or
// 16), so a model of eight units issues no idle lanes of a sixteen-wide loop; the scalars go four
// at a time under a uniform branch for the same reason.
template <int MM>
__device__ __forceinline__ void score_cells(const FwdCtx& c, int64_t rt, const float* lh, const float* scal,
                                            const int64_t* age, const float* sw_tail,
                                            const float* rowterm, const float* score_b, const float* cost,
                                            float* score, int* unit) {
    const int N = c.m.N, M = c.m.M, Sn = c.m.S;
    const int nt = blockDim.x, lane = threadIdx.x & 31;
    const bool bf = c.m.prod_bf16 != 0;
    const float lambda = c.m.lambda_cost;
    const float age_div = static_cast<float>(c.m.age_max);
    const bool wide = (M & 3) == 0;   // the weights' rows are then 16-byte aligned
    for (int i0 = threadIdx.x - lane; i0 < N; i0 += nt) {
        const int i = i0 + lane;
        const bool live = i < N;
        if (!live) continue;
        const float* mine = scal + static_cast<int64_t>(i) * Sn;
        // every load of the cell goes out before the first use: the scalars (up to sixteen, four at
        // a time under a uniform branch), then the derived logit parts and the age
        float feat[16];
#pragma unroll
        for (int s0 = 0; s0 < 16; s0 += 4) {
            if (s0 < Sn) {
#pragma unroll
                for (int s = 0; s < 4; ++s) feat[s0 + s] = s0 + s < Sn ? mine[s0 + s] : 0.0f;
            }
        }
        const float age_f = static_cast<float>(age[i]);
        float acc[MM];
        if (wide) {
#pragma unroll
            for (int j = 0; j < MM; j += 4) {
                if (j < M) {
                    const float4 v = *reinterpret_cast<const float4*>(lh + static_cast<int64_t>(i) * M + j);
                    acc[j] = v.x; acc[j + 1] = v.y; acc[j + 2] = v.z; acc[j + 3] = v.w;
                } else {
                    acc[j] = acc[j + 1] = acc[j + 2] = acc[j + 3] = 0.0f;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < MM; ++j) acc[j] = j < M ? lh[static_cast<int64_t>(i) * M + j] : 0.0f;
        }
        auto add_term = [&](float a, const float* w) {
            if (wide) {
#pragma unroll
                for (int j = 0; j < MM; j += 4) {
                    if (j < M) {
                        const float4 wv = *reinterpret_cast<const float4*>(w + j);
                        acc[j] += a * wv.x; acc[j + 1] += a * wv.y; acc[j + 2] += a * wv.z; acc[j + 3] += a * wv.w;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < MM; ++j)
                    if (j < M) acc[j] += a * w[j];
            }
        };
        add_term(maybe_bf16(age_f / age_div, bf), sw_tail);
#pragma unroll
        for (int s0 = 0; s0 < 16; s0 += 4) {
            if (s0 < Sn) {
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    if (s0 + s < Sn) add_term(maybe_bf16(feat[s0 + s], bf), sw_tail + (1 + s0 + s) * M);
            }
        }
        for (int s = 16; s < Sn; ++s) add_term(maybe_bf16(mine[s], bf), sw_tail + (1 + s) * M);   // rare: more than sixteen scalars
        float best = -INFINITY;
        int arg = 0;
#pragma unroll
        for (int j = 0; j < MM; ++j) {
            if (j < M) {
                const float logit = maybe_bf16(acc[j] + rowterm[j] + score_b[j], bf);
                if (c.io.logits) c.io.logits[(rt * N + i) * M + j] = logit;
                const float sc = lambda > 0.0f ? __fsub_rn(logit, __fmul_rn(lambda, cost[j])) : logit;
                if (j == 0 || sc > best) {
                    best = sc;
                    arg = j;
                }
            }
        }
        score[i] = best;
        unit[i] = arg;
    }
}

// ------------------------------------------------------------------------------------------------
// row: one block per row. Everything the position reads of the row arrives in two stagings, each
// one round trip to memory: (1) the front's partial sums, the derived logit parts of every cell,
// the scorer's scalars, the ages and the cells' maxima as bulk copies on an mbarrier (contiguous,
// 16-byte aligned runs; plain loads otherwise); (2) after the decision, the K selected cells' state
// rows and the K D message sources' V h rows, one bulk copy per row.
// Shared (dynamic), each segment padded to 16 bytes: pf [2 nF d], lh [N M], scal [N S], age [N] i64,
// cmax [N], rows [(K + K D) d], msg [K d], sw_head [2d M], sw_tail [(1+S) M], score [N], unit [N],
// ue [2d], rowterm [16], score_b [16], src [K D], ew [K D], rms [K].
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512, 2) k_row(FwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ SelectShared S;
    __shared__ int ired[32];
    __shared__ __align__(8) uint64_t bar;
    const int N = c.m.N, d = c.m.d, K = c.m.K, M = c.m.M, D = c.m.D, Sn = c.m.S;
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const int T = c.io.T;
    const bool bf = c.m.prod_bf16 != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    const int nrows = K + K * D, nF2 = 2 * c.nF;
    float* pf = reinterpret_cast<float*>(dyn);
    const bool staged = c.stage_cells != 0;  // else the per-cell inputs are read from memory in place
    float* lh_s = pf + pad4(nF2 * d);
    float* scal_s = lh_s + (staged ? pad4(N * M) : 0);
    int64_t* age = reinterpret_cast<int64_t*>(scal_s + (staged ? pad4(N * Sn) : 0));
    int* cmax = reinterpret_cast<int*>(reinterpret_cast<float*>(age) + pad4(2 * N));
    float* rows = reinterpret_cast<float*>(cmax + pad4(N));
    float* msg = rows + nrows * d;
    float* sw_head = msg + K * d;
    float* sw_tail = sw_head + pad4(2 * d * M);
    float* score = sw_tail + pad4((1 + Sn) * M);
    int* unit = reinterpret_cast<int*>(score + pad4(N));
    float* ue = reinterpret_cast<float*>(unit + pad4(N));
    float* rowterm = ue + 2 * d;
    float* score_b_s = rowterm + kMaxM;
    int* src = reinterpret_cast<int*>(score_b_s + kMaxM);
    float* ew = reinterpret_cast<float*>(src + pad4(K * D));
    float* rms = ew + pad4(K * D);
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    const float* h = state_h(c, row, t);
    HSNW_MARK(2, 0);
    if (tid == 0) mbar_init(&bar, 1);
    __syncthreads();
    // staging 1
    {
        const float* g_pf = c.part_front + static_cast<int64_t>(row) * nF2 * d;
        const float* g_lh = c.lh + static_cast<int64_t>(row) * N * M;
        const float* g_scal = c.io.scalars + rt * N * Sn;
        const int64_t* g_age = state_age(c, row, t);
        const int* g_cmax = c.cmax + static_cast<int64_t>(row) * N;
        const void* srcs[5] = {g_pf, g_lh, g_scal, g_age, g_cmax};
        void* dsts[5] = {pf, lh_s, scal_s, age, cmax};
        const size_t bytes[5] = {sizeof(float) * nF2 * d, staged ? sizeof(float) * N * M : 0,
                                 staged ? sizeof(float) * N * Sn : 0,
                                 sizeof(int64_t) * N, sizeof(int) * N};
        uint32_t total = 0;
        bool bulk[5];
#pragma unroll
        for (int s = 0; s < 5; ++s) {
            bulk[s] = bulk_ok(srcs[s], dsts[s], bytes[s]);
            if (bulk[s]) total += static_cast<uint32_t>(bytes[s]);
        }
        if (tid == 0) {
            mbar_expect_tx(&bar, total);
#pragma unroll
            for (int s = 0; s < 5; ++s)
                if (bulk[s]) bulk_g2s(dsts[s], srcs[s], static_cast<uint32_t>(bytes[s]), &bar);
        }
#pragma unroll
        for (int s = 0; s < 5; ++s)
            if (!bulk[s]) {
                const int words = static_cast<int>(bytes[s] >> 2);
                const uint32_t* from = static_cast<const uint32_t*>(srcs[s]);
                uint32_t* to = static_cast<uint32_t*>(dsts[s]);
                for (int e = tid; e < words; e += nt) to[e] = from[e];
            }
        cp_async_floats(sw_head, c.m.score_w_t, 2 * d * M);
        cp_async_floats(sw_tail, c.m.score_w_t + static_cast<int64_t>(3 * d) * M, (1 + Sn) * M);
        cp_async_commit();
        for (int j = tid; j < M; j += nt) {
            S.cost[j] = c.m.cost[j];
            score_b_s[j] = c.m.score_b[j];
        }
        cp_async_wait_all();
        mbar_wait(&bar, 0, c.status);
    }
    __syncthreads();
    HSNW_MARK(2, 1);
    // (u, z_hat) from the front's partial sums, slice by slice; eps = z - z_hat
    for (int x = tid; x < 2 * d; x += nt) {
        const bool is_p = x >= d;
        const int xx = is_p ? x - d : x;
        const float sum = sum4(pf + (is_p ? c.nF : 0) * d + xx, d, c.nF);
        const float out = maybe_bf16(sum + c.m.f_b2[x], bf);
        ue[x] = is_p ? c.io.z[rt * d + xx] - out : out;
        if (!is_p && c.io.us) c.io.us[rt * d + xx] = out;
    }
    __syncthreads();
    for (int j = warp; j < M; j += warps) {  // a warp per unit: lanes stride the 2d inputs
        float sum = 0.0f;
        for (int x = lane; x < 2 * d; x += 32) sum += maybe_bf16(ue[x], bf) * sw_head[x * M + j];
        sum = warp_sum(sum);
        if (lane == 0) rowterm[j] = sum;
    }
    __syncthreads();
    HSNW_MARK(2, 2);
    // the scorer: a thread per cell; the state's part of the logits is derived state
    const float* lh = staged ? lh_s : c.lh + static_cast<int64_t>(row) * N * M;
    const float* scal = staged ? scal_s : c.io.scalars + rt * N * Sn;
    if (M <= 8) score_cells<8>(c, rt, lh, scal, age, sw_tail, rowterm, score_b_s, S.cost, score, unit);
    else score_cells<kMaxM>(c, rt, lh, scal, age, sw_tail, rowterm, score_b_s, S.cost, score, unit);
    __syncthreads();
    int64_t* cells_o = c.io.cells + rt * K;
    int64_t* units_o = c.io.units + rt * K;
    uint8_t* valid_o = c.io.valid + rt * K;
    HSNW_MARK(2, 3);
    if (!c.io.forced) {
        SelectParams P;
        P.N = N; P.M = M; P.K = K; P.age_max = c.m.age_max; P.probes = c.m.probes;
        P.reserved = 0; P.fixed_units = 0;
        P.overhead = c.m.cell_overhead; P.shared_cost = c.m.shared_cost; P.limit = c.m.limit;
        uint64_t* cand = reinterpret_cast<uint64_t*>(rows);   // [warps][K + 1]: the rows arrive after the decision
        const bool cand_fits = sizeof(uint64_t) * warps * (K + 1) <= sizeof(float) * nrows * d;
        if (N > 256 && N <= 2048 && cand_fits) {
            // every warp reduces its cells to its K + 1 best keys, one warp merges them and finishes
            select_candidates_warp(N, K, score, cand + warp * (K + 1), warp * 32, nt);
            __syncthreads();
            if (warp == 0) select_merge_warp(P, score, unit, age, cand, warps * (K + 1), S);
            __syncthreads();
        } else if (N <= 2048) {  // one warp decides; the others wait at the barrier
            if (warp == 0) select_row_warp(P, score, unit, age, S);
            __syncthreads();
        } else {
            select_row(P, score, unit, age, S);
        }
        HSNW_MARK(2, 4);
        for (int k = tid; k < K; k += nt) {
            cells_o[k] = S.out_cell[k];
            units_o[k] = S.out_unit[k];
            valid_o[k] = static_cast<uint8_t>(S.out_flag[k] & 1);
            c.io.refreshed[rt * K + k] = static_cast<uint8_t>((S.out_flag[k] >> 1) & 1);
        }
        if (tid == 0) c.io.theta[rt] = S.theta;
    } else {
        for (int k = tid; k < K; k += nt) {
            const bool ok = valid_o[k] != 0;
            S.out_cell[k] = ok ? static_cast<int>(cells_o[k]) : 0;
            S.out_unit[k] = ok ? static_cast<int>(units_o[k]) : 0;
            S.out_flag[k] = ok ? 1 : 0;
        }
        __syncthreads();
    }
    // the sources and edge weights of the selected cells
    for (int e = tid; e < K * D; e += nt) {
        const int k = e / D, j = e - k * D;
        const int cell = S.out_cell[k];
        src[e] = c.m.pad_src[cell * D + j];
        ew[e] = maybe_bf16(c.m.edge_w[cell * D + j], bf);
    }
    // max |h| over the cells this position does not write (the update adds the written ones): the
    // written cells' entries of the block's copy are cleared first
    for (int k = tid; k < K; k += nt)
        if (S.out_flag[k] & 1) cmax[S.out_cell[k]] = 0;
    __syncthreads();
    {
        int top = 0;
        for (int i = tid; i < N; i += nt) top = max(top, cmax[i]);
        for (int w = 16; w > 0; w >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, w));
        if (lane == 0) ired[warp] = top;
    }
    __syncthreads();
    if (tid == 0) {
        int mx = 0;
        for (int w = 0; w < warps; ++w) mx = max(mx, ired[w]);
        c.hmax_part[row] = mx;
    }
    HSNW_MARK(2, 5);
    // staging 2: the selected cells' state rows and their sources' V h rows, one bulk copy a row
    {
        const float* g_vh = c.vh + static_cast<int64_t>(row) * N * d;
        const uint32_t row_bytes = static_cast<uint32_t>(sizeof(float) * d);
        const bool bulk = bulk_ok(h, rows, row_bytes) && bulk_ok(g_vh, rows, row_bytes);
        if (bulk) {
            if (warp == 0) {
                if (lane == 0) mbar_expect_tx(&bar, row_bytes * nrows);
                __syncwarp();
                for (int r = lane; r < nrows; r += 32) {
                    const float* from = r < K ? h + static_cast<int64_t>(S.out_cell[r]) * d
                                              : g_vh + static_cast<int64_t>(src[r - K]) * d;
                    bulk_g2s(rows + r * d, from, row_bytes, &bar);
                }
            }
            mbar_wait(&bar, 1, c.status);
        } else {
            for (int e = tid; e < nrows * d; e += nt) {
                const int r = div_magic(e, dmag), x = e - r * d;
                rows[e] = r < K ? h[static_cast<int64_t>(S.out_cell[r]) * d + x] : g_vh[static_cast<int64_t>(src[r - K]) * d + x];
            }
        }
    }
    __syncthreads();
    HSNW_MARK(2, 6);
    for (int e = tid; e < K * d; e += nt) {
        const int k = div_magic(e, dmag), x = e - k * d;
        float sum = 0.0f;
        for (int j = 0; j < D; ++j) sum += rows[(K + k * D + j) * d + x] * ew[k * D + j];  // edge order
        msg[e] = maybe_bf16(sum, bf);
    }
    __syncthreads();
    // the cell norm over [u; eps; h_old; m]: a warp per slot
    for (int k = warp; k < K; k += warps) {
        float sq = 0.0f;
        for (int j = lane; j < 4 * d; j += 32) {
            const int blk = div_magic(j, dmag), x = j - blk * d;
            const float v = blk == 0 ? ue[x] : blk == 1 ? ue[d + x] : blk == 2 ? rows[k * d + x] : msg[k * d + x];
            sq += v * v;
        }
        sq = warp_sum(sq);
        if (lane == 0) rms[k] = rsqrtf(sq / static_cast<float>(4 * d) + c.m.norm_eps);
    }
    __syncthreads();
    const int64_t pair0 = static_cast<int64_t>(row) * K;
    for (int e = tid; e < K * 4 * d; e += nt) {
        const int k = div_magic(e, magic_of(4 * d)), j = e - k * 4 * d;
        const int blk = div_magic(j, dmag), x = j - blk * d;
        const float v = blk == 0 ? ue[x] : blk == 1 ? ue[d + x] : blk == 2 ? rows[k * d + x] : msg[k * d + x];
        c.v[(pair0 + k) * 4 * d + j] = maybe_bf16(v * rms[k] * c.m.norm_w[j], bf);
    }
    for (int k = tid; k < K; k += nt) c.pair_unit[pair0 + k] = (S.out_flag[k] & 1) ? S.out_unit[k] : -1;
    if (c.io.rec_c) {
        for (int e = tid; e < K * d; e += nt) {
            c.io.rec_h_old[rt * K * d + e] = rows[e];
            c.io.rec_m[rt * K * d + e] = msg[e];
        }
        for (int k = tid; k < K; k += nt) c.io.rec_rms[rt * K + k] = rms[k];
    }
    HSNW_MARK(2, 7);
}

// ------------------------------------------------------------------------------------------------
// unit: blockIdx.x = job (unit j, slice s), blockIdx.y = pair tile. Slices 0 .. nU-1 are 32 columns
// of unit j's hidden layer (first layer, activation, the matching rows of the second layer as a
// partial sum); slices nU .. nU+nG-1 are 32 columns of the gate's linear for unit j's pairs.
// 256 threads: a thread owns one column and four pairs; the pairs' inputs are read 16 bytes at a
// time. Shared (dynamic): vbuf [32][4d], w1 [4d][32], w2 [32][d], act [32][32], list [256].
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_unit(FwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int warp_count[8];
    __shared__ int n_list;
    const int d = c.m.d, K = c.m.K, H = c.m.H, in = 4 * c.m.d;
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const int P = c.io.B * K, T = c.io.T;
    const bool bf = c.m.prod_bf16 != 0;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per_unit = c.nU + c.nG;
    const int j = blockIdx.x / per_unit, s = blockIdx.x - j * per_unit;
    const bool is_gate = s >= c.nU;
    const int sl = is_gate ? s - c.nU : s;
    const int c0 = sl * kUS;
    const int cols = min(kUS, (is_gate ? d : H) - c0);
    float* vbuf = reinterpret_cast<float*>(dyn);     // [32][4d]
    float* w1 = vbuf + kPB * in;                     // [4d][32]
    float* w2 = w1 + in * kUS;                       // [32][d]
    float* act = w2 + kUS * d;                       // [32][32]
    int* list = reinterpret_cast<int*>(act + kPB * kUS);  // [256]
    // the pairs of this tile routed to unit j, in pair order (a ballot compaction)
    const int p0 = blockIdx.y * kPairTile;
    {
        const int p = p0 + tid;
        const bool mine = p < P && c.pair_unit[p] == j;
        const unsigned mask = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(mask);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_count[w];
        if (mine) list[before + __popc(mask & ((1u << lane) - 1u))] = p;
        if (tid == 0) {
            int total = 0;
            for (int w = 0; w < 8; ++w) total += warp_count[w];
            n_list = total;
        }
        __syncthreads();
    }
    const int count = n_list;
    if (count == 0) return;
    if (is_gate) {
        for (int e = tid; e < in * kUS; e += 256) {
            const int x = e >> 5, cc = e & 31;
            w1[e] = cc < cols ? c.m.gate_t[static_cast<int64_t>(x) * d + c0 + cc] : 0.0f;
        }
    } else {
        const float* W1 = c.m.w1 + static_cast<int64_t>(j) * in * H;
        const float* W2 = c.m.w2 + static_cast<int64_t>(j) * H * d;
        for (int e = tid; e < in * kUS; e += 256) {
            const int x = e >> 5, cc = e & 31;
            w1[e] = cc < cols ? W1[static_cast<int64_t>(x) * H + c0 + cc] : 0.0f;
        }
        for (int e = tid; e < kUS * d; e += 256) {
            const int cc = div_magic(e, dmag), x = e - cc * d;
            w2[e] = cc < cols ? W2[static_cast<int64_t>(c0 + cc) * d + x] : 0.0f;
        }
    }
    const int cc = lane, pg = warp;  // a column and the pairs 4 pg .. 4 pg + 3 of a batch
    const float4* v4 = reinterpret_cast<const float4*>(c.v);
    float4* vbuf4 = reinterpret_cast<float4*>(vbuf);
    for (int base = 0; base < count; base += kPB) {
        const int nb = min(kPB, count - base);
        __syncthreads();
        for (int f = tid; f < nb * d; f += 256) {  // a pair's input is 4d floats = d float4
            const int pb = div_magic(f, dmag), x4 = f - pb * d;
            vbuf4[f] = v4[static_cast<int64_t>(list[base + pb]) * d + x4];
        }
        __syncthreads();
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int x4 = 0; x4 < d; ++x4) {
            const float w0 = w1[(4 * x4 + 0) * kUS + cc], wa = w1[(4 * x4 + 1) * kUS + cc];
            const float wb = w1[(4 * x4 + 2) * kUS + cc], wc = w1[(4 * x4 + 3) * kUS + cc];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float4 vv = vbuf4[(pg * 4 + p) * d + x4];
                acc[p] += vv.x * w0;
                acc[p] += vv.y * wa;
                acc[p] += vv.z * wb;
                acc[p] += vv.w * wc;
            }
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int pb = pg * 4 + p;
            float a = 0.0f;
            if (pb < nb && cc < cols) {
                const int pair = list[base + pb];
                if (is_gate) {
                    c.gate_pre[static_cast<int64_t>(pair) * d + c0 + cc] = maybe_bf16(acc[p] + c.m.gate_b[c0 + cc], bf);
                } else {
                    const float hid = maybe_bf16(acc[p] + c.m.b1[j * H + c0 + cc], bf);
                    if (c.io.rec_c) {
                        const int row = pair / K, k = pair - row * K;
                        store_hidden(c.io.rec_hidden, ((static_cast<int64_t>(row) * T + t) * K + k) * H + c0 + cc, hid, c.m.prod_bf16 != 0);
                    }
                    a = maybe_bf16(gelu_erf(hid), bf);
                }
            }
            if (!is_gate) act[pb * kUS + cc] = a;
        }
        if (is_gate) continue;
        __syncthreads();
        for (int e = tid; e < nb * d; e += 256) {
            const int pb = div_magic(e, dmag), x = e - pb * d;
            float sum = 0.0f;
#pragma unroll 8
            for (int k2 = 0; k2 < kUS; ++k2) sum += act[pb * kUS + k2] * w2[k2 * d + x];
            c.part_f[(static_cast<int64_t>(sl) * P + list[base + pb]) * d + x] = sum;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// unit on the tensor cores (bf16 products). blockIdx.x = (unit j, block cb): blocks 0 .. nB-1 are
// 128 hidden columns of unit j, block nB is the gate's linear for unit j's pairs; blockIdx.y = pair
// tile. Per batch of 32 pairs:
//   D1 [128 hidden columns, 32 pairs] = W1 tile [128, 4d] x v [32, 4d]^T      (tcgen05.mma, TMEM)
//   epilogue 1: + bias, round, record, activation, written as the bf16 operand of the next product
//   D2 [128 (d outputs, padded), 32 pairs] = W2 tile [128, 128] x act [32, 128]^T
//   epilogue 2: the block's partial sum of the unit's output.
// The weight tiles are bf16 images made on the host in the operand layout (umma.cuh) and arrive by
// one bulk copy each; the pairs' inputs are converted and laid out while they are staged.
// 512 threads: warp w reads TMEM lanes 32 (w % 4) .. +31 and the pairs 8 (w / 4) .. +7.
// Shared (dynamic): A1 [4d/8][128][8], A2 [16][128][8], B1 [4d/8][32][8], B2 [16][32][8] bf16, list.
// ------------------------------------------------------------------------------------------------
constexpr int kTP = 32;       // pairs of a tensor-core batch
constexpr int kTcPairTile = 64;  // pairs a tensor-core unit block scans: small tiles keep a popular
                                 // unit's pairs spread over several blocks
constexpr int kUnitTcThreads = 512;  // 16 warps: warp w reads TMEM lanes 32 (w % 4) .. +31, pairs 8 (w / 4) .. +7
constexpr int kTcPairTileMax = 512;  // the tile with thousands of pairs: about 64 pairs of the unit per weight tile loaded

template <int TP>
__global__ void __launch_bounds__(kUnitTcThreads) k_unit_tc(FwdCtx c, int t) {
    constexpr int CW = TP / 4;   // columns (pairs) of a warp's share of an accumulator
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int warp_count[kUnitTcThreads / 32];
    __shared__ int n_list;
    __shared__ __align__(8) uint64_t bar_w, bar_m;
    __shared__ uint32_t tmem_slot;
    const int d = c.m.d, K = c.m.K, H = c.m.H, in = 4 * c.m.d, planes = in >> 3;
    const int P = c.io.B * K, T = c.io.T;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nB = c.nU;
    const int j = blockIdx.x / (nB + 1), cb = blockIdx.x - j * (nB + 1);
    const bool is_gate = cb == nB;
    const int c0 = cb * 128;
    uint4* A1 = reinterpret_cast<uint4*>(dyn);                 // [planes][128]
    uint4* A2 = A1 + planes * 128;                             // [16][128]
    uint4* B1 = A2 + 16 * 128;                                 // [planes][32]
    uint4* B2 = B1 + planes * TP;                             // [16][32]
    int* list = reinterpret_cast<int*>(B2 + 16 * TP);         // [pair_tile]
    const int p0 = blockIdx.y * c.pair_tile;
    HSNW_MARK(0, 11);
    if (tid == 0) {
        mbar_init(&bar_w, 1);
        mbar_init(&bar_m, 1);
        n_list = 0;
    }
    for (int first = 0; first < c.pair_tile; first += kUnitTcThreads) {   // the tile's pairs of unit j, in their order
        const int p = p0 + first + tid;
        const bool mine = first + tid < c.pair_tile && p < P && c.pair_unit[p] == j;
        const unsigned mask = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(mask);
        __syncthreads();
        int before = n_list, total = 0;
        for (int w = 0; w < warp; ++w) before += warp_count[w];
        if (tid == 0) {
            total = before;
            for (int w = 0; w < kUnitTcThreads / 32; ++w) total += warp_count[w];
        }
        if (mine) list[before + __popc(mask & ((1u << lane) - 1u))] = p;
        __syncthreads();   // every read of the counts and of n_list is done
        if (tid == 0) n_list = total;
    }
    __syncthreads();
    const int count = n_list;
    HSNW_MARK(0, 0);
    if (count == 0) return;
    // the weight tiles: one bulk copy each
    if (tid == 0) {
        const uint32_t a1_bytes = static_cast<uint32_t>(planes) * 128 * 16, a2_bytes = 16 * 128 * 16;
        const unsigned char* g1 = is_gate ? static_cast<const unsigned char*>(c.m.umma_gate)
                                          : static_cast<const unsigned char*>(c.m.umma_w1)
                                                + (static_cast<size_t>(j) * nB + cb) * a1_bytes;
        mbar_expect_tx(&bar_w, a1_bytes + (is_gate ? 0u : a2_bytes));
        bulk_g2s(A1, g1, a1_bytes, &bar_w);
        if (!is_gate)
            bulk_g2s(A2, static_cast<const unsigned char*>(c.m.umma_w2) + (static_cast<size_t>(j) * nB + cb) * a2_bytes,
                     a2_bytes, &bar_w);
    }
    HSNW_MARK(0, 8);
    if (warp == 0) tmem_alloc(&tmem_slot, 2 * TP);
    HSNW_MARK(0, 9);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    HSNW_MARK(0, 10);
    const uint32_t taddr = tmem_slot;
    const uint32_t idesc = umma_idesc_bf16(128, TP);
    const int q = warp & 3, hf = warp >> 2;
    const int m = q * 32 + lane;           // this thread's TMEM lane: a hidden column, then an output
    uint32_t phase = 0;
    bool weights_in = false;
    const float4* v4 = reinterpret_cast<const float4*>(c.v);
    // the lane's bias is the same for every batch: its load is off the batches' critical path
    const bool col_ok = is_gate ? m < d : c0 + m < H;
    const float bias = col_ok ? (is_gate ? c.m.gate_b[m] : c.m.b1[j * H + c0 + m]) : 0.0f;
    for (int base = 0; base < count; base += TP) {
        const int nb = min(TP, count - base);
        // the pairs' inputs as the B operand: a thread converts 8 values and stores one 16-byte unit
        // (four units a thread per round, their eight loads in flight together)
        for (int idx0 = tid; idx0 < planes * TP; idx0 += 4 * kUnitTcThreads) {
            float4 lo[4], hi[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = idx0 + u * kUnitTcThreads;
                const int n = idx & (TP - 1), kc = idx / TP;
                lo[u] = hi[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (idx < planes * TP && n < nb) {
                    const float4* src = v4 + static_cast<int64_t>(list[base + n]) * d + kc * 2;
                    lo[u] = src[0];
                    hi[u] = src[1];
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = idx0 + u * kUnitTcThreads;
                if (idx < planes * TP)
                    B1[idx] = make_uint4(pack_bf16x2(lo[u].x, lo[u].y), pack_bf16x2(lo[u].z, lo[u].w),
                                         pack_bf16x2(hi[u].x, hi[u].y), pack_bf16x2(hi[u].z, hi[u].w));
            }
        }
        fence_async_smem();
        if (base == 0) HSNW_MARK(0, 1);
        if (!weights_in) {
            mbar_wait(&bar_w, 0, c.status);
            weights_in = true;
        }
        if (base == 0) HSNW_MARK(0, 2);
        tcgen05_fence_before();
        __syncthreads();
        if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
            tcgen05_fence_after();
            const uint64_t da = umma_desc(A1, 128), db = umma_desc(B1, TP);
            umma_chain(taddr, da, db, idesc, in >> 4, umma_kstep(128), umma_kstep(TP));
            umma_commit(&bar_m);
        }
        mbar_wait(&bar_m, phase, c.status);
        phase ^= 1u;
        tcgen05_fence_after();
        if (base == 0) HSNW_MARK(0, 3);
        // epilogue 1
        {
            float acc[CW];
#pragma unroll
            for (int c8 = 0; c8 < CW; c8 += 8) tmem_ld8(tmem_addr(taddr, q * 32, hf * CW + c8), acc + c8);
            uint16_t* b2_half = reinterpret_cast<uint16_t*>(B2);
#pragma unroll
            for (int i = 0; i < CW; ++i) {
                const int n = hf * CW + i;
                float a = 0.0f;
                if (n < nb && col_ok) {
                    const int pair = list[base + n];
                    const float pre = bf16r(acc[i] + bias);
                    if (is_gate) {
                        c.gate_pre[static_cast<int64_t>(pair) * d + m] = pre;
                    } else {
                        if (c.io.rec_c) {
                            const int row = pair / K, k = pair - row * K;
                            store_hidden(c.io.rec_hidden, ((static_cast<int64_t>(row) * T + t) * K + k) * H + c0 + m, pre, true);
                        }
                        a = gelu_erf(pre);
                    }
                }
                // B2 (n, k = m): plane m / 8, unit n, element m % 8
                if (!is_gate) b2_half[((m >> 3) * TP + n) * 8 + (m & 7)] = bf16_bits(a);
            }
        }
        if (is_gate) {
            tcgen05_fence_before();
            __syncthreads();
            continue;
        }
        if (base == 0) HSNW_MARK(0, 4);
        fence_async_smem();
        tcgen05_fence_before();
        __syncthreads();
        if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
            tcgen05_fence_after();
            const uint64_t da = umma_desc(A2, 128), db = umma_desc(B2, TP);
            umma_chain(taddr + TP, da, db, idesc, 8, umma_kstep(128), umma_kstep(TP));
            umma_commit(&bar_m);
        }
        mbar_wait(&bar_m, phase, c.status);
        phase ^= 1u;
        tcgen05_fence_after();
        if (base == 0) HSNW_MARK(0, 5);
        // epilogue 2: lane m is output x of the unit
        {
            float acc[CW];
#pragma unroll
            for (int c8 = 0; c8 < CW; c8 += 8) tmem_ld8(tmem_addr(taddr, q * 32, TP + hf * CW + c8), acc + c8);
            if (m < d) {
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    const int n = hf * CW + i;
                    if (n < nb) c.part_f[(static_cast<int64_t>(cb) * P + list[base + n]) * d + m] = acc[i];
                }
            }
        }
        tcgen05_fence_before();
        __syncthreads();
        if (base == 0) HSNW_MARK(0, 12);
    }
    HSNW_MARK(0, 6);
    if (warp == 0) tmem_dealloc(taddr, 2 * TP);
    HSNW_MARK(0, 7);
}

// ------------------------------------------------------------------------------------------------
// update: one block per row, 256 threads (512 when K d >= 2048). Reduces the second layer's partial sums, W_out, the
// candidate norm, tanh, sigmoid, the gated write of the K cells, the summary, and the derived
// state of the written cells (their logit parts, V h and maxima).
// Shared (dynamic): F [K d], y [K d], hnew [K d], delta [K d], wo [d d], vt [d d], swh [d M],
// cell_of [K], scale [K].
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512) k_update(FwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int ired[16];
    __shared__ int zero_slot;
    const int N = c.m.N, d = c.m.d, K = c.m.K, M = c.m.M;
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const int B = c.io.B, T = c.io.T, P = B * K;
    const bool bf = c.m.prod_bf16 != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    float* Fs = reinterpret_cast<float*>(dyn);
    float* ys = Fs + K * d;
    float* hnew = ys + K * d;
    float* delta = hnew + K * d;
    float* wo = delta + K * d;
    float* vt = wo + d * d;
    float* swh = vt + d * d;
    int* cell_of = reinterpret_cast<int*>(swh + pad4(d * M));
    float* scale = reinterpret_cast<float*>(cell_of + K);
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    const int64_t pair0 = static_cast<int64_t>(row) * K;
    const int64_t* cells = c.io.cells + rt * K;
    const int64_t* units = c.io.units + rt * K;
    const uint8_t* valid = c.io.valid + rt * K;
    const float* h = state_h(c, row, t);
    const float* q = state_q(c, row, t);
    const bool last = t + 1 == T;
    const bool clear = !last && c.io.reset[rt + 1] != 0;
    const bool tape = c.io.tape_state != 0;
    HSNW_MARK(1, 0);
    cp_async_floats(wo, c.m.wout_t, d * d);
    cp_async_floats(vt, c.m.v_t, d * d);
    cp_async_floats(swh, c.m.score_w_t + static_cast<int64_t>(2 * d) * M, d * M);
    cp_async_commit();
    for (int k = tid; k < K; k += nt) cell_of[k] = valid[k] ? static_cast<int>(cells[k]) : -1;
    if (tid == 0) zero_slot = -1;
    __syncthreads();
    for (int k = tid; k < K; k += nt)
        if (cell_of[k] == 0) zero_slot = k;  // at most one valid slot names cell 0
    // the executed unit's output: the second layer's partial sums in slice order, plus its bias;
    // the loads of an element go out together, four slices at a time
    // (and four elements abreast, in sum4's order: four running sums by slice mod 4)
    for (int e0 = tid; e0 < K * d; e0 += 4 * nt) {
        const float* from[4];
        float bias[4];
        bool ok[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt;
            const int k = min(div_magic(e, dmag), K - 1), x = e - (div_magic(e, dmag)) * d;
            ok[u] = e < K * d && cell_of[k] >= 0;
            from[u] = ok[u] ? c.part_f + (pair0 + k) * d + x : c.part_f;   // a padded slot's sum is not used
            bias[u] = ok[u] ? c.m.b2[static_cast<int>(units[k]) * d + x] : 0.0f;
        }
        const int64_t sa = static_cast<int64_t>(P) * d;
        float acc[4][4] = {};
        int sl = 0;
        for (; sl + 4 <= c.nU; sl += 4)
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int w = 0; w < 4; ++w) acc[u][w] += from[u][(sl + w) * sa];
        for (; sl < c.nU; ++sl)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u][0] += from[u][sl * sa];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt;
            if (e < K * d) Fs[e] = ok[u] ? maybe_bf16((acc[u][0] + acc[u][1]) + (acc[u][2] + acc[u][3]) + bias[u], bf) : 0.0f;
        }
    }
    HSNW_MARK(1, 1);
    cp_async_wait_all();
    __syncthreads();
    HSNW_MARK(1, 2);
    {
        const int per = max(1, min(4, K * d / nt));   // slots a thread: a weight is read once for them
        for (int e = tid; e < ((K + per - 1) / per) * d; e += nt) {
            const int k0 = (div_magic(e, dmag)) * per, x = e - (div_magic(e, dmag)) * d;
            float out[4];
            dot4_rows(Fs + k0 * d, d, min(per, K - k0), wo + x, d, d, out);
            for (int r = 0; r < per && k0 + r < K; ++r) ys[(k0 + r) * d + x] = maybe_bf16(out[r], bf);
        }
    }
    __syncthreads();
    for (int k = warp; k < K; k += warps) {
        float sq = 0.0f;
        for (int x = lane; x < d; x += 32) sq += ys[k * d + x] * ys[k * d + x];
        sq = warp_sum(sq);
        if (lane == 0) scale[k] = rsqrtf(sq / static_cast<float>(d) + c.m.cand_eps);
    }
    __syncthreads();
    float* h_write = tape ? c.io.tape_h + (static_cast<int64_t>(row) * (T + 1) + t + 1) * N * d
                          : c.io.h0 + static_cast<int64_t>(row) * N * d;
    int top = 0;
    HSNW_MARK(1, 3);
    for (int e = tid; e < K * d; e += nt) {
        const int k = div_magic(e, dmag), x = e - k * d;
        const int n = cell_of[k];
        float value = 0.0f, change = 0.0f, cv = 0.0f, bv = 0.0f, gp = 0.0f;
        if (n >= 0) {
            const float old = h[static_cast<int64_t>(n) * d + x];
            cv = tanhf(ys[e] * scale[k] * c.m.cand_w[x]);
            gp = c.gate_pre[(pair0 + k) * d + x];
            bv = sigmoid_f(gp);
            value = (1.0f - bv) * old + bv * cv;
            change = value - old;
            top = max(top, __float_as_int(fabsf(value)));
        }
        hnew[e] = value;
        Fs[e] = maybe_bf16(value, bf);  // the new state at the products' operand precision (F is spent)
        delta[e] = change;
        if (c.io.rec_c) {
            c.io.rec_c[rt * K * d + e] = cv;
            c.io.rec_b[rt * K * d + e] = bv;
            c.io.rec_y[rt * K * d + e] = ys[e];
            c.io.rec_gate_pre[rt * K * d + e] = gp;
        }
    }
    __syncthreads();
    // the state after the position: the tape's next record already holds a copy of this one (the
    // front phase wrote it, zeroed if the next position resets), so only the written cells move
    float* lh_row = c.lh + static_cast<int64_t>(row) * N * M;
    float* vh_row = c.vh + static_cast<int64_t>(row) * N * d;
    int* cmax_row = c.cmax + static_cast<int64_t>(row) * N;
    HSNW_MARK(1, 4);
    if (!clear) {
        for (int e = tid; e < K * d; e += nt) {
            const int k = div_magic(e, dmag), x = e - k * d;
            if (cell_of[k] >= 0) h_write[static_cast<int64_t>(cell_of[k]) * d + x] = hnew[e];
        }
        // the written cells' derived state: 32 threads a slot
        for (int k = warp; k < K; k += warps) {
            const int n = cell_of[k];
            if (n < 0) continue;
            derive_outputs(c, Fs + k * d, swh, vt, lh_row + static_cast<int64_t>(n) * M,
                           vh_row + static_cast<int64_t>(n) * d, lane, 32);
            int m = 0;
            for (int x = lane; x < d; x += 32) m = max(m, __float_as_int(fabsf(hnew[k * d + x])));
            for (int w = 16; w > 0; w >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, w));
            if (lane == 0) cmax_row[n] = m;
        }
    } else {
        if (!tape)
            for (int e = tid; e < N * d; e += nt) h_write[e] = 0.0f;
        for (int e = tid; e < N * M; e += nt) lh_row[e] = 0.0f;
        for (int e = tid; e < N * d; e += nt) vh_row[e] = 0.0f;
        for (int n = tid; n < N; n += nt) cmax_row[n] = 0;
    }
    float* q_next = tape ? c.io.tape_q + (static_cast<int64_t>(row) * (T + 1) + t + 1) * d
                         : c.io.q0 + static_cast<int64_t>(row) * d;
    HSNW_MARK(1, 5);
    for (int x = tid; x < d; x += nt) {
        float sum = 0.0f;
        for (int k = 0; k < K; ++k) sum += delta[k * d + x];
        const float after = q[x] + sum / static_cast<float>(N);
        c.io.qs[rt * d + x] = after;
        q_next[x] = clear ? 0.0f : after;
    }
    for (int e = tid; e < K * d; e += nt) {
        const int k = div_magic(e, dmag), x = e - k * d;
        float value;
        if (cell_of[k] >= 0) value = hnew[e];
        else value = zero_slot >= 0 ? hnew[zero_slot * d + x] : h[x];
        c.io.h_sel[rt * K * d + e] = value;
    }
    if (tape) {
        if (!clear) {
            int64_t* age_next = c.io.tape_age + (static_cast<int64_t>(row) * (T + 1) + t + 1) * N;
            for (int k = tid; k < K; k += nt)
                if (cell_of[k] >= 0) age_next[cell_of[k]] = 0;
        }
    } else {
        int64_t* ages = c.io.age0 + static_cast<int64_t>(row) * N;
        for (int n = tid; n < N; n += nt) ages[n] = clear ? 0 : ages[n] + 1;
        __syncthreads();
        for (int k = tid; k < K; k += nt)
            if (cell_of[k] >= 0) ages[cell_of[k]] = 0;
    }
    if (c.io.h_max) {
        for (int w = 16; w > 0; w >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, w));
        if (lane == 0) ired[warp] = top;
        __syncthreads();
        if (tid == 0) {
            int mx = c.hmax_part[row];
            for (int w = 0; w < warps; ++w) mx = max(mx, ired[w]);
            c.io.h_max[rt] = __int_as_float(mx);
        }
    }
    HSNW_MARK(1, 6);
    if (last && row == 0 && tid == 0) c.status[4] = c.io.tape_state ? 0 : c.marker;
    if (last && tid == 0) {
        // the position counter after the window (reference compile.py:1194-1200)
        int last_reset = 0;
        for (int s = 0; s < T; ++s)
            if (c.io.reset[static_cast<int64_t>(row) * T + s]) last_reset = s + 1;
        c.io.pos[row] = last_reset > 0 ? T + 1 - last_reset : c.io.pos[row] + T;
    }
}

size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct Layout {
    size_t status, pre_s, part_front, v, pair_unit, part_f, gate_pre, hmax_part, lh, vh, cmax, total;
};
Layout layout(const HsnwModel& m, int B, int T) {
    Layout L;
    const int nF = (m.H + kFS - 1) / kFS, nU = (m.H + kUS - 1) / kUS;
    const size_t Bz = static_cast<size_t>(B);
    size_t off = 0;
    L.status = off; off += 256 + 4 * 512 * 16 * sizeof(unsigned long long);  // status word, then the trace area
    L.pre_s = off; off += align_up(sizeof(float) * Bz * T * m.H);
    L.part_front = off; off += align_up(sizeof(float) * 2 * nF * Bz * m.d);
    L.v = off; off += align_up(sizeof(float) * Bz * m.K * 4 * m.d);
    L.pair_unit = off; off += align_up(sizeof(int) * Bz * m.K);
    L.part_f = off; off += align_up(sizeof(float) * nU * Bz * m.K * m.d);
    L.gate_pre = off; off += align_up(sizeof(float) * Bz * m.K * m.d);
    L.hmax_part = off; off += align_up(sizeof(int) * Bz);
    L.lh = off; off += align_up(sizeof(float) * Bz * m.N * m.M);
    L.vh = off; off += align_up(sizeof(float) * Bz * m.N * m.d);
    L.cmax = off; off += align_up(sizeof(int) * Bz * m.N);
    L.total = off;
    return L;
}

// 512 threads shorten a large row's scorer; with more rows than SMs 256 let more blocks share an SM
int row_threads(const HsnwModel& m, int B) { return m.N > 512 && B <= hsnw_sm_count_current() ? 512 : 256; }
// the per-cell logit parts and scalars of a row are staged in shared memory while they are small
bool stage_cells_fit(const HsnwModel& m) { return sizeof(float) * static_cast<size_t>(m.N) * (m.M + m.S) <= 96 * 1024; }

size_t row_shared(const HsnwModel& m, bool staged) {
    const int d = m.d, K = m.K, D = m.D, N = m.N, nF2 = 2 * ((m.H + kFS - 1) / kFS);
    const size_t cells = staged ? static_cast<size_t>(pad4(N * m.M)) + pad4(N * m.S) : 0;
    const size_t words = static_cast<size_t>(pad4(nF2 * d)) + cells + pad4(2 * N) + pad4(N)
        + static_cast<size_t>(K + K * D) * d + static_cast<size_t>(K) * d + pad4(2 * d * m.M) + pad4((1 + m.S) * m.M)
        + 2 * static_cast<size_t>(pad4(N)) + 2 * d + 2 * kMaxM + 2 * static_cast<size_t>(pad4(K * D)) + pad4(K);
    return sizeof(float) * words;
}
// Staging saves a second pass over memory when a row's block has the SM to itself; with more rows
// than SMs the blocks' residency matters more: then stage only if two blocks still fit an SM.
bool stage_cells(const HsnwModel& m, int B) {
    if (!stage_cells_fit(m)) return false;
    const int sms = hsnw_sm_count_current();
    return !(sms > 0 && B > sms && 2 * (row_shared(m, true) + 2048) > hsnw_max_shared());
}
size_t init_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(2 * kInitCells) * m.d + static_cast<size_t>(m.d) * m.M + static_cast<size_t>(m.d) * m.d);
}
size_t front_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(2) * m.d * kFS + static_cast<size_t>(kFRBig) * m.d + kFRBig * kFS);
}
size_t unit_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(kPB) * 4 * m.d + static_cast<size_t>(4) * m.d * kUS
        + static_cast<size_t>(kUS) * m.d + kPB * kUS + kPairTile);
}
size_t unit_tc_shared(const HsnwModel& m, int tp = kTP) {
    const size_t planes = static_cast<size_t>(4 * m.d) / 8;
    return 16 * (planes * 128 + 16 * 128 + planes * tp + 16 * tp) + sizeof(int) * kTcPairTileMax;
}
size_t update_shared(const HsnwModel& m) {
    return sizeof(float) * (4 * static_cast<size_t>(m.K) * m.d + 2 * static_cast<size_t>(m.d) * m.d + pad4(m.d * m.M) + 2 * m.K);
}

int check_model(const HsnwModel* m) {
    if (!m) return hsnw_fail(HSNW_E_ARG, "model is null");
    if (m->N < 1 || m->d < 4 || (m->d & 3) || m->K < 1 || m->K > m->N || m->H < 1 || m->M < 1 || m->D < 1
        || m->S < 0 || m->dc < 0)
        return hsnw_fail(HSNW_E_ARG, "window: sizes must be positive, K <= N and d a multiple of 4");
    if (m->M > kMaxM) return hsnw_fail(HSNW_E_UNSUPPORTED, "window: at most 16 units (M)");
    if (m->K > kMaxSlots) return hsnw_fail(HSNW_E_UNSUPPORTED, "window: at most 64 slots (K)");
    const size_t cap = hsnw_max_shared() - 4096;  // room for the kernels' static shared memory
    if (row_shared(*m, false) > cap || front_shared(*m) > cap || unit_shared(*m) > cap || update_shared(*m) > cap
        || init_shared(*m) > cap)
        return hsnw_fail(HSNW_E_UNSUPPORTED, "window: a phase's working set exceeds a block's shared memory");
    return HSNW_OK;
}

}  // namespace

extern "C" int64_t hsnw_forward_scratch_bytes(const HsnwModel* model, int32_t B, int32_t T) {
    if (!model || B < 1 || T < 1) return 0;
    return static_cast<int64_t>(layout(*model, B, T).total);
}

// where k_pre_tc reports a bounded wait that ran out: the forward's scratch word while a forward
// call is being enqueued, else nowhere
static thread_local int* g_pre_status = nullptr;

extern "C" int hsnw_front_projection(const HsnwModel* model, const float* z, const float* ctx, int64_t rows,
                                     float* out, void* stream) {
    if (!model || !z || !ctx || !out || rows < 1) return hsnw_fail(HSNW_E_ARG, "front_projection: null or empty");
    if (model->prod_bf16) {
        // bf16 products: the tensor-core tile kernel (status: the caller's scratch word, or none)
        const int Kp = (model->d + model->dc + 15) & ~15;
        const size_t shared = static_cast<size_t>(2) * (Kp / 8) * 128 * 16;
        if (shared <= hsnw_max_shared() - 4096) {
            const unsigned row_tiles = static_cast<unsigned>((rows + 127) / 128);
            hsnw_profile_mark(HSNW_K_PRE, static_cast<cudaStream_t>(stream));
            if (row_tiles * ((model->H + 127) / 128) >= 64) {
                const dim3 grid(row_tiles, static_cast<unsigned>((model->H + 127) / 128));
                k_pre_tc<128><<<grid, 128, shared, static_cast<cudaStream_t>(stream)>>>(*model, z, ctx, rows, out, g_pre_status);
            } else {   // few rows (a serving step): narrow tiles, four times the blocks
                const dim3 grid(row_tiles, static_cast<unsigned>((model->H + 31) / 32));
                k_pre_tc<32><<<grid, 128, shared, static_cast<cudaStream_t>(stream)>>>(*model, z, ctx, rows, out, g_pre_status);
            }
            return hsnw_check_launch("front_projection");
        }
    }
    const dim3 grid(static_cast<unsigned>((rows + kSlice - 1) / kSlice), static_cast<unsigned>((model->H + kSlice - 1) / kSlice));
    hsnw_profile_mark(HSNW_K_PRE, static_cast<cudaStream_t>(stream));
    k_pre<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(*model, z, ctx, rows, out);
    return hsnw_check_launch("front_projection");
}

static int forward_impl(const HsnwModel* model, const HsnwForward* io, void* stream_, bool phases = false,
                        bool carried = false) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (int rc = check_model(model)) return rc;
    if (!io || io->B < 1 || io->T < 1) return hsnw_fail(HSNW_E_ARG, "window_forward: B and T must be positive");
    if (!io->z || !io->ctx || !io->scalars || !io->reset || !io->h0 || !io->q0 || !io->age0 || !io->pos
        || !io->cells || !io->units || !io->valid || !io->refreshed || !io->theta || !io->h_sel || !io->qs)
        return hsnw_fail(HSNW_E_ARG, "window_forward: a required pointer is null");
    if (io->tape_state && (!io->tape_h || !io->tape_q || !io->tape_age || !io->h_max))
        return hsnw_fail(HSNW_E_ARG, "window_forward: the state tape is missing");
    if (io->rec_c && (!io->rec_b || !io->rec_h_old || !io->rec_y || !io->rec_gate_pre || !io->rec_m
        || !io->rec_rms || !io->rec_hidden))
        return hsnw_fail(HSNW_E_ARG, "window_forward: the record is all or nothing");
    const Layout L = layout(*model, io->B, io->T);
    if (!io->scratch || io->scratch_bytes < static_cast<int64_t>(L.total)
        || (reinterpret_cast<uintptr_t>(io->scratch) & 255))
        return hsnw_fail(HSNW_E_ARG, "window_forward: scratch too small or not 256-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    FwdCtx c;
    c.m = *model;
    c.io = *io;
    const bool unit_tc = model->prod_bf16 && model->umma_w1 && model->umma_gate && model->umma_w2 && model->d <= 128
        && unit_tc_shared(*model) <= hsnw_max_shared() - 4096;
    c.nF = (model->H + kFS - 1) / kFS;
    c.nU = unit_tc ? (model->H + 127) / 128 : (model->H + kUS - 1) / kUS;
    c.nG = (model->d + kUS - 1) / kUS;
    const int B = io->B, T = io->T;
    c.front_rows = B >= 256 ? kFRBig : kFR;
    c.n_front = 2 * c.nF * ((B + c.front_rows - 1) / c.front_rows);
    c.stage_cells = stage_cells(*model, io->B) ? 1 : 0;
    c.carried = carried ? 1 : 0;
    c.marker = 0x5eed0000 ^ io->B ^ (io->T << 12);
    c.copy_per_row = io->tape_state ? (model->N * model->d + kCopyFloats - 1) / kCopyFloats : 0;
    unsigned char* base = static_cast<unsigned char*>(io->scratch);
    c.status = reinterpret_cast<int*>(base + L.status);
    c.trace = reinterpret_cast<unsigned long long*>(base + L.status + 256);
    c.pre_s = reinterpret_cast<float*>(base + L.pre_s);
    c.part_front = reinterpret_cast<float*>(base + L.part_front);
    c.v = reinterpret_cast<float*>(base + L.v);
    c.pair_unit = reinterpret_cast<int*>(base + L.pair_unit);
    c.part_f = reinterpret_cast<float*>(base + L.part_f);
    c.gate_pre = reinterpret_cast<float*>(base + L.gate_pre);
    c.hmax_part = reinterpret_cast<int*>(base + L.hmax_part);
    c.lh = reinterpret_cast<float*>(base + L.lh);
    c.vh = reinterpret_cast<float*>(base + L.vh);
    c.cmax = reinterpret_cast<int*>(base + L.cmax);
    bool pre_done = false;   // the window-invariant front product is the same for both kernel families
    if (!phases && !model->phases_only && model->rows_bank) {
        // one persistent cluster per row when the shape fits (window_rows.cu)
        // (the status word, and the marker of derived values in the scratch: the row kernels keep none there)
        if (cudaMemsetAsync(c.status, 0, 8 * sizeof(int), stream) != cudaSuccess) return hsnw_check_launch("window_forward");
        g_pre_status = c.status;
        const int rc_pre = hsnw_front_projection(model, io->z, io->ctx, static_cast<int64_t>(B) * T, c.pre_s, stream);
        g_pre_status = nullptr;
        if (rc_pre) return rc_pre;
        pre_done = true;
        // an error of the row kernel's launch is the call's error; only a shape it does not take goes on
        const int rc_rows = hsnw_rows_forward(model, io, c.pre_s, c.status, stream);
        if (rc_rows != HSNW_DECLINED) {
            if (rc_rows == HSNW_OK) hsnw_set_path(HSNW_PATH_ROWS);
            return rc_rows;
        }
    }
    hsnw_set_path(HSNW_PATH_PHASES);
    const int rthreads = row_threads(*model, B);
    const int init_tiles = (model->N + kInitCells - 1) / kInitCells;
    const dim3 init_grid(B, c.carried ? (init_tiles < 8 ? init_tiles : 8) : init_tiles);   // carried: few blocks a row; as a rule they only look at the marker
    hsnw_profile_mark(HSNW_K_INIT, stream);
    k_init<<<init_grid, 256, init_shared(*model), stream>>>(c);
    if (!pre_done) {
        g_pre_status = c.status;
        const int rc_pre = hsnw_front_projection(model, io->z, io->ctx, static_cast<int64_t>(B) * T, c.pre_s, stream);
        g_pre_status = nullptr;
        if (rc_pre) return rc_pre;
    }
    const int front_grid = c.n_front + B * c.copy_per_row;
    c.pair_tile = B * model->K > 1024 ? kTcPairTileMax : kTcPairTile;
    // batches of 64 pairs where there are thousands of pairs and the wider operands still fit
    const bool tp64 = unit_tc && B * model->K > 1024 && unit_tc_shared(*model, 64) <= hsnw_max_shared() - 4096;
    const int pair_tile = unit_tc ? c.pair_tile : kPairTile;
    const dim3 unit_grid(model->M * (unit_tc ? c.nU + 1 : c.nU + c.nG), (B * model->K + pair_tile - 1) / pair_tile);
    const size_t sh_front = front_shared(*model), sh_row = row_shared(*model, c.stage_cells != 0);
    const size_t sh_unit = unit_shared(*model), sh_update = update_shared(*model), sh_unit_tc = unit_tc_shared(*model, tp64 ? 64 : kTP);
    for (int t = 0; t < T; ++t) {
        hsnw_profile_mark(HSNW_K_FRONT, stream);
        k_front<<<front_grid, 256, sh_front, stream>>>(c, t);
        hsnw_profile_mark(HSNW_K_ROW, stream);
        k_row<<<B, rthreads, sh_row, stream>>>(c, t);
        hsnw_profile_mark(HSNW_K_UNIT, stream);
        if (unit_tc && tp64) k_unit_tc<64><<<unit_grid, kUnitTcThreads, sh_unit_tc, stream>>>(c, t);
        else if (unit_tc) k_unit_tc<32><<<unit_grid, kUnitTcThreads, sh_unit_tc, stream>>>(c, t);
        else k_unit<<<unit_grid, 256, sh_unit, stream>>>(c, t);
        hsnw_profile_mark(HSNW_K_UPDATE, stream);
        k_update<<<B, model->K * model->d >= 2048 ? 512 : 256, sh_update, stream>>>(c, t);
        if (int rc = hsnw_check_launch("window_forward")) return rc;
    }
    return HSNW_OK;
}

extern "C" int hsnw_window_forward(const HsnwModel* model, const HsnwForward* io, void* stream) {
    return forward_impl(model, io, stream);
}

extern "C" int hsnw_stream_step(const HsnwModel* model, const HsnwForward* io, void* stream) {
    if (io && (io->T != 1 || io->tape_state))
        return hsnw_fail(HSNW_E_ARG, "stream_step: one position on a resident state (T = 1, tape_state = 0)");
    return forward_impl(model, io, stream, true);
}

extern "C" int hsnw_stream_continue(const HsnwModel* model, const HsnwForward* io, void* stream) {
    if (io && io->tape_state)
        return hsnw_fail(HSNW_E_ARG, "stream_continue: a resident state (tape_state = 0)");
    return forward_impl(model, io, stream, true, true);
}

void hsnw_forward_set_attributes() {
    const struct { const void* f; const char* n; } ks[] = {
        {reinterpret_cast<const void*>(k_init), "init"}, {reinterpret_cast<const void*>(k_pre_tc<128>), "pre_tc"}, {reinterpret_cast<const void*>(k_pre_tc<32>), "pre_tc32"},
        {reinterpret_cast<const void*>(k_front), "front"},
        {reinterpret_cast<const void*>(k_row), "row"}, {reinterpret_cast<const void*>(k_unit), "unit"},
        {reinterpret_cast<const void*>(k_unit_tc<32>), "unit_tc"},
        {reinterpret_cast<const void*>(k_unit_tc<64>), "unit_tc64"},
        {reinterpret_cast<const void*>(k_update), "update"}};
    for (const auto& k : ks)
        if (!hsnw_opt_in(k.f, k.n)) hsnw_attribute_failed();
}
