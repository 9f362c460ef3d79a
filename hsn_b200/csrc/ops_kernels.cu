// The window kernels that are launched by name through hsnw_launch, with the launch descriptor
// and the p[] / i[] / f[] slot meanings of the reference kernels of the same names
// (reference kernels/cuda/hsn_window.cu: hsn_win_select :533-562, hsn_win_cell_update :751-791,
// hsn_win_recurrence :50-58, hsn_win_recurrence_dense :117-123), so the reference's Python
// wrappers can drive them unchanged. The implementations are this library's own: one thread
// block per batch row, fp32 state, every reduction in a fixed order, no atomics.
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "select.cuh"

using namespace hsnw;

namespace {
__device__ __forceinline__ float load_as_float(const void* p, int64_t index, bool half) {
    return half ? bf16_value(static_cast<const uint16_t*>(p)[index]) : static_cast<const float*>(p)[index];
}
__device__ __forceinline__ void store_from_float(void* p, int64_t index, bool half, float v) {
    if (half) static_cast<uint16_t*>(p)[index] = bf16_bits(v);
    else static_cast<float*>(p)[index] = v;
}
}  // namespace

// ------------------------------------------------------------------------------------------------
// hsn_win_select: the hard decision of one position. One block per row, any multiple of 32 threads.
//   p: 0 logits [B,N,M] f32 (or the first M columns of a product [B N, W], f32 | bf16);
//      1 age [B,n_age,N] i64 (record t); 2 cost [M] f32; 3 cells, 4 units [B,n_out,K] i64,
//      5 valid [B,n_out,K] u8, 6 theta [B,n_out] f32, 7 refreshed [B,n_out,K] u8 (record t).
//   i: 0 B, 1 N, 2 M, 3 K, 4 age_max, 5 probes, 6 t, 7 n_out, 8 n_age, 9 W (0: M), 10 bf16 logits,
//      11 reserved cells, 12 reserved slots run unit k mod M.
//   f: 0 lambda_cost, 1 cell_overhead, 2 shared_cost, 3 limit.
// Dynamic shared memory: 2 N words (scores, units). K <= 64, M <= 64.
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_select(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ SelectShared S;
    const int N = a.i[1], M = a.i[2], K = a.i[3];
    const int t = a.i[6], n_out = a.i[7], n_age = a.i[8];
    const int width = a.i[9] > 0 ? a.i[9] : M;
    const bool half = a.i[10] != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const float lambda = a.f[0];
    float* score = reinterpret_cast<float*>(dyn);
    int* unit = reinterpret_cast<int*>(score + N);
    const float* cost = static_cast<const float*>(a.p[2]);
    for (int j = tid; j < M; j += nt) S.cost[j] = cost[j];
    const int64_t base = static_cast<int64_t>(row) * N * width;
    for (int i = tid; i < N; i += nt) {
        const int64_t r = base + static_cast<int64_t>(i) * width;
        float best = -INFINITY;
        int arg = 0;
        for (int j = 0; j < M; ++j) {
            const float logit = load_as_float(a.p[0], r + j, half);
            // the product and the difference are rounded separately, as torch's two ops are
            const float s = lambda > 0.0f ? __fsub_rn(logit, __fmul_rn(lambda, cost[j])) : logit;
            if (j == 0 || s > best) {
                best = s;
                arg = j;
            }
        }
        score[i] = best;
        unit[i] = arg;
    }
    __syncthreads();
    SelectParams P;
    P.N = N; P.M = M; P.K = K; P.age_max = a.i[4]; P.probes = a.i[5] != 0;
    P.reserved = a.i[11]; P.fixed_units = a.i[12] != 0;
    P.overhead = a.f[1]; P.shared_cost = a.f[2]; P.limit = a.f[3];
    const int64_t* age = static_cast<const int64_t*>(a.p[1]) + (static_cast<int64_t>(row) * n_age + t) * N;
    select_row(P, score, unit, age, S);
    const int64_t rec = static_cast<int64_t>(row) * n_out + t;
    int64_t* cells = static_cast<int64_t*>(a.p[3]) + rec * K;
    int64_t* units = static_cast<int64_t*>(a.p[4]) + rec * K;
    uint8_t* valid = static_cast<uint8_t*>(a.p[5]) + rec * K;
    uint8_t* refreshed = static_cast<uint8_t*>(a.p[7]) + rec * K;
    for (int k = tid; k < K; k += nt) {
        cells[k] = S.out_cell[k];
        units[k] = S.out_unit[k];
        valid[k] = static_cast<uint8_t>(S.out_flag[k] & 1);
        refreshed[k] = static_cast<uint8_t>((S.out_flag[k] >> 1) & 1);
    }
    if (tid == 0) static_cast<float*>(a.p[6])[rec] = S.theta;
}

// ------------------------------------------------------------------------------------------------
// hsn_win_cell_update: the end of one position's round (candidate norm, tanh, gate, gated write,
// summary, ages, tick, the slots' cells after the update, the row's max |h|, the next position's
// reset and, in the folded form, the next position's input row [z; q; ctx (; f)]).
//   p: 0 y [B,K,d], 1 gate [B K, stride] (f32 | bf16), 2 h [B,n_state,N,d], 3 q [B,n_state,d] f32,
//      4 age [B,n_state,N] i64 (record t), 5 pos [B] i64, 6 cells [B,n_slot,K] i64,
//      7 valid [B,n_slot,K] u8 (record t), 8 cand_w [d], 9 h_next, 10 q_next, 11 age_next (record
//      t_out), 12 pos_next, 13 h_sel [B,n_slot,K,d], 14 h_max [B,n_slot], 15 reset [B,n_slot] u8,
//      16 q_post [B,n_slot,d], 17 x [n_slot,B,d_z+d+d_c(+d)], 18 z [B,n_slot,d_z],
//      19 context [B,n_slot,d_c].
//   i: 0 B, 1 N, 2 d, 3 K, 4 cand_norm, 5 t, 6 n_state, 7 n_slot, 8 t_out, 9 has_reset, 10 has_pos,
//      11 has_post, 12 y bf16, 13 gate bf16, 14 gate stride (0: d), 15 write x, 16 x bf16, 17 d_z,
//      18 z bf16, 19 d_c, 20 ctx bf16, 21 fast cells.   f: 0 cand_eps.
// Dynamic shared memory: (N + 2 K d + 2 K) words. Any multiple of 32 threads.
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_cell_update(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ uint64_t red[33];
    const int B = a.i[0], N = a.i[1], d = a.i[2], K = a.i[3];
    const bool cand_norm = a.i[4] != 0;
    const int t = a.i[5], n_state = a.i[6], n_slot = a.i[7], t_out = a.i[8];
    const bool has_reset = a.i[9] != 0, has_pos = a.i[10] != 0, has_post = a.i[11] != 0;
    const bool y_half = a.i[12] != 0, gate_half = a.i[13] != 0;
    const int gate_stride = a.i[14] > 0 ? a.i[14] : d;
    const float cand_eps = a.f[0];
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    const int64_t s_in = static_cast<int64_t>(row) * n_state + t;
    const int64_t s_out = static_cast<int64_t>(row) * n_state + t_out;
    const int64_t rec = static_cast<int64_t>(row) * n_slot + t;
    const int64_t y_row = static_cast<int64_t>(row) * K * d;
    const int64_t gate_row = static_cast<int64_t>(row) * K * gate_stride;
    const float* h = static_cast<const float*>(a.p[2]) + s_in * N * d;
    const float* q = static_cast<const float*>(a.p[3]) + s_in * d;
    const int64_t* age = static_cast<const int64_t*>(a.p[4]) + s_in * N;
    const int64_t* cells = static_cast<const int64_t*>(a.p[6]) + rec * K;
    const uint8_t* valid = static_cast<const uint8_t*>(a.p[7]) + rec * K;
    const float* cand_w = static_cast<const float*>(a.p[8]);
    float* h_next = static_cast<float*>(a.p[9]) + s_out * N * d;
    float* q_next = static_cast<float*>(a.p[10]) + s_out * d;
    int64_t* age_next = static_cast<int64_t*>(a.p[11]) + s_out * N;
    float* h_sel = static_cast<float*>(a.p[13]) + rec * K * d;
    int* slot_of = reinterpret_cast<int*>(dyn);          // [N] the slot that writes the cell, or -1
    float* h_new = reinterpret_cast<float*>(slot_of + N);  // [K, d]
    float* delta = h_new + K * d;                        // [K, d]
    int* cell_of = reinterpret_cast<int*>(delta + K * d);  // [K] the slot's cell, -1 if padded
    float* scale = reinterpret_cast<float*>(cell_of + K);  // [K]
    const bool clear = has_reset && static_cast<const uint8_t*>(a.p[15])[rec + 1] != 0;
    for (int n = tid; n < N; n += nt) slot_of[n] = -1;
    for (int k = tid; k < K; k += nt) cell_of[k] = valid[k] ? static_cast<int>(cells[k]) : -1;
    __syncthreads();
    for (int k = tid; k < K; k += nt)
        if (cell_of[k] >= 0) slot_of[cell_of[k]] = k;  // valid slots name distinct cells
    // the candidate norm: a warp per slot folds the squares (lane-strided sums, then a shuffle tree)
    for (int k = warp; k < K; k += warps) {
        float sq = 0.0f;
        if (cand_norm)
            for (int x = lane; x < d; x += 32) {
                const float v = load_as_float(a.p[0], y_row + k * d + x, y_half);
                sq += v * v;
            }
        sq = warp_sum(sq);
        if (lane == 0) scale[k] = cand_norm ? rsqrtf(sq / static_cast<float>(d) + cand_eps) : 1.0f;
    }
    __syncthreads();
    for (int e = tid; e < K * d; e += nt) {
        const int k = e / d, x = e - k * d;
        const int n = cell_of[k];
        float value = 0.0f, change = 0.0f;
        if (n >= 0) {
            const float old = h[static_cast<int64_t>(n) * d + x];
            const float yv = load_as_float(a.p[0], y_row + e, y_half);
            const float pre = cand_norm ? yv * scale[k] * cand_w[x] : yv;
            const float c = tanhf(pre);
            const float gv = load_as_float(a.p[1], gate_row + static_cast<int64_t>(k) * gate_stride + x, gate_half);
            const float b = sigmoid_f(gv);
            value = (1.0f - b) * old + b * c;
            change = value - old;
        }
        h_new[e] = value;
        delta[e] = change;
    }
    __syncthreads();
    const bool next_input = a.i[15] != 0 && t + 1 < n_slot, x_half = a.i[16] != 0;
    const int d_z = a.i[17], d_c = a.i[19], n_fast = a.i[21];
    const int x_width = d_z + d + d_c + (n_fast > 0 ? d : 0);
    const int64_t next_row = (static_cast<int64_t>(t + 1) * B + row) * x_width;
    for (int x = tid; x < d; x += nt) {
        float sum = 0.0f;
        for (int k = 0; k < K; ++k) sum += delta[k * d + x];  // slot order
        const float after = q[x] + sum / static_cast<float>(N);
        if (has_post) static_cast<float*>(a.p[16])[rec * d + x] = after;
        q_next[x] = clear ? 0.0f : after;
        if (next_input) store_from_float(a.p[17], next_row + d_z + x, x_half, clear ? 0.0f : after);
    }
    if (next_input) {
        const int64_t from = static_cast<int64_t>(row) * n_slot + t + 1;
        const bool z_half = a.i[18] != 0, c_half = a.i[20] != 0;
        for (int e = tid; e < d_z; e += nt)
            store_from_float(a.p[17], next_row + e, x_half, load_as_float(a.p[18], from * d_z + e, z_half));
        for (int e = tid; e < d_c; e += nt)
            store_from_float(a.p[17], next_row + d_z + d + e, x_half, load_as_float(a.p[19], from * d_c + e, c_half));
        if (n_fast > 0) {
            for (int x = tid; x < d; x += nt) {
                float sum = 0.0f;
                for (int n = 0; n < n_fast; ++n) {
                    const int k = slot_of[n];
                    sum += k >= 0 ? h_new[k * d + x] : h[static_cast<int64_t>(n) * d + x];
                }
                store_from_float(a.p[17], next_row + d_z + d + d_c + x, x_half,
                                 clear ? 0.0f : sum / static_cast<float>(n_fast));
            }
        }
    }
    for (int n = tid; n < N; n += nt) age_next[n] = (clear || slot_of[n] >= 0) ? 0 : age[n] + 1;
    if (has_pos && tid == 0)
        static_cast<int64_t*>(a.p[12])[row] = static_cast<const int64_t*>(a.p[5])[row] + 1;
    // the slots' cells after the update; a padded slot reads cell 0
    for (int e = tid; e < K * d; e += nt) {
        const int k = e / d, x = e - k * d;
        float value;
        if (cell_of[k] >= 0) value = h_new[e];
        else {
            const int zero = slot_of[0];
            value = zero >= 0 ? h_new[zero * d + x] : h[x];
        }
        h_sel[e] = value;
    }
    // the next state: written cells from shared memory, the others carried over with 16-byte
    // transfers; the row's max |h| by the integer order of the bit patterns (a NaN is the largest)
    int top = 0;
    const bool vec = (d & 3) == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(h_next)
        | reinterpret_cast<uintptr_t>(h_new)) & 15) == 0;
    if (vec) {
        const int d4 = d >> 2;
        const float4* src = reinterpret_cast<const float4*>(h);
        float4* dst = reinterpret_cast<float4*>(h_next);
        for (int e = tid; e < N * d4; e += nt) {
            const int n = e / d4, x4 = e - n * d4;
            const int k = slot_of[n];
            float4 v = k >= 0 ? reinterpret_cast<const float4*>(h_new + k * d)[x4] : src[e];
            top = max(top, __float_as_int(fabsf(v.x)));
            top = max(top, __float_as_int(fabsf(v.y)));
            top = max(top, __float_as_int(fabsf(v.z)));
            top = max(top, __float_as_int(fabsf(v.w)));
            if (clear) v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            dst[e] = v;
        }
    } else {
        for (int e = tid; e < N * d; e += nt) {
            const int n = e / d, x = e - n * d;
            const int k = slot_of[n];
            const float v = k >= 0 ? h_new[k * d + x] : h[e];
            top = max(top, __float_as_int(fabsf(v)));
            h_next[e] = clear ? 0.0f : v;
        }
    }
    // an integer maximum over the block (bit patterns of non-negative floats order like ints)
    int* ired = reinterpret_cast<int*>(red);
    for (int w = 16; w > 0; w >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, w));
    if (lane == 0) ired[warp] = top;
    __syncthreads();
    if (tid == 0) {
        int m = 0;
        for (int w = 0; w < warps; ++w) m = max(m, ired[w]);
        static_cast<float*>(a.p[14])[rec] = __int_as_float(m);
    }
}

// ------------------------------------------------------------------------------------------------
// hsn_win_recurrence: the full-cut backward state recurrence of a window (reference semantics:
// python/hsn/train/split.py:128-174), t = T-1 .. 0, one block per row.
//   p: 0 c, 1 b, 2 h_old [B,T,K,d] f32; 3 cells [B,T,K] i64; 4 valid [B,T,K] u8; 5 reset [B,T] u8;
//      6 d_q_pre, 7 d_q_post [B,T,d], 8 d_h_sel [B,T,K,d] (read when flagged); 9 dc, 10 db out.
//      This library adds (zero in the reference's calls): 11 A [B,N,d], 12 R [B,d] in/out.
//   i: 0 B, 1 T, 2 K, 3 d, 4 N, 5 has_pre, 6 has_post, 7 has_sel, 8 carry: start from p11/p12 and
//      store the final cotangents there (zeroed on rows whose position 0 resets).
// Dynamic shared memory: (N + 1) d words (up to 227 KB after hsnw_prepare): the row's cotangent A.
//
// How the work is laid out. A position touches only the K selected cells, and along the state
// width every column is independent. A thread owns one (slot, group of V columns) item, V = 4 when
// d is a multiple of 4 (16-byte loads and stores) and 1 otherwise; it keeps the summary's
// cotangent R for its own columns in registers (every item of a column group adds the same
// d_q_post / d_q_pre, so the copies stay equal and R never crosses threads). The valid slots of a
// position name distinct cells, so a position's items never meet in A; across positions a cell
// may change hands, hence ONE block barrier a position. The position's record is loaded into
// registers one position ahead, so the loads of t-1 are in flight under the arithmetic of t.
// ------------------------------------------------------------------------------------------------
namespace {

template <int V>
struct Pack {
    float v[V];
};
template <int V>
__device__ __forceinline__ Pack<V> load_pack(const float* p) {
    Pack<V> r;
    if constexpr (V == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        r.v[0] = q.x; r.v[1] = q.y; r.v[2] = q.z; r.v[3] = q.w;
    } else {
        r.v[0] = *p;
    }
    return r;
}
template <int V>
__device__ __forceinline__ void store_pack(float* p, const Pack<V>& r) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    else *p = r.v[0];
}
template <int V>
__device__ __forceinline__ Pack<V> zero_pack() {
    Pack<V> r;
#pragma unroll
    for (int i = 0; i < V; ++i) r.v[i] = 0.0f;
    return r;
}

// What one item reads at one position.
template <int V>
struct RecurrenceItem {
    Pack<V> c, b, h_old, sel, pre, post;
    int cell;      // -1 on a padded slot: its values never enter (a select, not a product with a mask)
    bool cut;
};

struct RecurrenceArgs {
    const float *c, *b, *h_old, *pre, *post, *sel;
    const int64_t* cells;
    const uint8_t *valid, *reset;
    float *dc, *db;
    int T, K, d, N;
    bool has_pre, has_post, has_sel;
};

template <int V>
__device__ __forceinline__ RecurrenceItem<V> recurrence_fetch(const RecurrenceArgs& g, int row, int t, int k, int x) {
    RecurrenceItem<V> it;
    const int64_t rt = static_cast<int64_t>(row) * g.T + t, slot = rt * g.K + k, at = slot * g.d + x;
    it.cell = g.valid[slot] ? static_cast<int>(g.cells[slot]) : -1;
    it.cut = g.reset[rt] != 0;
    it.c = load_pack<V>(g.c + at);
    it.b = load_pack<V>(g.b + at);
    it.h_old = load_pack<V>(g.h_old + at);
    it.sel = g.has_sel ? load_pack<V>(g.sel + at) : zero_pack<V>();
    it.pre = g.has_pre ? load_pack<V>(g.pre + rt * g.d + x) : zero_pack<V>();
    it.post = g.has_post ? load_pack<V>(g.post + rt * g.d + x) : zero_pack<V>();
    return it;
}

// One row's sweep when there are more items than threads (K d / V > blockDim.x): the items are taken in
// rounds, R stays in shared memory (row N of A) and a position costs two barriers.
template <int V>
__device__ void recurrence_row_rounds(const RecurrenceArgs& g, float* A, int row, bool carry) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int per_slot = g.d / V, items = g.K * per_slot;
    const float n_f = static_cast<float>(g.N);
    float* R = A + static_cast<int64_t>(g.N) * g.d;
    for (int t = g.T - 1; t >= 0; --t) {
        const int64_t rt = static_cast<int64_t>(row) * g.T + t;
        for (int item = tid; item < items; item += nt) {
            const int k = item / per_slot, x = (item - k * per_slot) * V;
            const RecurrenceItem<V> it = recurrence_fetch<V>(g, row, t, k, x);
            Pack<V> dcv = zero_pack<V>(), dbv = zero_pack<V>();
            if (it.cell >= 0) {
                float* a = A + static_cast<int64_t>(it.cell) * g.d + x;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float carried = a[i] + it.sel.v[i];
                    const float share = (R[x + i] + it.post.v[i]) / n_f;
                    const float grad = carried + share;
                    dcv.v[i] = it.b.v[i] * grad;
                    dbv.v[i] = (it.c.v[i] - it.h_old.v[i]) * grad;
                    a[i] = (1.0f - it.b.v[i]) * carried - it.b.v[i] * share;
                }
            }
            const int64_t at = (rt * g.K + k) * g.d + x;
            store_pack<V>(g.dc + at, dcv);
            store_pack<V>(g.db + at, dbv);
        }
        __syncthreads();   // every item has read R; the cells' new values are in place
        const bool clear = g.reset[rt] != 0 && !(carry && t == 0);
        for (int x = tid; x < g.d; x += nt) {
            float r = R[x];
            if (g.has_post) r += g.post[rt * g.d + x];
            if (g.has_pre) r += g.pre[rt * g.d + x];
            R[x] = clear ? 0.0f : r;
        }
        if (clear)
            for (int e = tid; e < g.N * g.d; e += nt) A[e] = 0.0f;
        __syncthreads();
    }
}

// The same sweep with an item per thread, R in registers, the next position's record in flight and one
// barrier a position. Requires K d / V <= blockDim.x.
template <int V>
__device__ void recurrence_row_fast(const RecurrenceArgs& g, float* A, int row, bool carry, Pack<V> R) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int per_slot = g.d / V, items = g.K * per_slot;
    const bool mine = tid < items;
    const int k = mine ? tid / per_slot : 0, x = mine ? (tid - k * per_slot) * V : 0;
    const float n_f = static_cast<float>(g.N);
    RecurrenceItem<V> now{};
    if (mine) now = recurrence_fetch<V>(g, row, g.T - 1, k, x);
    for (int t = g.T - 1; t >= 0; --t) {
        RecurrenceItem<V> next{};
        if (mine && t > 0) next = recurrence_fetch<V>(g, row, t - 1, k, x);   // in flight under this position
        const bool cut = g.reset[static_cast<int64_t>(row) * g.T + t] != 0;      // the same for every thread
        if (mine) {
            Pack<V> dcv = zero_pack<V>(), dbv = zero_pack<V>();
#pragma unroll
            for (int i = 0; i < V; ++i) R.v[i] += now.post.v[i];
            if (now.cell >= 0) {
                float* a = A + static_cast<int64_t>(now.cell) * g.d + x;
                const Pack<V> held = load_pack<V>(a);
                Pack<V> left;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float carried = held.v[i] + now.sel.v[i];
                    const float share = R.v[i] / n_f;
                    const float grad = carried + share;
                    dcv.v[i] = now.b.v[i] * grad;
                    dbv.v[i] = (now.c.v[i] - now.h_old.v[i]) * grad;
                    left.v[i] = (1.0f - now.b.v[i]) * carried - now.b.v[i] * share;
                }
                store_pack<V>(a, left);
            }
            const int64_t at = ((static_cast<int64_t>(row) * g.T + t) * g.K + k) * g.d + x;
            store_pack<V>(g.dc + at, dcv);
            store_pack<V>(g.db + at, dbv);
#pragma unroll
            for (int i = 0; i < V; ++i) R.v[i] += now.pre.v[i];
        }
        const bool clear = cut && !(carry && t == 0);
        if (clear) {
            __syncthreads();   // the position's writes to A are over
            for (int e = tid; e < g.N * g.d; e += nt) A[e] = 0.0f;
            R = zero_pack<V>();
        }
        __syncthreads();       // the one barrier of a position: a cell may change hands at the next
        now = next;
    }
    // R of the row's columns, for the carry: slot 0's items hold one copy of every column group
    if (mine && k == 0) store_pack<V>(A + static_cast<int64_t>(g.N) * g.d + x, R);
    __syncthreads();
}

template <int V>
__device__ void recurrence_run(const HsnWinArgs& a, float* A) {
    RecurrenceArgs g;
    g.T = a.i[1]; g.K = a.i[2]; g.d = a.i[3]; g.N = a.i[4];
    g.has_pre = a.i[5] != 0; g.has_post = a.i[6] != 0; g.has_sel = a.i[7] != 0;
    const bool carry = a.i[8] != 0;
    g.c = static_cast<const float*>(a.p[0]);
    g.b = static_cast<const float*>(a.p[1]);
    g.h_old = static_cast<const float*>(a.p[2]);
    g.cells = static_cast<const int64_t*>(a.p[3]);
    g.valid = static_cast<const uint8_t*>(a.p[4]);
    g.reset = static_cast<const uint8_t*>(a.p[5]);
    g.pre = static_cast<const float*>(a.p[6]);
    g.post = static_cast<const float*>(a.p[7]);
    g.sel = static_cast<const float*>(a.p[8]);
    g.dc = static_cast<float*>(a.p[9]);
    g.db = static_cast<float*>(a.p[10]);
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int64_t Nd = static_cast<int64_t>(g.N) * g.d;
    float* R = A + Nd;
    float* A_io = carry ? static_cast<float*>(a.p[11]) + static_cast<int64_t>(row) * Nd : nullptr;
    float* R_io = carry ? static_cast<float*>(a.p[12]) + static_cast<int64_t>(row) * g.d : nullptr;
    if (carry) {
        block_copy_f32(A, A_io, static_cast<int>(Nd));
        for (int x = tid; x < g.d; x += nt) R[x] = R_io[x];
    } else {
        for (int e = tid; e < Nd + g.d; e += nt) A[e] = 0.0f;
    }
    __syncthreads();
    const int items = g.K * (g.d / V);
    if (items <= nt) {
        Pack<V> mineR = zero_pack<V>();
        if (tid < items) mineR = load_pack<V>(R + (tid % (g.d / V)) * V);
        __syncthreads();
        recurrence_row_fast<V>(g, A, row, carry, mineR);
    } else {
        recurrence_row_rounds<V>(g, A, row, carry);
    }
    if (carry) {
        const bool cut = g.reset[static_cast<int64_t>(row) * g.T] != 0;
        for (int e = tid; e < Nd; e += nt) A_io[e] = cut ? 0.0f : A[e];
        for (int x = tid; x < g.d; x += nt) R_io[x] = cut ? 0.0f : R[x];
    }
}

}  // namespace

extern "C" __global__ void hsn_win_recurrence(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    float* A = reinterpret_cast<float*>(dyn);
    // 16-byte items when every row of the record and of A starts on a 16-byte boundary
    bool wide = (a.i[3] & 3) == 0;
    for (int s : {0, 1, 2, 9, 10}) wide = wide && (reinterpret_cast<uintptr_t>(a.p[s]) & 15) == 0;
    if (a.i[5]) wide = wide && (reinterpret_cast<uintptr_t>(a.p[6]) & 15) == 0;
    if (a.i[6]) wide = wide && (reinterpret_cast<uintptr_t>(a.p[7]) & 15) == 0;
    if (a.i[7]) wide = wide && (reinterpret_cast<uintptr_t>(a.p[8]) & 15) == 0;
    if (wide) recurrence_run<4>(a, A);
    else recurrence_run<1>(a, A);
}

// ------------------------------------------------------------------------------------------------
// hsn_win_recurrence_dense: the recurrence of the rows that ran the dense round (every cell is
// written, q' = mean(h') does not read q; reference: python/hsn/train/split.py:177-209).
//   p: 0 c, 1 b, 2 h_old [B',T,N,d]; 3 reset [B',T] u8; 4 d_q_pre, 5 d_q_post [B',T,d];
//      6 dc, 7 db [B',T,N,d].   i: 0 B', 1 T, 2 N, 3 d, 4 has_pre, 5 has_post.
// Dynamic shared memory: (N + 1) d words (the reference's launch size; A lives there).
//
// Every element of the state is written at every position and reads only itself and the summary's
// cotangent of its column, which here is stateless: before position t it equals d_q_post[t] plus,
// when position t+1 exists and does not reset, d_q_pre[t+1]. So an element's whole history belongs to
// one thread, no value crosses threads and the sweep needs no barrier at all; each thread walks its
// elements (16 bytes at a time when d is a multiple of 4) with the next position's loads in flight.
// ------------------------------------------------------------------------------------------------
namespace {

template <int V>
__device__ void dense_run(const HsnWinArgs& a, float* A) {
    const int T = a.i[1], N = a.i[2], d = a.i[3];
    const bool has_pre = a.i[4] != 0, has_post = a.i[5] != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const float* c = static_cast<const float*>(a.p[0]);
    const float* b = static_cast<const float*>(a.p[1]);
    const float* h_old = static_cast<const float*>(a.p[2]);
    const uint8_t* reset = static_cast<const uint8_t*>(a.p[3]);
    const float* pre = static_cast<const float*>(a.p[4]);
    const float* post = static_cast<const float*>(a.p[5]);
    float* dc = static_cast<float*>(a.p[6]);
    float* db = static_cast<float*>(a.p[7]);
    const int64_t Nd = static_cast<int64_t>(N) * d;
    const int groups = static_cast<int>(Nd / V);
    const float n_f = static_cast<float>(N);
    for (int e = tid; e < groups; e += nt) store_pack<V>(A + static_cast<int64_t>(e) * V, zero_pack<V>());
    // (no barrier: a thread reads back only what it wrote itself)
    for (int t = T - 1; t >= 0; --t) {
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        const bool cut = reset[rt] != 0;
        const bool from_next = has_pre && t + 1 < T && reset[rt + 1] == 0;
        for (int e = tid; e < groups; e += nt) {
            const int64_t at = static_cast<int64_t>(e) * V;
            const int x = static_cast<int>(at % d);
            const int64_t o = rt * Nd + at;
            const Pack<V> cv = load_pack<V>(c + o), bv = load_pack<V>(b + o), hv = load_pack<V>(h_old + o);
            const Pack<V> po = has_post ? load_pack<V>(post + rt * d + x) : zero_pack<V>();
            const Pack<V> pr = from_next ? load_pack<V>(pre + (rt + 1) * d + x) : zero_pack<V>();
            const Pack<V> held = load_pack<V>(A + at);
            Pack<V> dcv, dbv, left;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float grad = held.v[i] + (pr.v[i] + po.v[i]) / n_f;
                dcv.v[i] = bv.v[i] * grad;
                dbv.v[i] = (cv.v[i] - hv.v[i]) * grad;
                left.v[i] = cut ? 0.0f : (1.0f - bv.v[i]) * grad;
            }
            store_pack<V>(dc + o, dcv);
            store_pack<V>(db + o, dbv);
            store_pack<V>(A + at, left);
        }
    }
}

}  // namespace

extern "C" __global__ void hsn_win_recurrence_dense(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    float* A = reinterpret_cast<float*>(dyn);
    bool wide = (a.i[3] & 3) == 0;
    for (int s : {0, 1, 2, 6, 7}) wide = wide && (reinterpret_cast<uintptr_t>(a.p[s]) & 15) == 0;
    if (a.i[4]) wide = wide && (reinterpret_cast<uintptr_t>(a.p[4]) & 15) == 0;
    if (a.i[5]) wide = wide && (reinterpret_cast<uintptr_t>(a.p[5]) & 15) == 0;
    if (wide) dense_run<4>(a, A);
    else dense_run<1>(a, A);
}
