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
// hsn_win_recurrence: the full-cut backward state recurrence of a window, t = T-1 .. 0, with the
// row's cotangents A [N,d] and R [d] in shared memory.
//   p: 0 c, 1 b, 2 h_old [B,T,K,d] f32; 3 cells [B,T,K] i64; 4 valid [B,T,K] u8; 5 reset [B,T] u8;
//      6 d_q_pre, 7 d_q_post [B,T,d], 8 d_h_sel [B,T,K,d] (read when flagged); 9 dc, 10 db out.
//      This library adds (zero in the reference's calls): 11 A [B,N,d], 12 R [B,d] in/out.
//   i: 0 B, 1 T, 2 K, 3 d, 4 N, 5 has_pre, 6 has_post, 7 has_sel, 8 carry: start from p11/p12 and
//      store the final cotangents there (zeroed on rows whose position 0 resets).
// Dynamic shared memory: (N + 1) d words (up to 227 KB after hsnw_prepare).
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_recurrence(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const int T = a.i[1], K = a.i[2], d = a.i[3], N = a.i[4];
    const bool has_pre = a.i[5] != 0, has_post = a.i[6] != 0, has_sel = a.i[7] != 0, carry = a.i[8] != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const float* c = static_cast<const float*>(a.p[0]);
    const float* b = static_cast<const float*>(a.p[1]);
    const float* h_old = static_cast<const float*>(a.p[2]);
    const int64_t* cells = static_cast<const int64_t*>(a.p[3]);
    const uint8_t* valid = static_cast<const uint8_t*>(a.p[4]);
    const uint8_t* reset = static_cast<const uint8_t*>(a.p[5]);
    const float* pre = static_cast<const float*>(a.p[6]);
    const float* post = static_cast<const float*>(a.p[7]);
    const float* sel = static_cast<const float*>(a.p[8]);
    float* dc = static_cast<float*>(a.p[9]);
    float* db = static_cast<float*>(a.p[10]);
    float* A = reinterpret_cast<float*>(dyn);
    float* R = A + static_cast<int64_t>(N) * d;
    if (carry) {
        block_copy_f32(A, static_cast<const float*>(a.p[11]) + static_cast<int64_t>(row) * N * d, N * d);
        for (int x = tid; x < d; x += nt) R[x] = static_cast<const float*>(a.p[12])[static_cast<int64_t>(row) * d + x];
    } else {
        for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
        for (int x = tid; x < d; x += nt) R[x] = 0.0f;
    }
    __syncthreads();
    const float n_f = static_cast<float>(N);
    const int KD = K * d;
    for (int t = T - 1; t >= 0; --t) {
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        if (has_post) {
            for (int x = tid; x < d; x += nt) R[x] += post[rt * d + x];
            __syncthreads();
        }
        for (int e = tid; e < KD; e += nt) {
            const int k = e / d, x = e - k * d;
            const int64_t s = rt * K + k, o = s * d + x;
            float dcv = 0.0f, dbv = 0.0f;
            if (valid[s]) {  // a padded slot's values never enter: a select, not a product with a mask
                const int n = static_cast<int>(cells[s]);
                float carried = A[n * d + x];
                if (has_sel) carried += sel[o];
                const float share = R[x] / n_f;
                const float g = carried + share;
                const float gate = b[o];
                dcv = gate * g;
                dbv = (c[o] - h_old[o]) * g;
                A[n * d + x] = (1.0f - gate) * carried - gate * share;
            }
            dc[o] = dcv;
            db[o] = dbv;
        }
        __syncthreads();
        const bool cut = reset[rt] != 0;
        if (has_pre)
            for (int x = tid; x < d; x += nt) R[x] += pre[rt * d + x];
        if (cut && !(carry && t == 0)) {
            for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
            for (int x = tid; x < d; x += nt) R[x] = 0.0f;
        }
        __syncthreads();
    }
    if (carry) {
        const bool cut = reset[static_cast<int64_t>(row) * T] != 0;
        float* A_out = static_cast<float*>(a.p[11]) + static_cast<int64_t>(row) * N * d;
        float* R_out = static_cast<float*>(a.p[12]) + static_cast<int64_t>(row) * d;
        for (int e = tid; e < N * d; e += nt) A_out[e] = cut ? 0.0f : A[e];
        for (int x = tid; x < d; x += nt) R_out[x] = cut ? 0.0f : R[x];
    }
}

// ------------------------------------------------------------------------------------------------
// hsn_win_recurrence_dense: the recurrence of the rows that ran the dense round (every cell is
// written, q' = mean(h') does not read q).
//   p: 0 c, 1 b, 2 h_old [B',T,N,d]; 3 reset [B',T] u8; 4 d_q_pre, 5 d_q_post [B',T,d];
//      6 dc, 7 db [B',T,N,d].   i: 0 B', 1 T, 2 N, 3 d, 4 has_pre, 5 has_post.
// Dynamic shared memory: (N + 1) d words.
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_recurrence_dense(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
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
    float* A = reinterpret_cast<float*>(dyn);
    float* R = A + static_cast<int64_t>(N) * d;
    for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
    for (int x = tid; x < d; x += nt) R[x] = 0.0f;
    __syncthreads();
    const float n_f = static_cast<float>(N);
    for (int t = T - 1; t >= 0; --t) {
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        if (has_post) {
            for (int x = tid; x < d; x += nt) R[x] += post[rt * d + x];
            __syncthreads();
        }
        for (int e = tid; e < N * d; e += nt) {
            const int64_t o = rt * N * d + e;
            const float g = A[e] + R[e % d] / n_f;
            const float gate = b[o];
            dc[o] = gate * g;
            db[o] = (c[o] - h_old[o]) * g;
            A[e] = (1.0f - gate) * g;
        }
        __syncthreads();
        const bool cut = reset[rt] != 0;
        for (int x = tid; x < d; x += nt) R[x] = (cut || !has_pre) ? 0.0f : pre[rt * d + x];
        if (cut)
            for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
        __syncthreads();
    }
}
