// The three glue kernels of the reverse sweep that are launched by name, once per position,
// between the sweep's two products: hsn_win_back_head, hsn_win_back_mid, hsn_win_back_tail.
// Launch descriptor and p[] / i[] / f[] slot meanings are the reference's (reference
// kernels/cuda/hsn_window.cu:1014-1427 and its callers python/hsn/kernels/window.py:1181-1290);
// the contract of each kernel is the PyTorch step of the same name in
// python/hsn/train/state_sweep.py (head_reference :441, middle_reference :487, tail_reference
// :497). The implementations are this library's own: one thread block per batch row, one warp
// per slot, fp32 state, every reduction in a fixed order, no atomics, products and sums rounded
// separately where the contract rounds them separately.
//
// Buffers (B rows, T positions, K slots of which the first F are fixed, N cells, width d, H hidden
// columns, M units; "operand" buffers hold fp32 or bf16 as flagged):
//   A [B,N,d], R [B,d] f32                 the state's cotangent, in and out
//   c, b, h_old, y, gate_pre, mv, d_h_sel, dc, db [B,T,K,d] f32; rms [B,T,K] f32
//   hidden [B,T,K,H] operand; cells, units [B,T,K] i64; valid [B,T,K] u8; reset [B,T] u8
//   d_q_pre, d_q_post [B,T,d] f32; d_h_fast [B,T,max(n_read,1),d] f32
//   op1 [B(K-F), M d], op2 [B(K-F), M H + d], op1_fast [F,B,d], op2_fast [F,B,H+d] operands
//   act_r [B(K-F), H], act_f [F,B,H], dv_r [B(K-F), 2d], dv_f [F,B,2d] operands (the products)
//   sigma [B,K] f32; out_tgt [N,d_out] i32 (-1: padding); out_w [N,d_out] f32
#include "../../include/hsn_window_b200.h"
#include "common.cuh"

using namespace hsnw;

namespace {
__device__ __forceinline__ float operand_load(const void* p, int64_t index, bool half) {
    return half ? bf16_value(static_cast<const uint16_t*>(p)[index]) : static_cast<const float*>(p)[index];
}
__device__ __forceinline__ void operand_store(void* p, int64_t index, bool half, float v) {
    if (half) static_cast<uint16_t*>(p)[index] = bf16_bits(v);
    else static_cast<float*>(p)[index] = v;
}

// A routed slot's values into its unit's block of its operand row: the block the later position
// used is cleared first (the sweep walks backward, so "later" was written one launch ago).
__device__ __forceinline__ void block_store(void* operand, int64_t row_base, int width, int before, int now,
                                            int x, bool half, float v) {
    if (before >= 0 && before != now) operand_store(operand, row_base + static_cast<int64_t>(before) * width + x, half, 0.0f);
    operand_store(operand, row_base + static_cast<int64_t>(now) * width + x, half, v);
}

__device__ __forceinline__ float activation_grad(int code, float x) {
    switch (code) {
        case 0: return gelu_erf_grad(x);
        case 1: return x > 0.0f ? 1.0f : 0.0f;
        case 2: {
            const float s = sigmoid_f(x);
            return s * (1.0f + x * (1.0f - s));
        }
        default: {
            const float th = tanhf(x);
            return 1.0f - th * th;
        }
    }
}
}  // namespace

// ------------------------------------------------------------------------------------------------
// hsn_win_back_head: the recurrence's step of position t and what the first product reads.
//   p: 0 A, 1 R, 2 c, 3 b, 4 h_old, 5 y, 6 cells, 7 units, 8 valid, 9 d_q_post, 10 d_h_sel,
//      11 d_h_fast, 12 cand_gain [d], 13 gate_pre, 14 gate_bias [d], 15 dc, 16 db, 17 op1,
//      18 op1_fast, 19 op2, 20 op2_fast, 21 sigma.
//   i: 0 B, 1 T, 2 K, 3 d, 4 N, 5 M, 6 H, 7 F, 8 t, 9 n_read, 10 candidate norm, 11 bf16 operands.
//   f: 0 the candidate norm's eps.
// Dynamic shared memory: d words. Any multiple of 32 threads.
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_back_head(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    float* share = reinterpret_cast<float*>(dyn);
    const int T = a.i[1], K = a.i[2], d = a.i[3], N = a.i[4], M = a.i[5], H = a.i[6], F = a.i[7], t = a.i[8];
    const int n_read = a.i[9];
    const bool cand_norm = a.i[10] != 0, half = a.i[11] != 0;
    const float eps = a.f[0];
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    const int B = gridDim.x, routed = K - F;
    float* A = static_cast<float*>(a.p[0]) + static_cast<int64_t>(row) * N * d;
    float* R = static_cast<float*>(a.p[1]) + static_cast<int64_t>(row) * d;
    const float* c = static_cast<const float*>(a.p[2]);
    const float* gate = static_cast<const float*>(a.p[3]);
    const float* h_old = static_cast<const float*>(a.p[4]);
    const float* y = static_cast<const float*>(a.p[5]);
    const int64_t* cells = static_cast<const int64_t*>(a.p[6]);
    const int64_t* units = static_cast<const int64_t*>(a.p[7]);
    const uint8_t* valid = static_cast<const uint8_t*>(a.p[8]);
    const float* post = static_cast<const float*>(a.p[9]);
    const float* sel = static_cast<const float*>(a.p[10]);
    const float* fast = static_cast<const float*>(a.p[11]);
    const float* cand_gain = static_cast<const float*>(a.p[12]);
    const float* gate_pre = static_cast<const float*>(a.p[13]);
    const float* gate_bias = static_cast<const float*>(a.p[14]);
    float* dc = static_cast<float*>(a.p[15]);
    float* db = static_cast<float*>(a.p[16]);
    float* sigma = static_cast<float*>(a.p[21]);
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    const float n_f = static_cast<float>(N);

    for (int x = tid; x < d; x += nt) {
        const float r = R[x] + post[rt * d + x];
        R[x] = r;
        share[x] = r / n_f;
    }
    const int read_width = n_read > 0 ? n_read : 1;
    for (int e = tid; e < n_read * d; e += nt) A[e] += fast[rt * read_width * d + e];
    __syncthreads();

    for (int k = warp; k < K; k += warps) {
        const int64_t s = rt * K + k;
        const bool ok = valid[s] != 0;
        const int n = ok ? static_cast<int>(cells[s]) : 0;
        const int unit_now = static_cast<int>(units[s]);
        const int unit_before = t + 1 < T ? static_cast<int>(units[s + K]) : -1;
        // pass 1: the recurrence, with the candidate norm's two means when it is on
        float sum_yy = 0.0f, sum_ys = 0.0f;
        for (int x = lane; x < d; x += 32) {
            const int64_t o = s * d + x;
            float dcv = 0.0f, dbv = 0.0f;
            if (ok) {
                const float carried = A[n * d + x] + sel[o];
                const float sh = share[x];
                const float g = carried + sh;
                const float bv = gate[o];
                dcv = __fmul_rn(bv, g);
                dbv = __fmul_rn(c[o] - h_old[o], g);
                A[n * d + x] = __fsub_rn(__fmul_rn(1.0f - bv, carried), __fmul_rn(bv, sh));
                if (cand_norm) {
                    const float cv = c[o], yv = y[o];
                    const float dz = __fmul_rn(dcv, 1.0f - __fmul_rn(cv, cv));
                    sum_yy += yv * yv;
                    sum_ys += yv * __fmul_rn(cand_gain[x], dz);
                }
            }
            dc[o] = dcv;
            db[o] = dbv;
        }
        float rho = 0.0f, mean_ys = 0.0f;
        if (cand_norm) {
            sum_yy = warp_sum(sum_yy);
            sum_ys = warp_sum(sum_ys);
            rho = rsqrtf(sum_yy / static_cast<float>(d) + eps);
            mean_ys = sum_ys / static_cast<float>(d);
        }
        // pass 2: the operands of the first product and the gate's part of the second's
        float sig = 0.0f;
        for (int x = lane; x < d; x += 32) {
            const int64_t o = s * d + x;
            float d_unit = 0.0f, d_gate = 0.0f;
            if (ok) {
                const float cv = c[o], bv = gate[o];
                float dz = __fmul_rn(dc[o], 1.0f - __fmul_rn(cv, cv));
                if (cand_norm) {
                    const float scaled = __fmul_rn(cand_gain[x], dz);
                    dz = __fsub_rn(__fmul_rn(rho, scaled), __fmul_rn(__fmul_rn(rho * rho * rho, y[o]), mean_ys));
                }
                d_unit = dz;
                d_gate = __fmul_rn(__fmul_rn(db[o], bv), 1.0f - bv);
                sig += d_gate * (gate_pre[o] - gate_bias[x]);
            }
            if (k >= F) {
                const int64_t line = static_cast<int64_t>(row) * routed + (k - F);
                block_store(a.p[17], line * M * d, d, unit_before, unit_now, x, half, d_unit);
                operand_store(a.p[19], line * (static_cast<int64_t>(M) * H + d) + static_cast<int64_t>(M) * H + x, half, d_gate);
            } else {
                const int64_t line = static_cast<int64_t>(k) * B + row;
                operand_store(a.p[18], line * d + x, half, d_unit);
                operand_store(a.p[20], line * (H + d) + H + x, half, d_gate);
            }
        }
        sig = warp_sum(sig);
        if (lane == 0) sigma[static_cast<int64_t>(row) * K + k] = sig;
    }
}

// ------------------------------------------------------------------------------------------------
// hsn_win_back_mid: through the activation, between the two products.
//   p: 0 act_r, 1 act_f, 2 hidden, 3 units, 4 valid, 5 b1 [M,H] f32, 6 op2, 7 op2_fast, 8 sigma.
//   i: 0 B, 1 T, 2 K, 3 d, 4 M, 5 H, 6 F, 7 t, 8 bf16 operands, 9 bf16 hidden, 10 activation
//      (0 gelu, 1 relu, 2 silu, 3 tanh).
// No dynamic shared memory. Any multiple of 32 threads.
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_back_mid(HsnWinArgs a) {
    const int T = a.i[1], K = a.i[2], d = a.i[3], M = a.i[4], H = a.i[5], F = a.i[6], t = a.i[7];
    const bool half = a.i[8] != 0, half_hidden = a.i[9] != 0;
    const int code = a.i[10];
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    const int B = gridDim.x, routed = K - F;
    const int64_t* units = static_cast<const int64_t*>(a.p[3]);
    const uint8_t* valid = static_cast<const uint8_t*>(a.p[4]);
    const float* b1 = static_cast<const float*>(a.p[5]);
    float* sigma = static_cast<float*>(a.p[8]);
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    for (int k = warp; k < K; k += warps) {
        const int64_t s = rt * K + k;
        const bool ok = valid[s] != 0;
        const int unit_now = static_cast<int>(units[s]);
        const int unit_before = t + 1 < T ? static_cast<int>(units[s + K]) : -1;
        const bool is_routed = k >= F;
        const int64_t line = is_routed ? static_cast<int64_t>(row) * routed + (k - F) : static_cast<int64_t>(k) * B + row;
        const void* act = is_routed ? a.p[0] : a.p[1];
        float sig = 0.0f;
        for (int x = lane; x < H; x += 32) {
            float d_hid = 0.0f;
            if (ok) {
                const float hv = operand_load(a.p[2], s * H + x, half_hidden);
                d_hid = __fmul_rn(operand_load(act, line * H + x, half), activation_grad(code, hv));
                sig += d_hid * (hv - b1[static_cast<int64_t>(unit_now) * H + x]);
            }
            if (is_routed) block_store(a.p[6], line * (static_cast<int64_t>(M) * H + d), H, unit_before, unit_now, x, half, d_hid);
            else operand_store(a.p[7], line * (H + d) + x, half, d_hid);
        }
        sig = warp_sum(sig);
        if (lane == 0) sigma[static_cast<int64_t>(row) * K + k] += sig;
    }
}

// ------------------------------------------------------------------------------------------------
// hsn_win_back_tail: the second product's result through the cell norm into the state's
// cotangent, the messages' part along the graph, the reset.
//   p: 0 A, 1 R, 2 dv_r, 3 dv_f, 4 sigma, 5 rms, 6 h_old, 7 mv, 8 cells, 9 valid, 10 out_tgt,
//      11 out_w, 12 d_q_pre, 13 reset.
//   i: 0 B, 1 T, 2 K, 3 d, 4 N, 5 F, 6 t, 7 d_out, 8 cell norm, 9 in_dim (the width the cell
//      norm averages over), 10 bf16 products.
// Dynamic shared memory: 2 K d + N words. Any multiple of 32 threads.
// ------------------------------------------------------------------------------------------------
extern "C" __global__ void hsn_win_back_tail(HsnWinArgs a) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const int T = a.i[1], K = a.i[2], d = a.i[3], N = a.i[4], F = a.i[5], t = a.i[6], d_out = a.i[7];
    const bool cell_norm = a.i[8] != 0, half = a.i[10] != 0;
    const float in_dim = static_cast<float>(a.i[9]);
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    const int B = gridDim.x, routed = K - F;
    float* ds = reinterpret_cast<float*>(dyn);          // [K][2d]: [dh ; what a message's source receives]
    int* slot_of = reinterpret_cast<int*>(ds + 2 * K * d);  // [N]: the slot that selected a cell, or -1
    float* A = static_cast<float*>(a.p[0]) + static_cast<int64_t>(row) * N * d;
    float* R = static_cast<float*>(a.p[1]) + static_cast<int64_t>(row) * d;
    const float* sigma = static_cast<const float*>(a.p[4]);
    const float* rms = static_cast<const float*>(a.p[5]);
    const float* h_old = static_cast<const float*>(a.p[6]);
    const float* mv = static_cast<const float*>(a.p[7]);
    const int64_t* cells = static_cast<const int64_t*>(a.p[8]);
    const uint8_t* valid = static_cast<const uint8_t*>(a.p[9]);
    const int32_t* out_tgt = static_cast<const int32_t*>(a.p[10]);
    const float* out_w = static_cast<const float*>(a.p[11]);
    const float* pre = static_cast<const float*>(a.p[12]);
    const uint8_t* reset = static_cast<const uint8_t*>(a.p[13]);
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    const bool cut = reset[rt] != 0;

    for (int n = tid; n < N; n += nt) slot_of[n] = -1;
    __syncthreads();
    for (int k = warp; k < K; k += warps) {
        const int64_t s = rt * K + k;
        const bool ok = valid[s] != 0;
        const bool is_routed = k >= F;
        const int64_t line = is_routed ? static_cast<int64_t>(row) * routed + (k - F) : static_cast<int64_t>(k) * B + row;
        const void* prod = is_routed ? a.p[2] : a.p[3];
        float r = 1.0f, back = 0.0f;
        if (cell_norm && ok) {
            r = rms[s];
            back = __fmul_rn(__fmul_rn(r, r) / in_dim, sigma[static_cast<int64_t>(row) * K + k]);
        }
        for (int x = lane; x < 2 * d; x += 32) {
            float v = 0.0f;
            if (ok) {
                v = operand_load(prod, line * 2 * d + x, half);
                if (cell_norm) {
                    const float state = x < d ? h_old[s * d + x] : mv[s * d + (x - d)];
                    v = __fsub_rn(__fmul_rn(r, v), __fmul_rn(back, state));
                }
            }
            ds[k * 2 * d + x] = v;
        }
        if (ok && lane == 0) slot_of[static_cast<int>(cells[s])] = k;
    }
    __syncthreads();
    for (int e = tid; e < N * d; e += nt) {
        const int n = e / d, x = e - n * d;
        float v = 0.0f;
        if (!cut) {
            v = A[e];
            const int own = slot_of[n];
            if (own >= 0) v += ds[own * 2 * d + x];
            for (int j = 0; j < d_out; ++j) {  // in out_tgt's order: by target cell, then by its slot
                const int target = out_tgt[n * d_out + j];
                if (target < 0) continue;
                const int slot = slot_of[target];
                if (slot >= 0) v = __fadd_rn(v, __fmul_rn(out_w[n * d_out + j], ds[slot * 2 * d + d + x]));
            }
        }
        A[e] = v;
    }
    for (int x = tid; x < d; x += nt) R[x] = cut ? 0.0f : R[x] + pre[rt * d + x];
}
