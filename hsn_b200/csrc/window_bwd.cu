// The reverse sweep of a window (the backward state recurrence) as batch-synchronous phases,
// t = T-1 .. 0; the state's cotangent A [B,N,d], R [B,d] lives in global memory (L2-resident at
// the training shapes), so one design covers every N and d and hands the cotangent from one
// window to the one before it.
//
//   head  one block per row: R += D_t; the gated carry (dc, db; A[cell] = (1-b) carried - b R/N);
//         with the state gradient also the candidate's backward (tanh, candidate norm, W_out
//         transposed) and the gate's (sigmoid), which leave d_unit, dg and the gate's part of the
//         cell norm's inner product for the next phase.
//   mid   weight-stationary: a block holds a 64-column slice of ONE unit's second layer and of the
//         state rows of its first layer and serves the pairs routed to that unit: the transposed
//         second layer, the activation's derivative, the transposed first layer on the 2d state
//         columns only, and the unit's part of the norm's inner product, as partial sums per slice.
//   tail  one block per row: reduce the partials in slice order, the gate's transposed linear, the
//         cell norm's backward, dh into A[cell], V transposed and the scatter of the message
//         cotangent into the sources (edge by edge in slot order: a fixed order, no atomics),
//         R += P_t, and the zeroing of the rows that reset at t.
//
// Follows state_gradient_backward / cell_state_vjp (reference python/hsn/train/state_gradient.py:
// 288-485); with full_cut only the head runs: recurrence_backward (python/hsn/train/split.py:128-174).
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "host_util.h"
#include "stage.cuh"
#include "umma.cuh"

#include <mutex>
#include <stdio.h>

using namespace hsnw;

// Optional phase timestamps for tuning (compiled in with -DHSNW_TRACE): event i of block b of the
// tail+head kernel lands at g_bwd_trace[b * 32 + i] (nanoseconds of the global timer).
#ifdef HSNW_TRACE
__device__ unsigned long long g_bwd_trace[64 * 32];
#define BW_MARK(i)                                                              \
    do {                                                                        \
        if (threadIdx.x == 0 && blockIdx.x < 64) {                              \
            unsigned long long now;                                             \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));             \
            g_bwd_trace[blockIdx.x * 32 + (i)] = now;                           \
        }                                                                       \
    } while (0)
extern "C" int hsnw_trace_read_bwd(unsigned long long* host) {
    return static_cast<int>(cudaMemcpyFromSymbol(host, g_bwd_trace, sizeof(g_bwd_trace)));
}
#else
#define BW_MARK(i) do { } while (0)
#endif

namespace {

constexpr int kUS = 32;          // columns of a unit slice
constexpr int kPB = 32;          // pairs a block multiplies at a time
constexpr int kPairTile = 256;

struct BwdCtx {
    HsnwModel m;
    HsnwBackward io;
    int nU;           // slices of a unit's hidden layer; slice nU of part_dv is the gate's
    float* d_unit;    // [P, d]   W_out^T dy
    float* dg;        // [P, d]   the gate's pre-activation cotangent
    float* sig_gate;  // [P]      <gate_pre - b_g, dg>
    float* part_dv;   // [nU + 1, P, 2d]
    float* part_sig;  // [nU, P]
    int* pair_unit;   // [P]  -1 on padded slots
    int* status;      // set to 1 by a bounded wait that ran out (the head of the caller's scratch; null with full_cut and no scratch)
};

// ------------------------------------------------------------------------------------------------
// head. Shared (dynamic): Rs [d], cell_of [K], rho [K], dot [K], dzs [K d], ysv [K d], sgs [K d],
// wo [d (d+1)].
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void head_phase(const BwdCtx& c, int t, unsigned char* dyn) {
    const int N = c.m.N, d = c.m.d, K = c.m.K, T = c.io.T;
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const bool full = c.io.full_cut != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    float* Rs = reinterpret_cast<float*>(dyn);
    int* cell_of = reinterpret_cast<int*>(Rs + d);
    float* rho = reinterpret_cast<float*>(cell_of + K);
    float* dot = rho + K;
    float* dzs = dot + K;         // [K d]  cand_w * dz, then dy
    float* ysv = dzs + K * d;     // [K d]
    float* sgs = ysv + K * d;     // [K d]  dg (gate_pre - b_g)
    float* wo = sgs + K * d;      // [d][d+1]
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    float* A = c.io.A + static_cast<int64_t>(row) * N * d;
    float* R = c.io.R + static_cast<int64_t>(row) * d;
    const int64_t* cells = c.io.cells + rt * K;
    const uint8_t* valid = c.io.valid + rt * K;
    const int64_t o0 = rt * K * d;
    if (!full) {
        for (int e = tid; e < d * d; e += nt) cp_async4(wo + (div_magic(e, dmag)) * (d + 1) + (e - div_magic(e, dmag) * d), c.m.wout_t + e);
        cp_async_commit();   // needed only by the last step of the phase
    }
    for (int x = tid; x < d; x += nt) {
        float r = R[x];
        if (c.io.d_q_post) r += c.io.d_q_post[rt * d + x];
        Rs[x] = r;
    }
    for (int k = tid; k < K; k += nt) cell_of[k] = valid[k] ? static_cast<int>(cells[k]) : -1;
    BW_MARK(8);
    __syncthreads();
    BW_MARK(9);
    const float n_f = static_cast<float>(N);
    for (int e = tid; e < K * d; e += nt) {
        const int k = div_magic(e, dmag), x = e - k * d;
        const int n = cell_of[k];
        float dcv = 0.0f, dbv = 0.0f, dz = 0.0f, dgv = 0.0f, yv = 0.0f, sgv = 0.0f;
        if (n >= 0) {
            float carried = A[static_cast<int64_t>(n) * d + x];
            if (c.io.d_h_sel) carried += c.io.d_h_sel[o0 + e];
            const float share = Rs[x] / n_f;
            const float g = carried + share;
            const float gate = c.io.b[o0 + e], cv = c.io.c[o0 + e];
            dcv = gate * g;
            dbv = (cv - c.io.h_old[o0 + e]) * g;
            A[static_cast<int64_t>(n) * d + x] = (1.0f - gate) * carried - gate * share;
            if (!full) {
                dz = c.m.cand_w[x] * (dcv * (1.0f - cv * cv));
                dgv = dbv * gate * (1.0f - gate);
                yv = c.io.y[o0 + e];
                sgv = dgv * (c.io.gate_pre[o0 + e] - c.m.gate_b[x]);
            }
        }
        c.io.dc[o0 + e] = dcv;
        c.io.db[o0 + e] = dbv;
        if (!full) {
            dzs[e] = dz;
            ysv[e] = yv;
            sgs[e] = sgv;
            c.dg[(static_cast<int64_t>(row) * K + k) * d + x] = dgv;
        }
    }
    if (full) {
        // the plain recurrence ends the position here
        __syncthreads();
        const bool cut = c.io.reset[rt] != 0;
        for (int x = tid; x < d; x += nt) {
            float r = Rs[x];
            if (c.io.d_q_pre) r += c.io.d_q_pre[rt * d + x];
            R[x] = cut ? 0.0f : r;
        }
        if (cut)
            for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
        return;
    }
    for (int x = tid; x < d; x += nt) R[x] = Rs[x];
    __syncthreads();
    BW_MARK(10);
    // per slot: rho = rsqrt(mean(y^2) + eps), dot = mean(y * cand_w * dz), sigma_gate; a warp each
    for (int k = warp; k < K; k += warps) {
        float sq = 0.0f, dt = 0.0f, s = 0.0f;
        for (int x = lane; x < d; x += 32) {
            const float yv = ysv[k * d + x];
            sq += yv * yv;
            dt += yv * dzs[k * d + x];
            s += sgs[k * d + x];
        }
        sq = warp_sum(sq);
        dt = warp_sum(dt);
        s = warp_sum(s);
        if (lane == 0) {
            rho[k] = rsqrtf(sq / static_cast<float>(d) + c.m.cand_eps);
            dot[k] = dt / static_cast<float>(d);
            c.sig_gate[static_cast<int64_t>(row) * K + k] = s;
        }
    }
    __syncthreads();
    // dy = rho (cand_w dz) - rho^3 y mean(y cand_w dz), in place of dzs
    for (int e = tid; e < K * d; e += nt) {
        const int k = div_magic(e, dmag);
        const float r = rho[k];
        dzs[e] = cell_of[k] >= 0 ? r * dzs[e] - r * r * r * ysv[e] * dot[k] : 0.0f;
    }
    BW_MARK(11);
    cp_async_wait_all();
    __syncthreads();
    BW_MARK(12);
    // d_unit = dy W_out (the transposed output projection): y[x] = sum_i F[i] wout_t[i][x]
    const int per = max(1, min(4, K * d / nt));   // slots a thread: a weight is read once for them
    for (int e = tid; e < ((K + per - 1) / per) * d; e += nt) {
        const int k0 = (div_magic(e, dmag)) * per, i = e - (div_magic(e, dmag)) * d;
        float out[4];
        dot4_rows(dzs + k0 * d, d, min(per, K - k0), wo + i * (d + 1), 1, d, out);
        for (int r = 0; r < per && k0 + r < K; ++r) c.d_unit[(static_cast<int64_t>(row) * K + k0 + r) * d + i] = out[r];
    }
    for (int k = tid; k < K; k += nt)
        c.pair_unit[static_cast<int64_t>(row) * K + k] = cell_of[k] >= 0 ? static_cast<int>(c.io.units[rt * K + k]) : -1;
    BW_MARK(13);
}

// ------------------------------------------------------------------------------------------------
// mid: blockIdx.x = (unit j, slice s), blockIdx.y = pair tile; 256 threads, a thread owns a column
// and four pairs. Slices 0 .. nU-1: 32 hidden columns of unit j (second layer transposed, the
// activation's derivative, the norm's inner product, first layer transposed on the state
// columns); slice nU: the gate's transposed linear for unit j's pairs.
// Shared (dynamic): w2 [32][d+1] | gate rows [2d][d+1], w1 [2d][33], du [32][d], dh [32][33], list.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_mid(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int warp_count[8];
    __shared__ int n_list;
    const int d = c.m.d, K = c.m.K, H = c.m.H, in = 4 * c.m.d, two = 2 * c.m.d;
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const int P = c.io.B * K, T = c.io.T;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool bf = c.m.prod_bf16 != 0;  // the products' operands are rounded as on the tensor cores
    const int per_unit = c.nU + 1;
    const int j = blockIdx.x / per_unit, s = blockIdx.x - j * per_unit;
    const bool is_gate = s == c.nU;
    const int c0 = s * kUS;
    const int cols = is_gate ? 0 : min(kUS, H - c0);
    float* du = reinterpret_cast<float*>(dyn);                       // [32][d]
    float* wA = du + kPB * d;                                        // w2 [32][d+1] or gate [2d][d+1]
    float* w1 = wA + (is_gate ? two : kUS) * (d + 1);                // [2d][33]
    float* dh = w1 + two * (kUS + 1);                                // [32][33]
    int* list = reinterpret_cast<int*>(dh + kPB * (kUS + 1));
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
        // the gate's transposed linear on the state columns: gate_pre[x] = sum_i v[i] gate_t[i][x]
        for (int e = tid; e < two * d; e += 256) {
            const int i = div_magic(e, dmag), x = e - i * d;
            wA[i * (d + 1) + x] = c.m.gate_t[static_cast<int64_t>(two + i) * d + x];
        }
        for (int base = 0; base < count; base += kPB) {
            const int nb = min(kPB, count - base);
            __syncthreads();
            for (int e = tid; e < nb * d; e += 256) {
                const int pb = div_magic(e, dmag), x = e - pb * d;
                du[e] = maybe_bf16(c.dg[static_cast<int64_t>(list[base + pb]) * d + x], bf);
            }
            __syncthreads();
            for (int e = tid; e < nb * two; e += 256) {
                const int pb = e / two, i = e - pb * two;
                c.part_dv[(static_cast<int64_t>(c.nU) * P + list[base + pb]) * two + i] =
                    dot4(du + pb * d, 1, wA + i * (d + 1), 1, d);
            }
        }
        return;
    }
    const float* W1 = c.m.w1 + static_cast<int64_t>(j) * in * H;
    const float* W2 = c.m.w2 + static_cast<int64_t>(j) * H * d;
    for (int e = tid; e < kUS * d; e += 256) {
        const int cc = div_magic(e, dmag), x = e - cc * d;
        wA[cc * (d + 1) + x] = cc < cols ? W2[static_cast<int64_t>(c0 + cc) * d + x] : 0.0f;
    }
    for (int e = tid; e < two * kUS; e += 256) {
        const int i = e >> 5, cc = e & 31;
        w1[i * (kUS + 1) + cc] = cc < cols ? W1[static_cast<int64_t>(two + i) * H + c0 + cc] : 0.0f;
    }
    const int cc = lane, pg = warp;
    for (int base = 0; base < count; base += kPB) {
        const int nb = min(kPB, count - base);
        __syncthreads();
        for (int e = tid; e < nb * d; e += 256) {
            const int pb = div_magic(e, dmag), x = e - pb * d;
            du[e] = maybe_bf16(c.d_unit[static_cast<int64_t>(list[base + pb]) * d + x], bf);
        }
        __syncthreads();
        // the transposed second layer, the activation's derivative, the inner product's share
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int pb = pg * 4 + p;
            float dhid = 0.0f, inner = 0.0f;
            if (pb < nb && cc < cols) {
                const float sum = dot4(du + pb * d, 1, wA + cc * (d + 1), 1, d);
                const int pair = list[base + pb];
                const int row = pair / K, k = pair - row * K;
                const float hid = load_hidden(c.io.hidden, ((static_cast<int64_t>(row) * T + t) * K + k) * H + c0 + cc, c.m.prod_bf16 != 0);
                dhid = maybe_bf16(sum * gelu_erf_grad(hid), bf);
                inner = dhid * (hid - c.m.b1[j * H + c0 + cc]);
            }
            dh[pb * (kUS + 1) + cc] = dhid;
            inner = warp_sum(inner);
            if (lane == 0 && pb < nb) c.part_sig[static_cast<int64_t>(s) * P + list[base + pb]] = inner;
        }
        __syncthreads();
        // the transposed first layer on the state columns [h ; m] of the cell input
        for (int e = tid; e < nb * two; e += 256) {
            const int pb = e / two, i = e - pb * two;
            c.part_dv[(static_cast<int64_t>(s) * P + list[base + pb]) * two + i] =
                dot4(dh + pb * (kUS + 1), 1, w1 + i * (kUS + 1), 1, kUS);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// mid on the tensor cores (bf16 products). blockIdx.x = (unit j, block cb): blocks 0 .. nB-1 are 128
// hidden columns of unit j, block nB is the gate's transposed linear; blockIdx.y = tile of 64 pairs.
// Per batch of 32 pairs:
//   D1 [128 hidden columns, 32 pairs] = W2 tile [128, d] x d_unit [32, d]^T
//   epilogue 1: times the activation's derivative at the recorded pre-activation, the block's
//               share of the cell norm's inner product, dhid as the bf16 operand of the next product
//   D2 [2d state columns (tiles of 128), 32 pairs] = W1 state tile [128, 128] x dhid [32, 128]^T
//   epilogue 2: the block's partial sum of dv.
// 256 threads: warp w reads TMEM lanes 32 (w % 4) .. +31 and the pairs 16 (w / 4) .. +15.
// Shared (dynamic): A3 [d/8][128][8], A4 [nT][16][128][8], B1 [d/8][32][8], B2 [16][32][8] bf16,
// sig [8][16] f32, list [64].
// ------------------------------------------------------------------------------------------------
constexpr int kTP = 32;
constexpr int kTcPairTile = 64;

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);   // one conversion for both halves
    return *reinterpret_cast<const uint32_t*>(&pair);
}

__global__ void __launch_bounds__(256) k_mid_tc(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int warp_count[8];
    __shared__ int n_list;
    __shared__ __align__(8) uint64_t bar_w, bar_m;
    __shared__ uint32_t tmem_slot;
    const int d = c.m.d, K = c.m.K, H = c.m.H, two = 2 * c.m.d, dplanes = c.m.d >> 3;
    const int P = c.io.B * K, T = c.io.T;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nB = c.nU, nT = (two + 127) / 128;
    const int j = blockIdx.x / (nB + 1), cb = blockIdx.x - j * (nB + 1);
    const bool is_gate = cb == nB;
    const int c0 = cb * 128;
    uint4* A3 = reinterpret_cast<uint4*>(dyn);                  // [d/8][128] (gate: [nT][d/8][128])
    uint4* A4 = A3 + (is_gate ? nT : 1) * dplanes * 128;       // [nT][16][128]
    uint4* B1 = A4 + (is_gate ? 0 : nT * 16 * 128);            // [d/8][32]
    uint4* B2 = B1 + dplanes * kTP;                            // [16][32]
    float* sig = reinterpret_cast<float*>(B2 + 16 * kTP);      // [8 warps][16 pairs]
    int* list = reinterpret_cast<int*>(sig + 8 * 16);          // [64]
    const int p0 = blockIdx.y * kTcPairTile;
    {
        const int p = p0 + tid;
        const bool mine = tid < kTcPairTile && p < P && c.pair_unit[p] == j;
        const unsigned mask = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(mask);
        if (tid == 0) {
            mbar_init(&bar_w, 1);
            mbar_init(&bar_m, 1);
        }
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
    if (tid == 0) {
        const uint32_t a3_bytes = static_cast<uint32_t>(dplanes) * 128 * 16, a4_bytes = static_cast<uint32_t>(nT) * 16 * 128 * 16;
        if (is_gate) {
            mbar_expect_tx(&bar_w, a3_bytes * nT);
            bulk_g2s(A3, c.m.umma_bw_gate, a3_bytes * nT, &bar_w);
        } else {
            const size_t blk = static_cast<size_t>(j) * nB + cb;
            mbar_expect_tx(&bar_w, a3_bytes + a4_bytes);
            bulk_g2s(A3, static_cast<const unsigned char*>(c.m.umma_bw_w2) + blk * a3_bytes, a3_bytes, &bar_w);
            bulk_g2s(A4, static_cast<const unsigned char*>(c.m.umma_bw_w1) + blk * a4_bytes, a4_bytes, &bar_w);
        }
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 128);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    const uint32_t idesc = umma_idesc_bf16(128, kTP);
    const int q = warp & 3, hf = warp >> 2;
    const int m = q * 32 + lane;
    uint32_t phase = 0;
    bool weights_in = false;
    const float* operand = is_gate ? c.dg : c.d_unit;
    for (int base = 0; base < count; base += kTP) {
        const int nb = min(kTP, count - base);
        for (int idx = tid; idx < dplanes * kTP; idx += 256) {
            const int n = idx & (kTP - 1), kc = idx >> 5;
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (n < nb) {
                const float4* src = reinterpret_cast<const float4*>(operand + static_cast<int64_t>(list[base + n]) * d) + kc * 2;
                const float4 lo = src[0], hi = src[1];
                packed = make_uint4(pack_bf16x2(lo.x, lo.y), pack_bf16x2(lo.z, lo.w), pack_bf16x2(hi.x, hi.y),
                                    pack_bf16x2(hi.z, hi.w));
            }
            B1[idx] = packed;
        }
        fence_async_smem();
        if (!weights_in) {
            mbar_wait(&bar_w, 0, c.status);
            weights_in = true;
        }
        tcgen05_fence_before();
        __syncthreads();
        if (is_gate) {
            // dv's gate part: [2d state columns, pairs] = gate tile [128, d] x dg [32, d]^T
            if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
                tcgen05_fence_after();
                const uint64_t db = umma_desc(B1, kTP);
                for (int tl = 0; tl < nT; ++tl) {
                    const uint64_t da = umma_desc(A3 + tl * dplanes * 128, 128);
                    umma_chain(taddr + tl * kTP, da, db, idesc, d >> 4, umma_kstep(128), umma_kstep(kTP));
                }
                umma_commit(&bar_m);
            }
            mbar_wait(&bar_m, phase, c.status);
            phase ^= 1u;
            tcgen05_fence_after();
            for (int tl = 0; tl < nT; ++tl) {
                float acc[16];
                tmem_ld8(tmem_addr(taddr, q * 32, tl * kTP + hf * 16), acc);
                tmem_ld8(tmem_addr(taddr, q * 32, tl * kTP + hf * 16 + 8), acc + 8);
                const int i = tl * 128 + m;
                if (i < two) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int n = hf * 16 + e;
                        if (n < nb) c.part_dv[(static_cast<int64_t>(nB) * P + list[base + n]) * two + i] = acc[e];
                    }
                }
            }
            tcgen05_fence_before();
            __syncthreads();
            continue;
        }
        if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
            tcgen05_fence_after();
            const uint64_t da = umma_desc(A3, 128), db = umma_desc(B1, kTP);
            umma_chain(taddr, da, db, idesc, d >> 4, umma_kstep(128), umma_kstep(kTP));
            umma_commit(&bar_m);
        }
        mbar_wait(&bar_m, phase, c.status);
        phase ^= 1u;
        tcgen05_fence_after();
        // epilogue 1: lane m is hidden column c0 + m
        {
            float acc[16];
            tmem_ld8(tmem_addr(taddr, q * 32, hf * 16), acc);
            tmem_ld8(tmem_addr(taddr, q * 32, hf * 16 + 8), acc + 8);
            const bool col_ok = c0 + m < H;
            const float b1v = col_ok ? c.m.b1[j * H + c0 + m] : 0.0f;
            uint16_t* b2_half = reinterpret_cast<uint16_t*>(B2);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int n = hf * 16 + e;
                float dhid = 0.0f, inner = 0.0f;
                if (n < nb && col_ok) {
                    const int pair = list[base + n];
                    const int row = pair / K, k = pair - row * K;
                    const float hid = load_hidden(c.io.hidden, ((static_cast<int64_t>(row) * T + t) * K + k) * H + c0 + m, true);
                    dhid = bf16r(acc[e] * gelu_erf_grad(hid));
                    inner = dhid * (hid - b1v);
                }
                b2_half[((m >> 3) * kTP + n) * 8 + (m & 7)] = bf16_bits(dhid);
                inner = warp_sum(inner);
                if (lane == 0) sig[warp * 16 + e] = inner;
            }
        }
        fence_async_smem();
        tcgen05_fence_before();
        __syncthreads();
        // the block's share of the inner product: the four lane quarters in order
        if (tid < kTP && tid < nb) {
            const int hf2 = tid >> 4, e = tid & 15;
            float total = 0.0f;
            for (int qq = 0; qq < 4; ++qq) total += sig[(hf2 * 4 + qq) * 16 + e];
            c.part_sig[static_cast<int64_t>(cb) * P + list[base + tid]] = total;
        }
        if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
            tcgen05_fence_after();
            const uint64_t db = umma_desc(B2, kTP);
            for (int tl = 0; tl < nT; ++tl) {
                const uint64_t da = umma_desc(A4 + tl * 16 * 128, 128);
                umma_chain(taddr + kTP + tl * kTP, da, db, idesc, 8, umma_kstep(128), umma_kstep(kTP));
            }
            umma_commit(&bar_m);
        }
        mbar_wait(&bar_m, phase, c.status);
        phase ^= 1u;
        tcgen05_fence_after();
        for (int tl = 0; tl < nT; ++tl) {
            float acc[16];
            tmem_ld8(tmem_addr(taddr, q * 32, kTP + tl * kTP + hf * 16), acc);
            tmem_ld8(tmem_addr(taddr, q * 32, kTP + tl * kTP + hf * 16 + 8), acc + 8);
            const int i = tl * 128 + m;
            if (i < two) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int n = hf * 16 + e;
                    if (n < nb) c.part_dv[(static_cast<int64_t>(cb) * P + list[base + n]) * two + i] = acc[e];
                }
            }
        }
        tcgen05_fence_before();
        __syncthreads();
    }
    if (warp == 0) tmem_dealloc(taddr, 128);
}

// ------------------------------------------------------------------------------------------------
// tail. Shared (dynamic): stage [K + K D][d], ds [K][2d], dvm [K][d], vt [d][d+1], cell_of [K],
// back [K], tgt [K + K D], first [K + K D], ew [K D].
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tail_phase(const BwdCtx& c, int t, unsigned char* dyn) {
    const int N = c.m.N, d = c.m.d, K = c.m.K, D = c.m.D, T = c.io.T, two = 2 * c.m.d;
    const uint32_t twomag = magic_of(2 * c.m.d);
    const uint32_t dmag = magic_of(d);   // e / d as a multiply-high
    const int P = c.io.B * K, U = K + K * D;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    float* stage = reinterpret_cast<float*>(dyn);   // [U][d] the rows of A this position touches
    float* ds = stage + U * d;                      // [K][2d]
    float* dvm = ds + K * two;                      // [K][d]
    float* vt = dvm + K * d;                        // [d][d+1]
    int* cell_of = reinterpret_cast<int*>(vt + d * (d + 1));
    float* back = reinterpret_cast<float*>(cell_of + K);  // [K] (rms^2 / n) sigma
    int* tgt = reinterpret_cast<int*>(back + K);    // [U] the row of A update u adds to (-1: none)
    int* first = tgt + U;                           // [U] the first update with the same target
    float* ew = reinterpret_cast<float*>(first + U);  // [K D]
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    const int64_t pair0 = static_cast<int64_t>(row) * K;
    float* A = c.io.A + static_cast<int64_t>(row) * N * d;
    float* R = c.io.R + static_cast<int64_t>(row) * d;
    const float in_dim = static_cast<float>(4 * d);
    BW_MARK(0);
    for (int e = tid; e < d * d; e += nt) cp_async4(vt + (div_magic(e, dmag)) * (d + 1) + (e - div_magic(e, dmag) * d), c.m.v_t + e);
    cp_async_commit();   // in flight while the position's values are gathered
    for (int k = tid; k < K; k += nt) {
        const bool ok = c.io.valid[rt * K + k] != 0;
        const int n = ok ? static_cast<int>(c.io.cells[rt * K + k]) : -1;
        cell_of[k] = n;
        tgt[k] = n;
        float sigma = c.sig_gate[pair0 + k];
        if (ok)
            for (int s = 0; s < c.nU; ++s) sigma += c.part_sig[static_cast<int64_t>(s) * P + pair0 + k];
        const float r = c.io.rms[rt * K + k];
        back[k] = r * r / in_dim * sigma;
    }
    for (int e = tid; e < K * D; e += nt) {
        const int k = e / D, j = e - k * D;
        const bool ok = c.io.valid[rt * K + k] != 0;
        const int n = ok ? static_cast<int>(c.io.cells[rt * K + k]) : 0;
        tgt[K + e] = ok ? c.m.pad_src[n * D + j] : -1;
        ew[e] = ok ? c.m.edge_w[n * D + j] : 0.0f;
    }
    __syncthreads();
    BW_MARK(1);
    for (int u = tid; u < U; u += nt) {
        int f = u;
        if (tgt[u] >= 0)
            for (int w = 0; w < u; ++w)
                if (tgt[w] == tgt[u]) {
                    f = w;
                    break;
                }
        first[u] = f;
    }
    BW_MARK(2);
    // ds = rms (g_n dv) - (rms^2 / n) sigma [h_old ; m] on the state columns
    // (four elements a thread per round: their partial sums' loads are in flight together)
    for (int e0 = tid; e0 < K * two; e0 += 4 * nt) {
        float dv[4], state[4];
        const float* from[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt;
            const int k = min(div_magic(e, twomag), K - 1), i = e - div_magic(e, twomag) * two;
            const bool ok = e < K * two && cell_of[k] >= 0;
            from[u] = ok ? c.part_dv + (pair0 + k) * two + i : c.part_dv;   // a padded slot's sum is not used
            state[u] = !ok ? 0.0f : i < d ? c.io.h_old[(rt * K + k) * d + i] : c.io.m[(rt * K + k) * d + i - d];
        }
        {   // the slices' partial sums in sum4's order (four running sums by slice mod 4), four elements abreast
            const int64_t sa = static_cast<int64_t>(P) * two;
            const int n = c.nU + 1;
            float acc[4][4] = {};
            int sl = 0;
            for (; sl + 4 <= n; sl += 4)
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int w = 0; w < 4; ++w) acc[u][w] += from[u][(sl + w) * sa];
            for (; sl < n; ++sl)
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u][0] += from[u][sl * sa];
#pragma unroll
            for (int u = 0; u < 4; ++u) dv[u] = (acc[u][0] + acc[u][1]) + (acc[u][2] + acc[u][3]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt;
            if (e >= K * two) continue;
            const int k = div_magic(e, twomag), i = e - k * two;
            ds[e] = cell_of[k] >= 0 ? c.io.rms[rt * K + k] * (c.m.norm_w[two + i] * dv[u]) - back[k] * state[u] : 0.0f;
        }
    }
    BW_MARK(3);
    cp_async_wait_all();
    __syncthreads();
    BW_MARK(4);
    // the touched rows of A, each loaded once (all loads in flight together)
#pragma unroll 4
    for (int e = tid; e < U * d; e += nt) {
        const int u = div_magic(e, dmag), x = e - u * d;
        if (tgt[u] >= 0 && first[u] == u) stage[e] = A[static_cast<int64_t>(tgt[u]) * d + x];
    }
    // dvm = dm V: m = sum_e a_e (V h_src), (V h)[x] = sum_i h[i] v_t[i][x]
    const int per = max(1, min(4, K * d / nt));   // slots a thread: a weight is read once for them
    for (int e = tid; e < ((K + per - 1) / per) * d; e += nt) {
        const int k0 = (div_magic(e, dmag)) * per, i = e - (div_magic(e, dmag)) * d;
        float out[4];
        dot4_rows(ds + k0 * two + d, two, min(per, K - k0), vt + i * (d + 1), 1, d, out);
        for (int r = 0; r < per && k0 + r < K; ++r) dvm[(k0 + r) * d + i] = out[r];
    }
    __syncthreads();
    BW_MARK(5);
    // a thread owns a column of some of the touched rows (row first[u] belongs to group first[u] mod
    // G, G = threads / d): a row's additions stay in slot order, the cells' own cotangents first,
    // then every edge
    const bool cut = c.io.reset[rt] != 0;
    int G = 1;
    while (2 * G * d <= nt) G *= 2;   // a power of two: the group of a row is a mask, not a division
    for (int e = tid; e < G * d; e += nt) {
        const int g = div_magic(e, dmag), x = e - g * d;
        for (int k = 0; k < K; ++k) {
            const int f = first[k];
            if (tgt[k] >= 0 && (f & (G - 1)) == g) stage[f * d + x] += ds[k * two + x];
        }
        for (int k = 0; k < K; ++k) {
            const float dv = dvm[k * d + x];
            for (int j = 0; j < D; ++j) {
                const int u = K + k * D + j, f = first[u];
                if (tgt[u] >= 0 && (f & (G - 1)) == g) stage[f * d + x] += ew[u - K] * dv;
            }
        }
    }
    for (int x = tid; x < d; x += nt) {
        float r = R[x];
        if (c.io.d_q_pre) r += c.io.d_q_pre[rt * d + x];
        R[x] = cut ? 0.0f : r;
    }
    __syncthreads();
    BW_MARK(6);
    if (cut) {
        for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
    } else {
        for (int e = tid; e < U * d; e += nt) {
            const int u = div_magic(e, dmag), x = e - u * d;
            if (tgt[u] >= 0 && first[u] == u) A[static_cast<int64_t>(tgt[u]) * d + x] = stage[e];
        }
    }
}

__global__ void __launch_bounds__(512) k_head(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    head_phase(c, t, dyn);
}

// The tail of position t and the head of position t - 1 of the same row in one launch.
__global__ void __launch_bounds__(512) k_tail_head(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    tail_phase(c, t, dyn);
    if (t > 0) {
        __syncthreads();
        head_phase(c, t - 1, dyn);
    }
}

size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
struct Layout {
    size_t d_unit, dg, sig_gate, part_dv, part_sig, pair_unit, total;
};
Layout layout(const HsnwModel& m, int B) {
    Layout L;
    const size_t P = static_cast<size_t>(B) * m.K;
    const int nU = (m.H + kUS - 1) / kUS;
    size_t off = 256;   // the status area: int 0 is the error word of the bounded waits
    L.d_unit = off; off += align_up(sizeof(float) * P * m.d);
    L.dg = off; off += align_up(sizeof(float) * P * m.d);
    L.sig_gate = off; off += align_up(sizeof(float) * P);
    L.part_dv = off; off += align_up(sizeof(float) * (nU + 1) * P * 2 * m.d);
    L.part_sig = off; off += align_up(sizeof(float) * nU * P);
    L.pair_unit = off; off += align_up(sizeof(int) * P);
    L.total = off;
    return L;
}
size_t head_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(m.d) + 3 * m.K + 3 * static_cast<size_t>(m.K) * m.d
        + static_cast<size_t>(m.d) * (m.d + 1));
}
size_t mid_shared(const HsnwModel& m) {
    const size_t d = m.d;
    const size_t wa = (2 * d > static_cast<size_t>(kUS) ? 2 * d : kUS) * (d + 1);
    return sizeof(float) * (kPB * d + wa + 2 * d * (kUS + 1) + kPB * (kUS + 1) + kPairTile);
}
size_t mid_tc_shared(const HsnwModel& m) {
    const size_t dplanes = m.d / 8, nT = (2 * static_cast<size_t>(m.d) + 127) / 128;
    const size_t a = nT * dplanes * 128 > dplanes * 128 + nT * 16 * 128 ? nT * dplanes * 128 : dplanes * 128 + nT * 16 * 128;
    return 16 * (a + dplanes * kTP + 16 * kTP) + sizeof(float) * 8 * 16 + sizeof(int) * kTcPairTile;
}
size_t tail_shared(const HsnwModel& m) {
    const size_t d = m.d, K = m.K, U = K + K * m.D;
    return sizeof(float) * (U * d + 3 * K * d + d * (d + 1) + 2 * K + 2 * U + K * m.D);
}

}  // namespace

extern "C" int64_t hsnw_backward_scratch_bytes(const HsnwModel* model, int32_t B, int32_t T) {
    (void)T;
    if (!model || B < 1) return 0;
    return static_cast<int64_t>(layout(*model, B).total);
}

// The sizes the reverse sweep's kernels take (the forward's check_model has the same bounds): the index
// arithmetic divides by multiply-highs that need d >= 2, and rows move 16 bytes at a time.
static int check_backward_model(const HsnwModel& m) {
    if (m.d < 4 || m.d % 4) return hsnw_fail(HSNW_E_UNSUPPORTED, "window_backward: d must be a multiple of 4");
    if (m.H < 1 || m.M < 1 || m.D < 1) return hsnw_fail(HSNW_E_ARG, "window_backward: H, M and D must be positive");
    return HSNW_OK;
}

extern "C" int hsnw_window_backward(const HsnwModel* model, const HsnwBackward* io, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (!model || !io) return hsnw_fail(HSNW_E_ARG, "window_backward: null argument");
    const HsnwModel& m = *model;
    if (m.N < 1 || m.d < 1 || m.K < 1 || m.K > m.N || io->B < 1 || io->T < 1)
        return hsnw_fail(HSNW_E_ARG, "window_backward: sizes must be positive and K <= N");
    if (!io->c || !io->b || !io->h_old || !io->cells || !io->valid || !io->reset || !io->dc || !io->db
        || !io->A || !io->R)
        return hsnw_fail(HSNW_E_ARG, "window_backward: a required pointer is null");
    const bool full = io->full_cut != 0;
    if (!full && (!io->y || !io->gate_pre || !io->m || !io->rms || !io->hidden || !io->units))
        return hsnw_fail(HSNW_E_ARG, "window_backward: the state gradient needs the round's record");
    if (int rc = check_backward_model(m)) return rc;
    // the status area at the head of the scratch: int 0 is set to 1 by a bounded wait that ran out
    const bool has_scratch = io->scratch && io->scratch_bytes >= 256 && !(reinterpret_cast<uintptr_t>(io->scratch) & 255);
    if (!full && !has_scratch)
        return hsnw_fail(HSNW_E_ARG, "window_backward: scratch too small or not 256-byte aligned");
    int* status = has_scratch ? static_cast<int*>(io->scratch) : nullptr;
    if (status && cudaMemsetAsync(status, 0, 256, static_cast<cudaStream_t>(stream_)) != cudaSuccess)
        return hsnw_check_launch("window_backward");
    if (!full) {
        // one persistent cluster per row when the shape fits (window_rows_bwd.cu); an error of its launch is
        // the call's error, only a shape it does not take goes on to the phases
        const int rc_rows = hsnw_rows_backward(model, io, status, static_cast<cudaStream_t>(stream_));
        if (rc_rows != HSNW_DECLINED) {
            if (rc_rows == HSNW_OK) hsnw_set_path(HSNW_PATH_ROWS);
            return rc_rows;
        }
    }
    hsnw_set_path(HSNW_PATH_PHASES);
    const size_t cap = hsnw_max_shared() - 4096;
    const size_t sh_head = head_shared(m), sh_mid = mid_shared(m), sh_tail = tail_shared(m);
    const size_t sh_both = sh_head > sh_tail ? sh_head : sh_tail;
    if (sh_head > cap || (!full && (sh_mid > cap || sh_tail > cap)))
        return hsnw_fail(HSNW_E_UNSUPPORTED, "window_backward: a phase's working set exceeds a block's shared memory");
    const Layout L = layout(m, io->B);
    if (!full && (!io->scratch || io->scratch_bytes < static_cast<int64_t>(L.total)
        || (reinterpret_cast<uintptr_t>(io->scratch) & 255)))
        return hsnw_fail(HSNW_E_ARG, "window_backward: scratch too small or not 256-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    BwdCtx c;
    c.m = m;
    c.io = *io;
    const bool mid_tc = !full && m.prod_bf16 && m.umma_bw_w2 && m.umma_bw_w1 && m.umma_bw_gate && m.d % 16 == 0
        && m.d <= 128 && mid_tc_shared(m) <= cap;
    c.nU = mid_tc ? (m.H + 127) / 128 : (m.H + kUS - 1) / kUS;
    unsigned char* base = static_cast<unsigned char*>(io->scratch);
    c.d_unit = full ? nullptr : reinterpret_cast<float*>(base + L.d_unit);
    c.dg = full ? nullptr : reinterpret_cast<float*>(base + L.dg);
    c.sig_gate = full ? nullptr : reinterpret_cast<float*>(base + L.sig_gate);
    c.part_dv = full ? nullptr : reinterpret_cast<float*>(base + L.part_dv);
    c.part_sig = full ? nullptr : reinterpret_cast<float*>(base + L.part_sig);
    c.pair_unit = full ? nullptr : reinterpret_cast<int*>(base + L.pair_unit);
    c.status = status;
    const int B = io->B, T = io->T;
    const int ht = m.K * m.d >= 2048 ? 512 : 256;   // threads of the head and tail: wide rows have the work for 16 warps
    const int pair_tile = mid_tc ? kTcPairTile : kPairTile;
    const dim3 mid_grid(m.M * (c.nU + 1), (B * m.K + pair_tile - 1) / pair_tile);
    const size_t sh_mid_tc = mid_tc_shared(m);
    if (full) {
        for (int t = T - 1; t >= 0; --t) {
            hsnw_profile_mark(HSNW_K_HEAD, stream);
            k_head<<<B, ht, sh_head, stream>>>(c, t);
        }
        return hsnw_check_launch("window_backward");
    }
    // head(T-1) | mid(T-1) | tail(T-1) + head(T-2) | mid(T-2) | ... | tail(0)
    hsnw_profile_mark(HSNW_K_HEAD, stream);
    k_head<<<B, ht, sh_head, stream>>>(c, T - 1);
    for (int t = T - 1; t >= 0; --t) {
        hsnw_profile_mark(HSNW_K_MID, stream);
        if (mid_tc) k_mid_tc<<<mid_grid, 256, sh_mid_tc, stream>>>(c, t);
        else k_mid<<<mid_grid, 256, sh_mid, stream>>>(c, t);
        hsnw_profile_mark(HSNW_K_TAIL_HEAD, stream);
        k_tail_head<<<B, ht, sh_both, stream>>>(c, t);
        if (int rc = hsnw_check_launch("window_backward")) return rc;
    }
    return HSNW_OK;
}

// ------------------------------------------------------------------------------------------------
// The reverse sweep for callers that cannot allocate: its scratch is this fixed array, part of the
// library's image on every GPU that loads it (held until the process exits).
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = static_cast<size_t>(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
constexpr int kStaticDevices = 64;
std::mutex static_mutex;
void* static_scratch_address[kStaticDevices] = {};  // the array's device address, per device
}  // namespace

extern "C" int64_t hsnw_static_scratch_bytes(void) { return static_cast<int64_t>(kStaticScratchBytes); }

extern "C" int hsnw_window_backward_static(const HsnwModel* model, const HsnwBackward* io, void* stream) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (!model || !io) return hsnw_fail(HSNW_E_ARG, "window_backward_static: null argument");
    if (io->B < 1 || io->T < 1 || model->K < 1 || model->d < 1 || model->H < 1)
        return hsnw_fail(HSNW_E_ARG, "window_backward_static: sizes must be positive");
    const size_t need = layout(*model, io->B).total;
    if (need > kStaticScratchBytes) {
        char buffer[200];
        snprintf(buffer, sizeof(buffer),
                 "window_backward_static: B x K = %d x %d pairs need %zu bytes of scratch, the built-in array holds %zu;"
                 " use hsnw_window_backward with the caller's scratch",
                 io->B, model->K, need, kStaticScratchBytes);
        return hsnw_fail(HSNW_E_UNSUPPORTED, buffer);
    }
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kStaticDevices)
        return hsnw_fail(HSNW_E_CUDA, "window_backward_static: no current device");
    void* address = nullptr;
    {
        // In host code the array's name is only a handle; its address on the current device comes
        // from the runtime. Looked up on the first call per device, with that device current.
        std::lock_guard<std::mutex> lock(static_mutex);
        if (!static_scratch_address[device]) {
            void* found = nullptr;
            const cudaError_t status = cudaGetSymbolAddress(&found, g_static_scratch);
            if (status != cudaSuccess || !found) {
                cudaGetLastError();
                char buffer[200];
                snprintf(buffer, sizeof(buffer), "window_backward_static: cudaGetSymbolAddress: %s",
                         cudaGetErrorString(status));
                return hsnw_fail(HSNW_E_CUDA, buffer);
            }
            static_scratch_address[device] = found;
        }
        address = static_scratch_address[device];
    }
    HsnwBackward local = *io;
    local.scratch = address;
    local.scratch_bytes = static_cast<int64_t>(kStaticScratchBytes);
    return hsnw_window_backward(model, &local, stream);
}

void hsnw_backward_set_attributes() {
    const struct { const void* f; const char* n; } ks[] = {
        {reinterpret_cast<const void*>(k_head), "head"}, {reinterpret_cast<const void*>(k_mid), "mid"},
        {reinterpret_cast<const void*>(k_mid_tc), "mid_tc"},
        {reinterpret_cast<const void*>(k_tail_head), "tail_head"}};
    for (const auto& k : ks)
        if (!hsnw_opt_in(k.f, k.n)) hsnw_attribute_failed();
}
