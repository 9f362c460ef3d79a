// The reverse sweep of a window (state gradient) as ONE persistent kernel: a thread-block cluster
// per batch row walks t = T-1 .. 0 with the row's state cotangent A [N, d] resident in the
// cluster's shared memory (block r owns the cells [r N/C, (r+1) N/C)) and R [d] replicated.
// The counterpart of window_rows.cu for window_bwd.cu's phases; same arithmetic and rounding
// points (reference python/hsn/train/state_gradient.py:288-485), other orders of fp32 partial sums.
//
// Per position, four cluster barriers:
//   H   the slots' owners (slot k belongs to block k mod C): R += D_t, the gated carry through
//       A[cell] at the cell's owner, dc, db, the candidate's and the gate's backward, d_unit = dy
//       W_out; d_unit and dg go to every block                                          | sync 1
//   M   every block, on its 128 hidden columns of the units the slots ran (two streamed chunks a
//       unit: W2's rows and the state rows of W1): the transposed second layer, the activation's
//       derivative at the recorded pre-activation, the norm's inner product, the transposed first
//       layer on the 2d state columns; and its share of the gate's transposed linear; partial sums
//       go to the slots' owners                                                         | sync 2
//   T1  the owners: the cell norm's backward ds, dvm = dm V; both go to every block     | sync 3
//   T2  every block adds, for its own cells, the slots' own cotangents and then every edge's
//       share in slot order (the fixed order of window_bwd.cu's tail); R += P_t; the reset | sync 4
// The decisions are recorded, so the chunks of the next position are requested (TMA bulk copies
// into a 3-deep ring) while this one computes; the position's records are prefetched one position
// ahead with cp.async. Every ring wait is bounded.
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "stage.cuh"
#include "host_util.h"
#include "rows.cuh"
#include "umma.cuh"

using namespace hsnw;

namespace {

#ifdef HSNW_TRACE
#define BMARK(i)                                                                              \
    do {                                                                                      \
        if (tid == 0 && row == 0 && t == T / 2) {                                             \
            unsigned long long now;                                                           \
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);                     \
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");        \
            trace_s[(i)] = now;                                                               \
        }                                                                                     \
    } while (0)
#else
#define BMARK(i) do { } while (0)
#endif

constexpr int kRowThreadsB = kConsumers + 128;   // + the producer warp (copies), two issuer warps (tensor-core products), the decision warp
constexpr int kDhidOperand = 2 * 16 * 16 * 8;   // bytes of one
constexpr int kMaxKB = 8;
constexpr int kMaxMB = 16;

struct RowsBwdCtx {
    HsnwModel m;
    HsnwBackward io;
    int C, Nc, Ks;
    uint32_t bank_bytes, w2_bytes;   // a unit's weights on the block's 128 columns (two pieces: W2's, then W1's state rows = a ring slot), the first piece
    unsigned long long* trace;       // phase timestamps (HSNW_TRACE builds): after the status area of the caller's scratch, or null
    int* status;                     // set to 1 by a ring wait that ran out
};

__host__ __device__ inline size_t up16b(size_t v) { return (v + 15) & ~static_cast<size_t>(15); }

struct RowsBwdSmem {
    size_t ring, A, wout, vt, gate, norm_w, cand_w, gate_b, b1, R, Rs, rec[2], hid[2], dq[2], dec[2], du_all, b2, dg_all,
        inbox_dv, inbox_sig, inbox_g, ds_all, dvm_all, red, own, total;
};
// rec: per owned slot c, b, h_old, y, gate_pre, m, d_h_sel [7][Ks][d], then rms [Ks]
// dec: cell_of [K], unit_of [K], tgt [K D], ew [K D], ulist [16], umask [16], n_units
__host__ __device__ inline RowsBwdSmem rows_bwd_smem(const HsnwModel& m, int C, uint32_t slot_bytes) {
    RowsBwdSmem L;
    const size_t d = m.d, N = m.N, K = m.K, M = m.M, D = m.D, Nc = N / C, Ks = (K + C - 1) / C;
    size_t o = 0;
    auto take = [&o](size_t bytes) {
        const size_t at = o;
        o += up16b(bytes);
        return at;
    };
    L.ring = take(3 * static_cast<size_t>(slot_bytes) + 1024);   // two slots of each kind (the first kind's are half as large) + room to start on a 1024-byte boundary
    L.A = take(4 * Nc * d);
    L.wout = take(2 * d * d);
    L.vt = take(2 * d * d);
    L.gate = take(2 * (2 * d / C) * d);
    L.norm_w = take(4 * 2 * d);
    L.cand_w = take(4 * d);
    L.gate_b = take(4 * d);
    L.b1 = take(4 * M * 128);
    L.R = take(4 * d);
    L.Rs = take(4 * d);
    for (int s = 0; s < 2; ++s) {
        L.rec[s] = take(4 * (7 * Ks * d + Ks) + 16);
        L.hid[s] = take(2 * K * 128);   // the recorded pre-activations of the block's columns, bfloat16
        L.dq[s] = take(4 * 2 * d);
        L.dec[s] = take(4 * (2 * K + 2 * K * D + 2 * kMaxMB + 4 + K + K * D));
    }
    L.du_all = take(2 * 16 * d);        // d_unit of every slot as a bf16 operand [d/8][16][8]
    L.b2 = take(2 * kDhidOperand);      // two bf16 operands [16][16][8]: dhid of a unit on the block's 128 columns
    L.dg_all = take(4 * K * d);
    L.inbox_dv = take(4 * C * Ks * 2 * d);
    L.inbox_sig = take(4 * C * Ks + 16);
    L.inbox_g = take(4 * Ks * 2 * d);
    L.ds_all = take(4 * K * d);
    L.dvm_all = take(4 * K * d);
    L.red = take(4 * 8 * 8);            // the epilogue warps' shares of the slots' inner products
    L.own = take(4 * Ks * (8 * d + 8));   // dzs, ysv, sgs, dy, ds [2d], dc, db per owned slot; rho, dot, sig_gate, back
    L.total = o;
    return L;
}

template <int D_>
__global__ void __launch_bounds__(kRowThreadsB, 1) k_rows_bwd(RowsBwdCtx c) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t full_p[2], empty_p[2], full_q[2], empty_q[2];   // the two rings' slots
    __shared__ int failed_s;
    __shared__ __align__(8) uint64_t bar_d1[2], bar_d2;   // a unit's first product (two accumulators in turn); the position's second products
    __shared__ __align__(8) uint64_t bar_act[2];          // a unit's dhid operand is written (two buffers in turn): one arrival per compute warp
    __shared__ __align__(8) uint64_t bar_sp[2];           // a unit's second product has read its operand buffer
    __shared__ __align__(8) uint64_t bar_dec;             // the next position's unit lists are in place
    __shared__ __align__(8) uint64_t bar_rec;             // the next position's records have landed (bulk copies by the decision warp)
    __shared__ uint32_t tmem_slot;
#ifdef HSNW_TRACE
    __shared__ unsigned long long trace_s[32];   // written to memory when the kernel ends (a store before a barrier delays it)
#endif

    cg::cluster_group cl = cg::this_cluster();
    constexpr int d = D_, two = 2 * D_;
    const int C = c.C, r = static_cast<int>(cl.block_rank());
    const int row = blockIdx.x / C;
    const int N = c.m.N, K = c.m.K, M = c.m.M, D = c.m.D, H = c.m.H;
    const int T = c.io.T, Nc = c.Nc, Ks = c.Ks;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool consumer = warp < kConsumers / 32;
    const int role = warp - kConsumers / 32;   // 0: copies; 1: the first products; 2: the second products; 3: the next position's decision
    const int gcols = two / C;          // the gate's state outputs of this block
    const int cmask = C - 1, cshift = __ffs(C) - 1;   // the cluster size is a power of two
    const int gshift = __ffs(gcols) - 1;              // so is 2d / C (d is 16, 32 or 64)
    const int cell0 = r * Nc;
    const int U = K + K * D;
    const uint32_t nc_magic = 0xffffffffu / static_cast<uint32_t>(Nc) + 1u;   // n / Nc as a multiply-high
    const uint32_t d_magic = 0xffffffffu / static_cast<uint32_t>(D) + 1u;      // e / D the same way (the magic wraps to 0 for D = 1)
    auto div_D = [&](int e) { return D == 1 ? e : static_cast<int>(__umulhi(static_cast<uint32_t>(e), d_magic)); };

    const RowsBwdSmem L = rows_bwd_smem(c.m, C, c.bank_bytes - c.w2_bytes);
    const uint32_t slot_bytes = c.bank_bytes - c.w2_bytes;   // the larger piece
    unsigned char* ring = dyn + L.ring + ((1024u - (smem_addr(dyn + L.ring) & 1023u)) & 1023u);
    float* A_s = reinterpret_cast<float*>(dyn + L.A);
    uint16_t* wout = reinterpret_cast<uint16_t*>(dyn + L.wout);
    uint16_t* vt = reinterpret_cast<uint16_t*>(dyn + L.vt);
    uint16_t* gate = reinterpret_cast<uint16_t*>(dyn + L.gate);
    float* norm_w = reinterpret_cast<float*>(dyn + L.norm_w);
    float* cand_w = reinterpret_cast<float*>(dyn + L.cand_w);
    float* gate_b = reinterpret_cast<float*>(dyn + L.gate_b);
    float* b1s = reinterpret_cast<float*>(dyn + L.b1);
    float* R_s = reinterpret_cast<float*>(dyn + L.R);
    float* Rs = reinterpret_cast<float*>(dyn + L.Rs);
    uint16_t* du_op = reinterpret_cast<uint16_t*>(dyn + L.du_all);
    uint16_t* b2 = reinterpret_cast<uint16_t*>(dyn + L.b2);
    float* dg_all = reinterpret_cast<float*>(dyn + L.dg_all);
    float* inbox_dv = reinterpret_cast<float*>(dyn + L.inbox_dv);
    float* inbox_sig = reinterpret_cast<float*>(dyn + L.inbox_sig);
    float* inbox_g = reinterpret_cast<float*>(dyn + L.inbox_g);
    float* ds_all = reinterpret_cast<float*>(dyn + L.ds_all);
    float* dvm_all = reinterpret_cast<float*>(dyn + L.dvm_all);
    float* red = reinterpret_cast<float*>(dyn + L.red);
    float* own = reinterpret_cast<float*>(dyn + L.own);
    float* dzs = own;
    float* ysv = own + Ks * d;
    float* sgs = own + 2 * Ks * d;
    float* dy = own + 3 * Ks * d;
    float* ds = own + 4 * Ks * d;          // [Ks][2d]
    float* rho = own + 6 * Ks * d;
    float* dot = rho + Ks;
    float* sig_gate = dot + Ks;
    float* back = sig_gate + Ks;
    float* dcs = back + Ks;                // [Ks][d] dc and db of the position, written to memory off the critical path
    float* dbs = dcs + Ks * d;
    const unsigned char* bank = static_cast<const unsigned char*>(c.m.rows_bank_bw);

    auto rec_of = [&](int buf) { return reinterpret_cast<float*>(dyn + L.rec[buf]); };
    auto hid_of = [&](int buf) { return reinterpret_cast<uint16_t*>(dyn + L.hid[buf]); };
    auto dq_of = [&](int buf) { return reinterpret_cast<float*>(dyn + L.dq[buf]); };
    auto dec_of = [&](int buf) { return reinterpret_cast<int*>(dyn + L.dec[buf]); };
    // a position's decision block: cell_of [K], unit_of [K], tgt [K D], ew [K D] (floats), ulist [16],
    // umask [16], n_units
    const int o_unit = K, o_tgt = 2 * K, o_ew = 2 * K + K * D, o_ulist = 2 * K + 2 * K * D, o_umask = o_ulist + kMaxMB,
              o_n = o_umask + kMaxMB, o_own_n = o_n + 1, o_own = o_n + 2;   // own: the updates u whose target is a cell of this block

    // the records of position t, asynchronously, into buffer t & 1
    auto prefetch = [&](int t, int me, int crew) {   // by `crew` threads, `me` this one's index among them
        const int buf = t & 1;
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        float* rc = rec_of(buf);
        const float* srcs[7] = {c.io.c, c.io.b, c.io.h_old, c.io.y, c.io.gate_pre, c.io.m, c.io.d_h_sel};
#pragma unroll
        for (int a = 0; a < 7; ++a) {   // the array's index is a constant in every copy of the body
            if (!srcs[a]) continue;
            for (int e = me; e < Ks * (d / 4); e += crew) {
                const int kl = e / (d / 4), x4 = e - kl * (d / 4);
                const int k = kl * C + r;
                if (k < K) cp_async16(rc + (a * Ks + kl) * d + 4 * x4, srcs[a] + (rt * K + k) * d + 4 * x4);
            }
        }
        uint16_t* hd = hid_of(buf);
        const uint16_t* recorded = static_cast<const uint16_t*>(c.io.hidden);
        for (int e = me; e < K * 16; e += crew) {   // 128 bfloat16 a slot: sixteen 16-byte copies
            const int k = e >> 4, c8 = e & 15;
            cp_async16(hd + k * 128 + 8 * c8, recorded + (rt * K + k) * H + r * 128 + 8 * c8);
        }
        float* q = dq_of(buf);
        for (int e = me; e < 2 * (d / 4); e += crew) {
            const int which = e / (d / 4), x4 = e - which * (d / 4);
            const float* from = which == 0 ? c.io.d_q_post : c.io.d_q_pre;
            if (from) cp_async16(q + which * d + 4 * x4, from + rt * d + 4 * x4);
        }
        cp_async_commit();
    };
    // the same as bulk copies by ONE thread (the decision warp's, during the unit stage), arriving on bar_rec: a
    // slot's row of an array is d floats, the slot's recorded pre-activations 128 bfloat16, both whole 16-byte units
    auto prefetch_bulk = [&](int t) {
        const int buf = t & 1;
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        float* rc = rec_of(buf);
        const float* srcs[7] = {c.io.c, c.io.b, c.io.h_old, c.io.y, c.io.gate_pre, c.io.m, c.io.d_h_sel};
        int owned = 0;
        for (int kl = 0; kl < Ks; ++kl) owned += kl * C + r < K ? 1 : 0;
        int present = 0;
        for (int a = 0; a < 7; ++a) present += srcs[a] ? 1 : 0;
        const uint32_t row_bytes = static_cast<uint32_t>(sizeof(float)) * d;
        mbar_expect_tx(&bar_rec, static_cast<uint32_t>(present * owned) * row_bytes + static_cast<uint32_t>(K) * 256u
                                     + ((c.io.d_q_post ? 1u : 0u) + (c.io.d_q_pre ? 1u : 0u)) * row_bytes);
        for (int a = 0; a < 7; ++a) {
            if (!srcs[a]) continue;
            for (int kl = 0; kl < Ks; ++kl) {
                const int k = kl * C + r;
                if (k < K) bulk_g2s(rc + (a * Ks + kl) * d, srcs[a] + (rt * K + k) * d, row_bytes, &bar_rec);
            }
        }
        uint16_t* hd = hid_of(buf);
        const uint16_t* recorded = static_cast<const uint16_t*>(c.io.hidden);
        for (int k = 0; k < K; ++k) bulk_g2s(hd + k * 128, recorded + (rt * K + k) * H + r * 128, 256u, &bar_rec);
        float* q = dq_of(buf);
        if (c.io.d_q_post) bulk_g2s(q, c.io.d_q_post + rt * d, row_bytes, &bar_rec);
        if (c.io.d_q_pre) bulk_g2s(q + d, c.io.d_q_pre + rt * d, row_bytes, &bar_rec);
    };
    // the decision of position t: each thread loads what it will store (decision_store), so the
    // loads' latency is spent under other work
    int ld_cell = -1, ld_unit = -1, ld_tgt = -1;
    float ld_ew = 0.0f, ld_rms = 0.0f;
    auto decision_load = [&](int t, int me) {   // `me`: the thread's index among the (at least 128) that call it
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        if (me < K) {
            const bool ok = c.io.valid[rt * K + me] != 0;
            ld_cell = ok ? static_cast<int>(c.io.cells[rt * K + me]) : -1;
            ld_unit = ok ? static_cast<int>(c.io.units[rt * K + me]) : -1;
        }
        if (me >= 32 && me < 32 + K * D) {
            const int e = me - 32, k = div_D(e), jj = e - k * D;
            const bool ok = c.io.valid[rt * K + k] != 0;
            const int n = ok ? static_cast<int>(c.io.cells[rt * K + k]) : 0;
            ld_tgt = ok ? c.m.pad_src[n * D + jj] : -1;
            ld_ew = ok ? c.m.edge_w[n * D + jj] : 0.0f;
        }
        if (me >= 128 - 8 && me < 128 - 8 + Ks) {
            const int k = (me - (128 - 8)) * C + r;
            ld_rms = k < K ? c.io.rms[rt * K + k] : 0.0f;
        }
    };
    auto decision_store = [&](int t, int me) {
        int* dc_ = dec_of(t & 1);
        if (me < K) {
            dc_[me] = ld_cell;
            dc_[o_unit + me] = ld_unit;
        }
        if (me >= 32 && me < 32 + K * D) {
            dc_[o_tgt + me - 32] = ld_tgt;
            reinterpret_cast<float*>(dc_)[o_ew + me - 32] = ld_ew;
        }
        if (me >= 128 - 8 && me < 128 - 8 + Ks) rec_of(t & 1)[7 * Ks * d + me - (128 - 8)] = ld_rms;
    };
    // the units a position's slots ran, ascending, with each one's slots as a bit mask (warp 0)
    auto unit_lists = [&](int t) {
        int* dc_ = dec_of(t & 1);
        const int my_unit = lane < K ? dc_[o_unit + lane] : -1;
        int n = 0;
        for (int j = 0; j < M; ++j) {
            const unsigned mask = __ballot_sync(0xffffffffu, my_unit == j);
            if (mask) {
                if (lane == 0) {
                    dc_[o_ulist + n] = j;
                    dc_[o_umask + n] = static_cast<int>(mask);
                }
                ++n;
            }
        }
        if (lane == 0) dc_[o_n] = n;
        // the updates that land on this block's cells, in update order (slots, then edges)
        int count = 0;
        for (int u0 = 0; u0 < U; u0 += 32) {
            const int u = u0 + lane;
            const int tgt = u < U ? (u < K ? dc_[u] : dc_[o_tgt + u - K]) : -1;
            const bool mine = tgt >= cell0 && tgt < cell0 + Nc;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) dc_[o_own + count + __popc(mask & ((1u << lane) - 1u))] = u;
            count += __popc(mask);
        }
        if (lane == 0) dc_[o_own_n] = count;
        __syncwarp();
    };

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&full_p[s], 1);
            mbar_init(&empty_p[s], 1);
            mbar_init(&full_q[s], 1);
            mbar_init(&empty_q[s], 1);
        }
        mbar_init(&bar_d1[0], 1);
        mbar_init(&bar_d1[1], 1);
        mbar_init(&bar_d2, 1);
        mbar_init(&bar_act[0], kConsumers / 32);
        mbar_init(&bar_act[1], kConsumers / 32);
        mbar_init(&bar_sp[0], 1);
        mbar_init(&bar_sp[1], 1);
        mbar_init(&bar_dec, 1);
        mbar_init(&bar_rec, 1);
        failed_s = 0;
    }
    for (int e = tid; e < d * d; e += kConsumers) {
        wout[e] = bf16_bits(c.m.wout_t[e]);
        vt[e] = bf16_bits(c.m.v_t[e]);
    }
    for (int e = tid; e < gcols * d; e += kConsumers) gate[e] = bf16_bits(c.m.gate_t[static_cast<int64_t>(two + r * gcols) * d + e]);
    for (int e = tid; e < two; e += kConsumers) norm_w[e] = c.m.norm_w[two + e];
    for (int e = tid; e < d; e += kConsumers) {
        cand_w[e] = c.m.cand_w[e];
        gate_b[e] = c.m.gate_b[e];
        R_s[e] = c.io.R[static_cast<int64_t>(row) * d + e];
    }
    for (int e = tid; e < M * 128; e += kConsumers) b1s[e] = c.m.b1[(e >> 7) * H + r * 128 + (e & 127)];
    {
        const float* A = c.io.A + (static_cast<int64_t>(row) * N + cell0) * d;
        for (int e = tid; e < Nc * d; e += kConsumers) A_s[e] = A[e];
    }
    for (int buf = 0; buf < 2; ++buf) {   // optional inputs that are absent read as zeros
        for (int e = tid; e < 7 * Ks * d + Ks; e += kConsumers) rec_of(buf)[e] = 0.0f;
        for (int e = tid; e < 2 * d; e += kConsumers) dq_of(buf)[e] = 0.0f;
    }
    for (int e = tid; e < 16 * d; e += kConsumers) du_op[e] = 0;
    for (int e = tid; e < kDhidOperand; e += kConsumers) b2[e] = 0;   // (uint16 elements: both operands)
    if (warp == 0) tmem_alloc(&tmem_slot, 256);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    // completed phases of the per-unit barriers before this position (bar_d1, bar_act and bar_sp complete once per
    // unit, a position's even-numbered units on [0], the odd ones on [1]), of bar_d2 and of bar_dec
    uint32_t units_even = 0, units_odd = 0, d2_phase = 0, dec_phase = 0;
    if (consumer) {
        prefetch(T - 1, tid, kConsumers);
        decision_load(T - 1, tid);
        decision_store(T - 1, tid);
    }
    __syncthreads();
    if (warp == 0) unit_lists(T - 1);
    __syncthreads();
    // The stream of weight pieces, two a unit: W2's (the first product's) and W1's state rows (the second's). Each
    // kind has a ring of two slots and one consumer, its issuer warp (a slot's barrier tells two consecutive rounds
    // apart, no more: a warp that waited for a slot's round must have seen the round before, which holds when it
    // consumes every round itself). The producer warp requests the pieces in order of use, across the positions, two
    // units ahead. Unit number n (counted over the window) uses slot n & 1 of both rings, round n >> 1.
    uint32_t units_before = 0;          // units of the positions before this one
    unsigned char* ring_q = ring + 2 * c.w2_bytes;
    int cur_t = T - 1, cur_p = 0, cur_q = 0;   // the next pieces to request (producer's lane 0): position, unit index per kind
    // Request pieces of position cur_t, whose first unit is number `base`, up to its unit `limit` (exclusive). The two
    // rings are served independently, whichever slot is handed back first: a second-layer slot comes back only after
    // its unit's epilogue, and requests in order of use would hold the next first-layer pieces behind it.
    auto request = [&](uint32_t base, int limit) {
        const int* dc_ = dec_of(cur_t & 1);
        const int n = min(limit, dc_[o_n]);
        auto try_one = [&](bool second, bool wait) {   // the kind's next piece, if its slot is free (or after waiting for it)
            int& cur = second ? cur_q : cur_p;
            if (cur >= n) return false;
            const uint32_t unit = base + static_cast<uint32_t>(cur), slot = unit & 1u;
            uint64_t* empty = second ? &empty_q[slot] : &empty_p[slot];
            if (unit >= 2) {
                const uint32_t parity = ((unit >> 1) - 1u) & 1u;
                if (wait) {
                    ring_wait(empty, parity, c.status, &failed_s);
                } else {
                    uint32_t done;
                    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                                 : "=r"(done)
                                 : "r"(smem_addr(empty)), "r"(parity)
                                 : "memory");
                    if (!done) return false;
                }
            }
            uint64_t* full = second ? &full_q[slot] : &full_p[slot];
            const int j = dc_[o_ulist + cur];
            const unsigned char* from = bank + (static_cast<size_t>(j) * C + r) * c.bank_bytes + (second ? c.w2_bytes : 0u);
            const uint32_t bytes = second ? slot_bytes : c.w2_bytes;
            mbar_expect_tx(full, bytes);
            bulk_g2s(second ? ring_q + slot * slot_bytes : ring + slot * c.w2_bytes, from, bytes, full);
            ++cur;
            return true;
        };
        while ((cur_p < n || cur_q < n) && !failed_s) {
            const bool a = try_one(false, false), b = try_one(true, false);
            // nothing was handed back: sleep on the first-layer ring's slot if a piece of it is outstanding (it comes
            // back first), else on the other's (ring_wait: bounded, with a suspend-time hint)
            if (!a && !b) try_one(cur_p >= n, true);
        }
    };
    if (role == 0 && lane == 0) request(0u, 2);
    cl.sync();

    const float n_f = static_cast<float>(N);
    for (int t = T - 1; t >= 0; --t) {
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        const int buf = t & 1;
        float* rc = rec_of(buf);
        const uint16_t* hd = hid_of(buf);
        const float* q = dq_of(buf);
        const int* dc_ = dec_of(buf);
        const float* ew = reinterpret_cast<const float*>(dc_) + o_ew;
        const bool cut = c.io.reset[rt] != 0;
        BMARK(0);
        if (role == 3 && t > 0) {
            // The next position's decision block (recorded: it depends on nothing this sweep computes), a position
            // ahead and off every critical path: cells, units, edges and rms from memory, then the unit lists; the
            // producer warp requests that position's first pieces when this is in place.
            for (int pass = 0; pass < 4; ++pass) {
                decision_load(t - 1, lane + 32 * pass);
                decision_store(t - 1, lane + 32 * pass);
            }
            __syncwarp();
            unit_lists(t - 1);
            if (lane == 0) mbar_arrive(&bar_dec);
        }
        // ---------------- H
        if (consumer) {
            // this position's records: requested a position ago (the first position's by these warps before the loop)
            if (t == T - 1) cp_async_wait_all();
            else ring_wait(&bar_rec, static_cast<uint32_t>(T - 2 - t) & 1u, c.status, &failed_s);
            consumer_sync();
            if (tid < d) Rs[tid] = R_s[tid] + q[tid];
            consumer_sync();
            for (int e = tid; e < Ks * d; e += kConsumers) {
                const int kl = e / d, x = e - kl * d, k = kl * C + r;
                if (k >= K) continue;
                const int n = dc_[k];
                float dcv = 0.0f, dbv = 0.0f, dz = 0.0f, dgv = 0.0f, yv = 0.0f, sgv = 0.0f;
                if (n >= 0) {
                    const int no = static_cast<int>(__umulhi(static_cast<uint32_t>(n), nc_magic));
                    float* a = peer(cl, A_s, no) + (n - no * Nc) * d + x;
                    const float carried = *a + rc[(6 * Ks + kl) * d + x];
                    const float share = Rs[x] / n_f;
                    const float g = carried + share;
                    const float cv = rc[(0 * Ks + kl) * d + x], gt = rc[(1 * Ks + kl) * d + x];
                    dcv = gt * g;
                    dbv = (cv - rc[(2 * Ks + kl) * d + x]) * g;
                    *a = (1.0f - gt) * carried - gt * share;
                    dz = cand_w[x] * (dcv * (1.0f - cv * cv));
                    dgv = dbv * gt * (1.0f - gt);
                    yv = rc[(3 * Ks + kl) * d + x];
                    sgv = dgv * (rc[(4 * Ks + kl) * d + x] - gate_b[x]);
                }
                dcs[e] = dcv;
                dbs[e] = dbv;
                dzs[e] = dz;
                ysv[e] = yv;
                sgs[e] = sgv;
                const float dgb = bf16r(dgv);
                for (int p = 0; p < C; ++p) peer(cl, dg_all, p)[k * d + x] = dgb;
            }
            consumer_sync();
            // per owned slot, one warp without block barriers: rho, the mean, the gate's inner product,
            // dy = rho (cand_w dz) - rho^3 y mean(y cand_w dz), then d_unit = dy W_out to every block
            for (int kl = warp; kl < Ks; kl += kConsumers / 32) {
                const int k = kl * C + r;
                float sq = 0.0f, dt = 0.0f, s = 0.0f;
                for (int x = lane; x < d; x += 32) {
                    const float yv = ysv[kl * d + x];
                    sq += yv * yv;
                    dt += yv * dzs[kl * d + x];
                    s += sgs[kl * d + x];
                }
                sq = warp_sum(sq);
                dt = warp_sum(dt);
                s = warp_sum(s);
                const float rr = rsqrtf(sq / static_cast<float>(d) + c.m.cand_eps);
                const float mean = dt / static_cast<float>(d);
                if (lane == 0) sig_gate[kl] = s;
                const bool ok = k < K && dc_[k] >= 0;
                for (int x = lane; x < d; x += 32)
                    dy[kl * d + x] = ok ? rr * dzs[kl * d + x] - rr * rr * rr * ysv[kl * d + x] * mean : 0.0f;
                __syncwarp();
                if (k < K) {
                    for (int i = lane; i < d; i += 32) {
                        const uint16_t dub = bf16_bits(dot_bf16w(dy + kl * d, 1, wout + i * d, 1, d));
                        for (int p = 0; p < C; ++p) peer(cl, du_op, p)[((i >> 3) * 16 + k) * 8 + (i & 7)] = dub;
                    }
                }
            }
        }
        BMARK(1);
        cl.sync();   // 1
        BMARK(2);
        // ---------------- M
        BMARK(3);
        // The transposed layers on the streamed weights, on the tensor cores. A unit's weights on the block's
        // 128 hidden columns arrive as two pieces, each a ring slot of its own: W2's ([128 columns][d outputs])
        // and the state rows of W1 ([2d state inputs][128 columns]). D1 [128 columns, 16 slots] = W2 x
        // d_unit^T (its slot is handed back as soon as the product has run); the epilogue multiplies by the
        // activation's derivative at the recorded pre-activation for the slots that ran the unit (zero for
        // the others), adds to the norm's inner products and writes the bf16 operand of the second product;
        // D2 [2d state inputs, 16 slots] += W1 state part x dhid^T accumulates over the position's units in
        // tensor memory. Each kind of product has an issuer warp of its own (a product costs its issuing warp
        // about 70 cycles of instructions: one warp that issued a unit's 12 products between its epilogues was
        // the unit's critical path); the eight compute warps read D1, warp w the columns 32 (w % 4) .. and the
        // slots 4 (w / 4) .. 4 (w / 4) + 3, and go from unit to unit without a block barrier.
        const int n_units = dc_[o_n];
        const int n_chunks = 2 * n_units;
        const uint32_t idesc = umma_idesc_bf16(128, 16);
        auto unit_parity = [&](int i) { return (((i & 1) ? units_odd : units_even) + static_cast<uint32_t>(i >> 1)) & 1u; };
        if (role == 0) {
            if (lane == 0 && cur_t == t) request(units_before, 1 << 30);   // the rest of this position's pieces, each as its slot is handed back
            __syncwarp();
            // This warp arrives at the stage's cluster barrier now and waits for it after the next position's
            // first requests: the last of them waits for this position's last product, and the other warps
            // should not wait for this one on top of that.
            cl.barrier_arrive();
            if (lane == 0) {
                if (t > 0) {
                    // the next position's first two units, as soon as its unit lists are in place (their slots' tenants
                    // are pieces of this position or older: spent before this stage ends)
                    ring_wait(&bar_dec, dec_phase & 1u, c.status, &failed_s);
                    cur_t = t - 1;
                    cur_p = cur_q = 0;
                    request(units_before + static_cast<uint32_t>(n_units), 2);
                }
            }
            __syncwarp();
        } else if (role == 1) {
            fence_async_smem();
            tcgen05_fence_after();
            for (int i = 0; i < n_units; ++i) {
                // D1: tensor memory columns 64 b .. 64 b + 15, b = unit parity; unit i - 2's epilogue has read them
                if (i >= 2) ring_wait(&bar_act[i & 1], unit_parity(i - 2), c.status, &failed_s);
                const uint32_t unit = units_before + static_cast<uint32_t>(i), slot = unit & 1u;
                ring_wait(&full_p[slot], (unit >> 1) & 1u, c.status, &failed_s);
                tcgen05_fence_after();
                const unsigned char* tile = ring + slot * c.w2_bytes;
                if (d == 64)
                    umma_chain_sw128<4>(taddr + 64 * (i & 1), umma_desc_sw128(tile), 0, umma_desc(du_op, 16), umma_kstep(16), idesc, false);
                else
                    umma_chain_fixed<d / 16>(taddr + 64 * (i & 1), umma_desc(tile, 128), umma_desc(du_op, 16), idesc, umma_kstep(128),
                                             umma_kstep(16), false);
                umma_commit(&empty_p[slot]);   // the piece is spent when this product has read it
                umma_commit(&bar_d1[i & 1]);
            }
            tcgen05_fence_before();
        } else if (role == 2) {
            for (int i = 0; i < n_units; ++i) {
                ring_wait(&bar_act[i & 1], unit_parity(i), c.status, &failed_s);
                const uint32_t unit = units_before + static_cast<uint32_t>(i), slot = unit & 1u;
                ring_wait(&full_q[slot], (unit >> 1) & 1u, c.status, &failed_s);
                tcgen05_fence_after();
                const unsigned char* tile = ring_q + slot * slot_bytes;
                // D2 (columns 128 .. 143) accumulates over the position's units
                if (d == 64)   // (two K-blocks of 64 hidden columns, 2d rows each)
                    umma_chain_sw128<8>(taddr + 128, umma_desc_sw128(tile), (128 * 128) >> 4,
                                        umma_desc(b2 + (i & 1) * (kDhidOperand / 2), 16), umma_kstep(16), idesc, i > 0);
                else
                    umma_chain_fixed<8>(taddr + 128, umma_desc(tile, two), umma_desc(b2 + (i & 1) * (kDhidOperand / 2), 16), idesc,
                                        umma_kstep(two), umma_kstep(16), i > 0);
                umma_commit(&empty_q[slot]);
                umma_commit(&bar_sp[i & 1]);
                if (i + 1 == n_units) umma_commit(&bar_d2);
            }
            tcgen05_fence_before();
        } else if (role == 3) {
            // off every critical path: the position's dc and db to memory, the next position's records into their buffer
            for (int e = lane; e < Ks * d; e += 32) {
                const int kl = e / d, x = e - kl * d, k = kl * C + r;
                if (k < K) {
                    c.io.dc[(rt * K + k) * d + x] = dcs[e];
                    c.io.db[(rt * K + k) * d + x] = dbs[e];
                }
            }
            if (lane == 0 && t > 0) prefetch_bulk(t - 1);
            __syncwarp();
        } else if (consumer) {
            const int hc = lane + 32 * (warp & 3), sh = warp >> 2;
            float inner[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                // under the first products, what waits for nothing: the gate's transposed linear on this block's
                // state outputs (the position's dc and db go to memory and the next position's records are
                // requested by the decision warp meanwhile). Before the epilogues on purpose: the copies and the
                // issuer warps get ahead meanwhile and every unit then costs less. (After them, under the last
                // unit's second product, a position of one or two units is 0.9 us shorter and one of four or more
                // longer; choosing by the unit count cost the benchmark's windows 0.15 us a position.)
                for (int e = tid; e < K * gcols; e += kConsumers) {
                    const int k = e >> gshift, il = e - k * gcols;
                    const float sum = dc_[k] >= 0 ? dot_bf16w(dg_all + k * d, 1, gate + il * d, 1, d) : 0.0f;
                    peer(cl, inbox_g, k & cmask)[(k >> cshift) * two + r * gcols + il] = sum;
                }
            }
            for (int i = 0; i < n_units; ++i) {
                const int j = dc_[o_ulist + i];
                const unsigned mask = static_cast<unsigned>(dc_[o_umask + i]);
                const float bias = b1s[j * 128 + hc];
                uint16_t* b2i = b2 + (i & 1) * (kDhidOperand / 2);
                const uint32_t parity = unit_parity(i);
                // (the buffer's previous tenant, unit i - 2: its second product has read it)
                if (i >= 2) ring_wait(&bar_sp[i & 1], parity ^ 1u, c.status, &failed_s);
                ring_wait(&bar_d1[i & 1], parity, c.status, &failed_s);
                tcgen05_fence_after();
                float acc[8];
                tmem_ld8(tmem_addr(taddr, 32 * (warp & 3), 64 * (i & 1)), acc);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int k = 4 * sh + q;
                    float dh = 0.0f;
                    if (mask & (1u << k)) {
                        const float hv = bf16_value(hd[k * 128 + hc]);
                        dh = bf16r((sh ? acc[4 + q] : acc[q]) * gelu_erf_grad(hv));
                        inner[q] += dh * (hv - bias);
                    }
                    b2i[((hc >> 3) * 16 + k) * 8 + (hc & 7)] = bf16_bits(dh);
                }
                fence_async_smem();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_act[i & 1]);   // this warp's part of the operand is written
            }
            BMARK(4);
            // the slots' inner products: every warp's sums, then the four warps of each half in order
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float sum = warp_sum(inner[q]);
                if (lane == 0) red[warp * 4 + q] = sum;
            }
            // the block's partial of dv from the accumulator, to the slots' owners
            if (warp < 4 && 32 * warp < two) {
                float acc[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
                if (n_chunks > 0) {
                    ring_wait(&bar_d2, d2_phase & 1u, c.status, &failed_s);
                    tcgen05_fence_after();
                    tmem_ld8(tmem_addr(taddr, 32 * warp, 128), acc);
                }
                const int i = 32 * warp + lane;
                if (i < two) {
#pragma unroll
                    for (int k = 0; k < kMaxKB; ++k)
                        if (k < K) peer(cl, inbox_dv, k & cmask)[(r * Ks + (k >> cshift)) * two + i] = acc[k];
                }
            }
            tcgen05_fence_before();
            consumer_sync();
            if (tid < K) {
                const int k = tid, half = k >> 2, q = k & 3;
                const float* part = red + (4 * half) * 4 + q;   // warps 4 half .. 4 half + 3
                const float sum = (part[0] + part[4]) + (part[8] + part[12]);
                peer(cl, inbox_sig, k & cmask)[r * Ks + (k >> cshift)] = sum;
            }
        }
        units_before += static_cast<uint32_t>(n_units);
        units_even += static_cast<uint32_t>((n_units + 1) >> 1);
        units_odd += static_cast<uint32_t>(n_units >> 1);
        if (n_chunks > 0) ++d2_phase;
        if (t > 0) ++dec_phase;
#ifdef HSNW_TRACE
        if (!consumer && lane == 0 && row == 0 && t == T / 2) {
            unsigned long long now;
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");
            trace_s[16 + role] = now;   // when the producer and the issuers reach the barrier
        }
#endif
        BMARK(5);
        if (role == 0) cl.barrier_wait();   // 2 (the producer warp arrived above)
        else cl.sync();
        BMARK(6);
        // ---------------- T1: the owners' slots
        if (consumer) {
            if (tid < Ks) {
                const int kl = tid;
                float sigma = sig_gate[kl];
                for (int p = 0; p < C; ++p) sigma += inbox_sig[p * Ks + kl];
                const float rm = rc[7 * Ks * d + kl];
                back[kl] = rm * rm / static_cast<float>(4 * d) * sigma;
            }
            consumer_sync();
            for (int e = tid; e < Ks * two; e += kConsumers) {
                const int kl = e / two, i = e - kl * two, k = kl * C + r;
                float out = 0.0f;
                if (k < K && dc_[k] >= 0) {
                    float sum = 0.0f;
                    for (int p = 0; p < C; ++p) sum += inbox_dv[(p * Ks + kl) * two + i];
                    sum += inbox_g[kl * two + i];
                    const float state = i < d ? rc[(2 * Ks + kl) * d + i] : rc[(5 * Ks + kl) * d + i - d];
                    out = rc[7 * Ks * d + kl] * (norm_w[i] * sum) - back[kl] * state;
                }
                ds[e] = out;
            }
            consumer_sync();
            for (int e = tid; e < Ks * d; e += kConsumers) {
                const int kl = e / d, i = e - kl * d, k = kl * C + r;
                if (k >= K) continue;
                const float dvm = dot_bf16w(ds + kl * two + d, 1, vt + i * d, 1, d), own_ds = ds[kl * two + i];
                for (int p = 0; p < C; ++p) {
                    peer(cl, dvm_all, p)[k * d + i] = dvm;
                    peer(cl, ds_all, p)[k * d + i] = own_ds;
                }
            }
        }
        BMARK(7);
        cl.sync();   // 3
        BMARK(8);
        if (consumer) {
            // ---------------- T2: this block's cells; thread (x, g) takes the targets n = g (mod groups)
            {
                const int x = tid % d, g = tid / d, groups = kConsumers / d;
                const int n_own = dc_[o_own_n];
                for (int e = 0; e < n_own; ++e) {
                    const int u = dc_[o_own + e];
                    const int n = u < K ? dc_[u] : dc_[o_tgt + u - K];
                    if ((n & (groups - 1)) != g) continue;   // groups is a power of two
                    const float add = u < K ? ds_all[u * d + x] : ew[u - K] * dvm_all[div_D(max(u - K, 0)) * d + x];
                    A_s[(n - cell0) * d + x] += add;
                }
                if (tid < d) R_s[tid] = cut ? 0.0f : Rs[tid] + q[d + tid];
            }
            if (cut) {
                consumer_sync();
                for (int e = tid; e < Nc * d; e += kConsumers) A_s[e] = 0.0f;
            }
        }
        BMARK(9);
        cl.sync();   // 4
        BMARK(10);
    }
    {
        float* A = c.io.A + (static_cast<int64_t>(row) * N + cell0) * d;
        for (int e = tid; e < Nc * d; e += kConsumers) A[e] = A_s[e];
        if (r == 0)
            for (int x = tid; x < d; x += kConsumers) c.io.R[static_cast<int64_t>(row) * d + x] = R_s[x];
    }
    tcgen05_fence_before();
    __syncthreads();
#ifdef HSNW_TRACE
    if (row == 0 && tid < 32 && c.trace) c.trace[r * 32 + tid] = trace_s[tid];
#endif
    if (warp == 0) tmem_dealloc(taddr, 256);
}

}  // namespace

static bool rows_bwd_shape(const HsnwModel& m, RowsBwdCtx* c) {
    if (!m.prod_bf16 || m.phases_only || !m.rows_bank_bw) return false;
    if (m.H % 128) return false;
    const int C = m.H / 128;
    if (C != 1 && C != 2 && C != 4 && C != 8) return false;
    if (m.N % C || m.N / C < 2 || (2 * m.d) % C || kConsumers % (2 * m.d / C)) return false;
    if (m.d != 16 && m.d != 32 && m.d != 64) return false;
    if (m.K > kMaxKB || m.M > kMaxMB || m.K < 1 || m.K * m.D > 96 || m.K * (2 * m.d / C) > kConsumers) return false;
    c->C = C;
    c->Nc = m.N / C;
    c->Ks = (m.K + C - 1) / C;
    c->w2_bytes = static_cast<uint32_t>(256 * m.d);
    c->bank_bytes = static_cast<uint32_t>(768 * m.d);
    return true;
}

int hsnw_rows_backward(const HsnwModel* model, const HsnwBackward* io, int* status, cudaStream_t stream) {
    RowsBwdCtx c;
    if (io->full_cut || !rows_bwd_shape(*model, &c)) return HSNW_DECLINED;
    const RowsBwdSmem L = rows_bwd_smem(*model, c.C, c.bank_bytes - c.w2_bytes);
    if (L.total + 1024 > hsnw_max_shared()) return HSNW_DECLINED;
    c.m = *model;
    c.io = *io;
    c.status = status;
    // the phase timestamps of HSNW_TRACE builds follow the status area, when the scratch has the room
    c.trace = (io->scratch && io->scratch_bytes >= 256 + static_cast<int64_t>(c.C) * 32 * 8)
        ? reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(io->scratch) + 256) : nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(io->B) * c.C, 1, 1);
    cfg.blockDim = dim3(kRowThreadsB, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(c.C);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void (*kernel)(RowsBwdCtx) = model->d == 64 ? k_rows_bwd<64> : model->d == 32 ? k_rows_bwd<32> : k_rows_bwd<16>;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        return HSNW_DECLINED;
    }
    hsnw_profile_mark(HSNW_K_ROWS_BWD, stream);
    if (cudaLaunchKernelEx(&cfg, kernel, c) != cudaSuccess) return hsnw_check_launch("window_backward (row clusters)");
    return hsnw_check_launch("window_backward (row clusters)");
}

void hsnw_rows_bwd_set_attributes() {
    if (!hsnw_opt_in(reinterpret_cast<const void*>(k_rows_bwd<64>), "rows_bwd<64>")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_rows_bwd<32>), "rows_bwd<32>")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_rows_bwd<16>), "rows_bwd<16>"))
        hsnw_attribute_failed();
}
