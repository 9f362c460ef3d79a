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

using namespace hsnw;

namespace {

constexpr int kSlice = 64;
constexpr int kPairTile = 256;
constexpr int kPairBatch = 8;

struct BwdCtx {
    HsnwModel m;
    HsnwBackward io;
    int nHS;
    float* d_unit;    // [P, d]   W_out^T dy
    float* dg;        // [P, d]   the gate's pre-activation cotangent
    float* sig_gate;  // [P]      <gate_pre - b_g, dg>
    float* part_dv;   // [nHS, P, 2d]
    float* part_sig;  // [nHS, P]
    int* pair_unit;   // [P]  -1 on padded slots
};

// ------------------------------------------------------------------------------------------------
// head. Shared (dynamic): Rs [d], cell_of [K], rho [K], dot [K], dy [K d], ysv [K d], wo [d (d+1)].
// ------------------------------------------------------------------------------------------------
__global__ void k_head(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const int N = c.m.N, d = c.m.d, K = c.m.K, T = c.io.T;
    const bool full = c.io.full_cut != 0;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, warps = nt >> 5;
    float* Rs = reinterpret_cast<float*>(dyn);
    int* cell_of = reinterpret_cast<int*>(Rs + d);
    float* rho = reinterpret_cast<float*>(cell_of + K);
    float* dot = rho + K;
    float* sg = dot + K;
    float* dzs = sg + K;          // [K d]  cand_w * dz
    float* ysv = dzs + K * d;     // [K d]
    float* wo = ysv + K * d;      // [d][d+1]
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    float* A = c.io.A + static_cast<int64_t>(row) * N * d;
    float* R = c.io.R + static_cast<int64_t>(row) * d;
    const int64_t* cells = c.io.cells + rt * K;
    const uint8_t* valid = c.io.valid + rt * K;
    const int64_t o0 = rt * K * d;
    if (!full)
        for (int e = tid; e < d * d; e += nt) wo[(e / d) * (d + 1) + (e % d)] = c.m.wout_t[e];
    for (int x = tid; x < d; x += nt) {
        float r = R[x];
        if (c.io.d_q_post) r += c.io.d_q_post[rt * d + x];
        Rs[x] = r;
    }
    for (int k = tid; k < K; k += nt) cell_of[k] = valid[k] ? static_cast<int>(cells[k]) : -1;
    __syncthreads();
    const float n_f = static_cast<float>(N);
    for (int e = tid; e < K * d; e += nt) {
        const int k = e / d, x = e - k * d;
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
            c.dg[(static_cast<int64_t>(row) * K + k) * d + x] = dgv;
            // the gate's share of the inner product is folded per slot below
            c.d_unit[(static_cast<int64_t>(row) * K + k) * d + x] = sgv;  // staged, overwritten below
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
    // per slot: rho = rsqrt(mean(y^2) + eps), dot = mean(y * cand_w * dz), sigma_gate; a warp each
    for (int k = warp; k < K; k += warps) {
        float sq = 0.0f, dt = 0.0f, s = 0.0f;
        for (int x = lane; x < d; x += 32) {
            const float yv = ysv[k * d + x];
            sq += yv * yv;
            dt += yv * dzs[k * d + x];
            s += c.d_unit[(static_cast<int64_t>(row) * K + k) * d + x];
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
        const int k = e / d;
        const float r = rho[k];
        dzs[e] = cell_of[k] >= 0 ? r * dzs[e] - r * r * r * ysv[e] * dot[k] : 0.0f;
    }
    __syncthreads();
    // d_unit = dy W_out (the transposed output projection): y[x] = sum_i F[i] wout_t[i][x]
    for (int e = tid; e < K * d; e += nt) {
        const int k = e / d, i = e - k * d;
        float sum = 0.0f;
        for (int x = 0; x < d; ++x) sum += dzs[k * d + x] * wo[i * (d + 1) + x];
        c.d_unit[(static_cast<int64_t>(row) * K + k) * d + i] = sum;
    }
    for (int k = tid; k < K; k += nt)
        c.pair_unit[static_cast<int64_t>(row) * K + k] = cell_of[k] >= 0 ? static_cast<int>(c.io.units[rt * K + k]) : -1;
}

// ------------------------------------------------------------------------------------------------
// mid: blockIdx.x = (unit j, slice s), blockIdx.y = pair tile. 256 threads.
// Shared (dynamic): w2 [64][d+1], w1 [2d][65], du [8][d], dh [8][64], list [256].
// ------------------------------------------------------------------------------------------------
__global__ void k_mid(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ int warp_count[8];
    __shared__ int n_list;
    const int d = c.m.d, K = c.m.K, H = c.m.H, in = 4 * c.m.d, two = 2 * c.m.d;
    const int P = c.io.B * K, T = c.io.T;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = blockIdx.x / c.nHS, s = blockIdx.x - j * c.nHS;
    const int c0 = s * kSlice;
    const int cols = min(kSlice, H - c0);
    float* w2 = reinterpret_cast<float*>(dyn);          // [64][d+1]
    float* w1 = w2 + kSlice * (d + 1);                  // [2d][65]
    float* du = w1 + two * (kSlice + 1);                // [8][d]
    float* dh = du + kPairBatch * d;                    // [8][64]
    float* hm = dh + kPairBatch * kSlice;               // [8][64]  hid - b1
    int* list = reinterpret_cast<int*>(hm + kPairBatch * kSlice);
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
    const float* W1 = c.m.w1 + static_cast<int64_t>(j) * in * H;
    const float* W2 = c.m.w2 + static_cast<int64_t>(j) * H * d;
    for (int e = tid; e < kSlice * d; e += blockDim.x) {
        const int cc = e / d, x = e - cc * d;
        w2[cc * (d + 1) + x] = cc < cols ? W2[static_cast<int64_t>(c0 + cc) * d + x] : 0.0f;
    }
    for (int e = tid; e < two * kSlice; e += blockDim.x) {
        const int i = e >> 6, cc = e & 63;
        w1[i * (kSlice + 1) + cc] = cc < cols ? W1[static_cast<int64_t>(two + i) * H + c0 + cc] : 0.0f;
    }
    const int cc = tid & 63, pg = tid >> 6;
    for (int base = 0; base < count; base += kPairBatch) {
        const int nb = min(kPairBatch, count - base);
        __syncthreads();
        for (int e = tid; e < nb * d; e += blockDim.x) {
            const int pb = e / d, x = e - pb * d;
            du[e] = c.d_unit[static_cast<int64_t>(list[base + pb]) * d + x];
        }
        __syncthreads();
        // the transposed second layer and the activation's derivative
        for (int half = 0; half < 2; ++half) {
            const int pb = pg + 4 * half;
            float dhid = 0.0f, centred = 0.0f;
            if (pb < nb && cc < cols) {
                float sum = 0.0f;
                for (int x = 0; x < d; ++x) sum += du[pb * d + x] * w2[cc * (d + 1) + x];
                const int p = list[base + pb];
                const int row = p / K, k = p - row * K;
                const float hid = c.io.hidden[((static_cast<int64_t>(row) * T + t) * K + k) * H + c0 + cc];
                dhid = sum * gelu_erf_grad(hid);
                centred = hid - c.m.b1[j * H + c0 + cc];
            }
            dh[pb * kSlice + cc] = dhid;
            hm[pb * kSlice + cc] = dhid * centred;
        }
        __syncthreads();
        // the unit's part of the norm's inner product: a warp per pair
        if (warp < nb) {
            float sum = hm[warp * kSlice + lane] + hm[warp * kSlice + lane + 32];
            sum = warp_sum(sum);
            if (lane == 0) c.part_sig[static_cast<int64_t>(s) * P + list[base + warp]] = sum;
        }
        // the transposed first layer on the state columns [h ; m] of the cell input
        for (int e = tid; e < nb * two; e += blockDim.x) {
            const int pb = e / two, i = e - pb * two;
            float sum = 0.0f;
            for (int k2 = 0; k2 < kSlice; ++k2) sum += dh[pb * kSlice + k2] * w1[i * (kSlice + 1) + k2];
            c.part_dv[(static_cast<int64_t>(s) * P + list[base + pb]) * two + i] = sum;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// tail. Shared (dynamic): cell_of [K], back [K], dv [K 2d], dvm [K d], vt [d (d+1)].
// ------------------------------------------------------------------------------------------------
__global__ void k_tail(BwdCtx c, int t) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const int N = c.m.N, d = c.m.d, K = c.m.K, D = c.m.D, T = c.io.T, two = 2 * c.m.d;
    const int P = c.io.B * K;
    const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    int* cell_of = reinterpret_cast<int*>(dyn);
    float* back = reinterpret_cast<float*>(cell_of + K);  // [K] (rms^2 / n) sigma
    float* ds = back + K;        // [K][2d]
    float* dvm = ds + K * two;   // [K][d]
    float* vt = dvm + K * d;     // [d][d+1]
    const int64_t rt = static_cast<int64_t>(row) * T + t;
    const int64_t pair0 = static_cast<int64_t>(row) * K;
    float* A = c.io.A + static_cast<int64_t>(row) * N * d;
    float* R = c.io.R + static_cast<int64_t>(row) * d;
    const float in_dim = static_cast<float>(4 * d);
    for (int e = tid; e < d * d; e += nt) vt[(e / d) * (d + 1) + (e % d)] = c.m.v_t[e];
    for (int k = tid; k < K; k += nt) {
        const bool ok = c.io.valid[rt * K + k] != 0;
        cell_of[k] = ok ? static_cast<int>(c.io.cells[rt * K + k]) : -1;
        float sigma = c.sig_gate[pair0 + k];
        if (ok)
            for (int s = 0; s < c.nHS; ++s) sigma += c.part_sig[static_cast<int64_t>(s) * P + pair0 + k];
        const float r = c.io.rms[rt * K + k];
        back[k] = r * r / in_dim * sigma;
    }
    __syncthreads();
    // ds = rms (g_n dv) - (rms^2 / n) sigma [h_old ; m] on the state columns
    for (int e = tid; e < K * two; e += nt) {
        const int k = e / two, i = e - k * two;
        float out = 0.0f;
        if (cell_of[k] >= 0) {
            float dv = 0.0f;
            for (int s = 0; s < c.nHS; ++s) dv += c.part_dv[(static_cast<int64_t>(s) * P + pair0 + k) * two + i];
            // the gate's transposed linear: gate_pre[x] = sum_j v[j] gate_t[j][x]
            const float* g_row = c.m.gate_t + static_cast<int64_t>(two + i) * d;
            const float* dg = c.dg + (pair0 + k) * d;
            float gsum = 0.0f;
            for (int x = 0; x < d; ++x) gsum += dg[x] * g_row[x];
            dv += gsum;
            const float state = i < d ? c.io.h_old[(rt * K + k) * d + i] : c.io.m[(rt * K + k) * d + i - d];
            out = c.io.rms[rt * K + k] * (c.m.norm_w[two + i] * dv) - back[k] * state;
        }
        ds[e] = out;
    }
    __syncthreads();
    // dvm = dm V: m = sum_e a_e (V h_src), (V h)[x] = sum_i h[i] v_t[i][x]
    for (int e = tid; e < K * d; e += nt) {
        const int k = e / d, i = e - k * d;
        float sum = 0.0f;
        for (int x = 0; x < d; ++x) sum += ds[k * two + d + x] * vt[i * (d + 1) + x];
        dvm[e] = sum;
    }
    __syncthreads();
    // a thread owns a column x of the row's A: its own cells first, then every edge in slot order
    const bool cut = c.io.reset[rt] != 0;
    for (int x = tid; x < d; x += nt) {
        for (int k = 0; k < K; ++k) {
            const int n = cell_of[k];
            if (n >= 0) A[static_cast<int64_t>(n) * d + x] += ds[k * two + x];
        }
        for (int k = 0; k < K; ++k) {
            const int n = cell_of[k];
            if (n < 0) continue;
            for (int j = 0; j < D; ++j) {
                const int srcc = c.m.pad_src[n * D + j];
                A[static_cast<int64_t>(srcc) * d + x] += c.m.edge_w[n * D + j] * dvm[k * d + x];
            }
        }
        float r = R[x];
        if (c.io.d_q_pre) r += c.io.d_q_pre[rt * d + x];
        R[x] = cut ? 0.0f : r;
    }
    if (cut) {
        __syncthreads();
        for (int e = tid; e < N * d; e += nt) A[e] = 0.0f;
    }
}

size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
struct Layout {
    size_t d_unit, dg, sig_gate, part_dv, part_sig, pair_unit, total;
};
Layout layout(const HsnwModel& m, int B) {
    Layout L;
    const size_t P = static_cast<size_t>(B) * m.K;
    const int nHS = (m.H + kSlice - 1) / kSlice;
    size_t off = 0;
    L.d_unit = off; off += align_up(sizeof(float) * P * m.d);
    L.dg = off; off += align_up(sizeof(float) * P * m.d);
    L.sig_gate = off; off += align_up(sizeof(float) * P);
    L.part_dv = off; off += align_up(sizeof(float) * nHS * P * 2 * m.d);
    L.part_sig = off; off += align_up(sizeof(float) * nHS * P);
    L.pair_unit = off; off += align_up(sizeof(int) * P);
    L.total = off;
    return L;
}
size_t head_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(m.d) + 4 * m.K + 2 * static_cast<size_t>(m.K) * m.d
        + static_cast<size_t>(m.d) * (m.d + 1));
}
size_t mid_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(kSlice) * (m.d + 1) + static_cast<size_t>(2) * m.d * (kSlice + 1)
        + static_cast<size_t>(kPairBatch) * m.d + 2 * kPairBatch * kSlice + kPairTile);
}
size_t tail_shared(const HsnwModel& m) {
    return sizeof(float) * (static_cast<size_t>(2) * m.K + 3 * static_cast<size_t>(m.K) * m.d
        + static_cast<size_t>(m.d) * (m.d + 1));
}

}  // namespace

extern "C" int64_t hsnw_backward_scratch_bytes(const HsnwModel* model, int32_t B, int32_t T) {
    (void)T;
    if (!model || B < 1) return 0;
    return static_cast<int64_t>(layout(*model, B).total);
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
    const size_t cap = hsnw_max_shared();
    if (head_shared(m) > cap || (!full && (mid_shared(m) > cap || tail_shared(m) > cap)))
        return hsnw_fail(HSNW_E_UNSUPPORTED, "window_backward: a phase's working set exceeds a block's shared memory");
    const Layout L = layout(m, io->B);
    if (!full && (!io->scratch || io->scratch_bytes < static_cast<int64_t>(L.total)
        || (reinterpret_cast<uintptr_t>(io->scratch) & 255)))
        return hsnw_fail(HSNW_E_ARG, "window_backward: scratch too small or not 256-byte aligned");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    BwdCtx c;
    c.m = m;
    c.io = *io;
    c.nHS = (m.H + kSlice - 1) / kSlice;
    unsigned char* base = static_cast<unsigned char*>(io->scratch);
    c.d_unit = full ? nullptr : reinterpret_cast<float*>(base + L.d_unit);
    c.dg = full ? nullptr : reinterpret_cast<float*>(base + L.dg);
    c.sig_gate = full ? nullptr : reinterpret_cast<float*>(base + L.sig_gate);
    c.part_dv = full ? nullptr : reinterpret_cast<float*>(base + L.part_dv);
    c.part_sig = full ? nullptr : reinterpret_cast<float*>(base + L.part_sig);
    c.pair_unit = full ? nullptr : reinterpret_cast<int*>(base + L.pair_unit);
    const int B = io->B, T = io->T;
    const dim3 mid_grid(m.M * c.nHS, (B * m.K + kPairTile - 1) / kPairTile);
    const size_t sh_head = head_shared(m), sh_mid = mid_shared(m), sh_tail = tail_shared(m);
    for (int t = T - 1; t >= 0; --t) {
        k_head<<<B, 256, sh_head, stream>>>(c, t);
        if (full) continue;
        k_mid<<<mid_grid, 256, sh_mid, stream>>>(c, t);
        k_tail<<<B, 256, sh_tail, stream>>>(c, t);
    }
    return hsnw_check_launch("window_backward");
}

void hsnw_backward_set_attributes() {
    const struct { const void* f; const char* n; } ks[] = {
        {reinterpret_cast<const void*>(k_head), "head"}, {reinterpret_cast<const void*>(k_mid), "mid"},
        {reinterpret_cast<const void*>(k_tail), "tail"}};
    for (const auto& k : ks)
        if (!hsnw_opt_in(k.f, k.n)) hsnw_attribute_failed();
}
