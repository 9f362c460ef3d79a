// The window's prologue on the device: from the token and context ids of a window to what the forward
// sweep reads per position (reference python/hsn/model/hsn.py:1707-1860 with model.key_address on,
// one address byte, no reader; python/hsn/model/router.py:597-765):
//   z [B,T,d]        = E(byte_emb(x_t)), the encoder's two-layer MLP (python/hsn/model/encoder.py:74-128)
//   ctx [B,T,dc]     = ctx_emb(context id)
//   scalars [B,T,N,S] = budget, round, context id / n_context, the two running averages per cell,
//                       position / unroll, one, and (S = 9) the two address features
//                       sqrt(d) <byte_codes[x], cell_addresses[n]> of the current and the previous byte
//   positions [B,T]  = the session position before each step (hsn.py:347-355)
// Everything here is a function of an id: the encoder's output depends on the byte alone, the address
// feature on (byte, cell). So two small tables are built per call, z_table [V,d] and addr_table [V,N]
// (the weights change between windows, the tables are cheap: V rows), and the window itself is gathers
// and one coalesced write of the scalars, which is what bounds it (HBM writes: 4 N S bytes a row-position).
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "host_util.h"

using namespace hsnw;

namespace {

constexpr int kTableThreads = 256;

// One block per byte value v: z_table[v] = fc2(act(fc1(emb[v]))), addr_table[v][n].
// Dynamic shared memory: d + H floats. A warp per output: its lanes walk the weight row (consecutive
// addresses) and the partial sums meet by shuffles, in a fixed order.
__global__ void __launch_bounds__(kTableThreads) k_pro_tables(HsnwPrologue p, float* z_table, float* addr_table) {
    extern __shared__ __align__(16) unsigned char dyn[];
    float* x = reinterpret_cast<float*>(dyn);   // [d]  the byte's embedding
    float* hid = x + p.d;                        // [H]
    const int v = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int kWarps = kTableThreads / 32;
    const bool bf = p.prod_bf16 != 0;
    for (int i = tid; i < p.d; i += kTableThreads) x[i] = maybe_bf16(p.byte_emb[static_cast<int64_t>(v) * p.d + i], bf);
    __syncthreads();
    // (four outputs a round: the rows' loads, each a trip to L2, are in flight together)
    for (int h0 = 4 * warp; h0 < p.H; h0 += 4 * kWarps) {
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int i = lane; i < p.d; i += 32) {
            float w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = h0 + u < p.H ? p.enc_w1[static_cast<int64_t>(h0 + u) * p.d + i] : 0.0f;   // [out, in]
#pragma unroll
            for (int u = 0; u < 4; ++u) sum[u] += x[i] * maybe_bf16(w[u], bf);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] = warp_sum(sum[u]);
        if (lane < 4 && h0 + lane < p.H) {
            const float mine = lane == 0 ? sum[0] : lane == 1 ? sum[1] : lane == 2 ? sum[2] : sum[3];
            const float pre = maybe_bf16(mine + maybe_bf16(p.enc_b1[h0 + lane], bf), bf);
            hid[h0 + lane] = maybe_bf16(gelu_erf(pre), bf);
        }
    }
    __syncthreads();
    for (int o0 = 4 * warp; o0 < p.d; o0 += 4 * kWarps) {
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int h = lane; h < p.H; h += 32) {
            float w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = o0 + u < p.d ? p.enc_w2[static_cast<int64_t>(o0 + u) * p.H + h] : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) sum[u] += hid[h] * maybe_bf16(w[u], bf);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] = warp_sum(sum[u]);
        if (lane < 4 && o0 + lane < p.d) {
            const float mine = lane == 0 ? sum[0] : lane == 1 ? sum[1] : lane == 2 ? sum[2] : sum[3];
            z_table[static_cast<int64_t>(v) * p.d + o0 + lane] = maybe_bf16(mine + maybe_bf16(p.enc_b2[o0 + lane], bf), bf);
        }
    }
    if (addr_table) {   // float32 whatever the products' precision: the reference takes these outside autocast
        const float root = sqrtf(static_cast<float>(p.d));
        const float* code = p.byte_codes + static_cast<int64_t>(v) * p.d;
        for (int n0 = 4 * warp; n0 < p.N; n0 += 4 * kWarps) {
            float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int i = lane; i < p.d; i += 32) {
                float a[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) a[u] = n0 + u < p.N ? p.cell_addresses[static_cast<int64_t>(n0 + u) * p.d + i] : 0.0f;
#pragma unroll
                for (int u = 0; u < 4; ++u) sum[u] += code[i] * a[u];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) sum[u] = warp_sum(sum[u]);
            if (lane < 4 && n0 + lane < p.N) {
                const float mine = lane == 0 ? sum[0] : lane == 1 ? sum[1] : lane == 2 ? sum[2] : sum[3];
                addr_table[static_cast<int64_t>(v) * p.N + n0 + lane] = mine * root;
            }
        }
    }
}

// One block per row: the position before each step (t - s after the row's last reset s <= t, else the
// carried position + t: a running maximum of the reset indices) and the byte before each position.
__global__ void __launch_bounds__(256) k_pro_positions(HsnwPrologue p, int64_t* positions, int32_t* previous) {
    __shared__ int warp_top[8];
    __shared__ int carried_s;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t base = static_cast<int64_t>(b) * p.T;
    const int64_t start = p.pos0[b];
    if (tid == 0) carried_s = -1;
    __syncthreads();
    for (int t0 = 0; t0 < p.T; t0 += 256) {
        const int t = t0 + tid;
        const bool in = t < p.T;
        const bool cut = in && p.reset[base + t] != 0;
        int last = cut ? t : -1;
#pragma unroll
        for (int w = 1; w < 32; w <<= 1) {   // the running maximum inside the warp
            const int other = __shfl_up_sync(0xffffffffu, last, w);
            if (lane >= w) last = max(last, other);
        }
        if (lane == 31) warp_top[warp] = last;
        __syncthreads();
        int before = carried_s;
        for (int w = 0; w < warp; ++w) before = max(before, warp_top[w]);
        last = max(last, before);
        if (in) {
            positions[base + t] = last >= 0 ? t - last : start + t;
            const int32_t prior = t > 0 ? static_cast<int32_t>(p.tokens[base + t - 1])
                                        : (p.prev_tokens ? static_cast<int32_t>(p.prev_tokens[b]) : p.bos);
            previous[base + t] = cut ? p.bos : prior;
        }
        __syncthreads();
        if (tid == 255) carried_s = last;   // the chunk's last thread holds the maximum so far
        __syncthreads();
    }
}

constexpr int kProTile = 1024;   // cells of a row staged in shared memory at a time (36 KB of scalars)

// One block per (row, position): the gathers and the scalars of every cell.
__global__ void k_pro_rows(HsnwPrologue p, const float* z_table, const float* addr_table, const int64_t* positions,
                           const int32_t* previous) {
    const int64_t rt = blockIdx.x;
    const int b = static_cast<int>(rt / p.T);
    const int tid = threadIdx.x, nt = blockDim.x;
    const int token = static_cast<int>(p.tokens[rt]);
    const int ctx_id = static_cast<int>(p.ctx_ids[rt]);
    block_copy_f32(p.z + rt * p.d, z_table + static_cast<int64_t>(token) * p.d, p.d);
    block_copy_f32(p.ctx + rt * p.dc, p.ctx_emb + static_cast<int64_t>(ctx_id) * p.dc, p.dc);
    int64_t pos = positions[rt];
    if (p.position_mode == 1) pos = pos < static_cast<int64_t>(p.unroll) - 1 ? pos : static_cast<int64_t>(p.unroll) - 1;
    else if (p.position_mode == 2) pos = pos % static_cast<int64_t>(p.unroll);
    const float f_ctx = static_cast<float>(ctx_id) / p.n_context;
    const float f_pos = static_cast<float>(pos) / p.unroll;
    const float* util = p.ema_utility + (p.ema_per_row ? static_cast<int64_t>(b) * p.N : 0);
    const float* chosen = p.ema_selected + (p.ema_per_row ? static_cast<int64_t>(b) * p.N : 0);
    const float* cur = addr_table ? addr_table + static_cast<int64_t>(token) * p.N : nullptr;
    const float* prev = addr_table ? addr_table + static_cast<int64_t>(previous[rt]) * p.N : nullptr;
    // A cell's S scalars by the cell's thread into shared memory (one control flow for every lane: a thread per
    // output element took a nine-way divergent branch per element and made the kernel instruction bound), then the
    // row's N S floats to memory as 16-byte stores.
    extern __shared__ __align__(16) unsigned char dyn[];
    float* row_s = reinterpret_cast<float*>(dyn);   // [kProTile][S]: a tile of the row's cells
    float* out = p.scalars + rt * p.N * p.S;
    const bool wide = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    for (int n0 = 0; n0 < p.N; n0 += kProTile) {
        const int cells = min(kProTile, p.N - n0);
        for (int i = tid; i < cells; i += nt) {
            const int n = n0 + i;
            float v[9];
            v[0] = p.budget_frac;
            v[1] = p.round_frac;
            v[2] = f_ctx;
            v[3] = util[n];
            v[4] = chosen[n];
            v[5] = f_pos;
            v[6] = 1.0f;
            v[7] = cur ? cur[n] : 0.0f;
            v[8] = prev ? prev[n] : 0.0f;
#pragma unroll
            for (int s = 0; s < 9; ++s)
                if (s < p.S) row_s[i * p.S + s] = v[s];
        }
        __syncthreads();
        const int total = cells * p.S;
        float* to = out + static_cast<int64_t>(n0) * p.S;   // (kProTile S floats are a multiple of 16 bytes)
        if (wide && (total & 3) == 0) {
            for (int e = tid; e < total >> 2; e += nt) reinterpret_cast<float4*>(to)[e] = reinterpret_cast<const float4*>(row_s)[e];
        } else {
            for (int e = tid; e < total; e += nt) to[e] = row_s[e];
        }
        __syncthreads();
    }
}

size_t table_floats(const HsnwPrologue& p) {
    return static_cast<size_t>(p.V) * p.d + (p.S == 9 ? static_cast<size_t>(p.V) * p.N : 0);
}
size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace

extern "C" int64_t hsnw_prologue_scratch_bytes(const HsnwPrologue* p) {
    if (!p || p->B < 1 || p->T < 1 || p->V < 1) return 0;
    return static_cast<int64_t>(align256(sizeof(float) * table_floats(*p)) + align256(sizeof(int64_t) * p->B * p->T)
                                + align256(sizeof(int32_t) * static_cast<size_t>(p->B) * p->T));
}

extern "C" int hsnw_window_prologue(const HsnwPrologue* p, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (!p) return hsnw_fail(HSNW_E_ARG, "window_prologue: null argument");
    if (p->B < 1 || p->T < 1 || p->V < 2 || p->d < 1 || p->H < 1 || p->dc < 1 || p->N < 1)
        return hsnw_fail(HSNW_E_ARG, "window_prologue: sizes must be positive");
    if (p->S != 7 && p->S != 9)
        return hsnw_fail(HSNW_E_UNSUPPORTED, "window_prologue: 7 scalars, or 9 with the address features of one byte");
    if (!p->byte_emb || !p->enc_w1 || !p->enc_b1 || !p->enc_w2 || !p->enc_b2 || !p->ctx_emb || !p->ema_utility
        || !p->ema_selected || !p->tokens || !p->ctx_ids || !p->reset || !p->pos0 || !p->z || !p->ctx || !p->scalars)
        return hsnw_fail(HSNW_E_ARG, "window_prologue: a required pointer is null");
    if (p->S == 9 && (!p->byte_codes || !p->cell_addresses))
        return hsnw_fail(HSNW_E_ARG, "window_prologue: the address features need byte_codes and cell_addresses");
    if (p->unroll <= 0.0f || p->n_context <= 0.0f || p->bos < 0 || p->bos >= p->V)
        return hsnw_fail(HSNW_E_ARG, "window_prologue: unroll and n_context must be positive, bos a byte value");
    if (!p->scratch || p->scratch_bytes < hsnw_prologue_scratch_bytes(p) || (reinterpret_cast<uintptr_t>(p->scratch) & 255))
        return hsnw_fail(HSNW_E_ARG, "window_prologue: scratch too small or not 256-byte aligned");
    const size_t shared = sizeof(float) * (static_cast<size_t>(p->d) + p->H);
    if (shared > 48 * 1024) return hsnw_fail(HSNW_E_UNSUPPORTED, "window_prologue: d + H beyond 12288");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    unsigned char* base = static_cast<unsigned char*>(p->scratch);
    float* z_table = reinterpret_cast<float*>(base);
    float* addr_table = p->S == 9 ? z_table + static_cast<size_t>(p->V) * p->d : nullptr;
    size_t off = align256(sizeof(float) * table_floats(*p));
    int64_t* positions = p->positions ? p->positions : reinterpret_cast<int64_t*>(base + off);
    off += align256(sizeof(int64_t) * p->B * p->T);
    int32_t* previous = reinterpret_cast<int32_t*>(base + off);
    hsnw_profile_mark(HSNW_K_PROLOGUE, stream);
    k_pro_tables<<<p->V, kTableThreads, shared, stream>>>(*p, z_table, addr_table);
    k_pro_positions<<<p->B, 256, 0, stream>>>(*p, positions, previous);
    const size_t row_bytes = sizeof(float) * static_cast<size_t>(p->N < kProTile ? p->N : kProTile) * p->S;
    k_pro_rows<<<static_cast<unsigned>(static_cast<int64_t>(p->B) * p->T), 256, row_bytes, stream>>>(*p, z_table, addr_table, positions, previous);
    return hsnw_check_launch("window_prologue");
}
