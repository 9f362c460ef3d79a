// The forward sweep of a window as ONE persistent kernel: a thread-block cluster per batch row
// walks the row's T positions with the row's state resident in the cluster's shared memory.
//
// Why: at a few dozen rows per GPU the batch-synchronous phases (window_fwd.cu) are bound by the
// latency of 4 launches and ~20 dependent trips to L2 per position. Rows are independent in the
// forward sweep, so a row can run alone: its state (h, V h, the state's part of the logits, ages,
// the cell graph) lives in distributed shared memory for the whole window, the phases of a position
// are separated by 4 hardware cluster barriers instead of kernel boundaries, and the only traffic
// per position is the unit bank streamed from L2 by the TMA (bulk copies through a ring, issued by
// a producer warp), the position's inputs (bulk copies, a position ahead) and the tape's records
// written back.
//
// Cluster of C = H / 128 blocks; block r owns the cells [r N/C, (r+1) N/C), the hidden columns
// [128 r, 128 r + 128) of every unit (two 64-column chunks), the columns [256 r, 256 r + 256) of
// the merged front first layer, the rows [r 4d/C, (r+1) 4d/C) of the gate's input, and the slots
// k = r (mod C) at the update. Per position:
//   A  front MLPs on the block's columns -> partial (u, z_hat) pushed to every block   | sync 1
//   B  u, eps, the scorer on the block's cells (4 threads a cell) -> (score, unit, age) pushed
//      to every block                                                                  | sync 2
//   C  the decision in every block on identical inputs: a cell's place in the scored order is the
//      number of larger keys, counted by the cell's thread against all keys; the budget, the
//      threshold and the probes by one warp
//   D  gather of the selected rows and message sources through distributed shared memory,
//      messages, cell norm -> the slots' inputs as a bf16 tensor-core operand; then per streamed
//      chunk (unit, 64 columns) two tcgen05 products with accumulators in tensor memory: the first
//      layer (its epilogue adds the bias, rounds, records, applies the activation for the slots
//      that chose the unit), the second layer accumulating over all the position's chunks; four
//      warps run the epilogues, the other four the gate's partial sums meanwhile; partial F and
//      gate pushed to the slots' owners                                                | sync 3
//   E  W_out, candidate norm, tanh, sigmoid, the gated write pushed to the cell's owner, the
//      slot's change of the summary pushed everywhere                                  | sync 4
//   F  summary, ages, the written cells' derived state (logit parts, V h) to their owners, the
//      tape's next record from the block's cells, the next reset.
//
// The arithmetic, the rounding points (bf16 operands and outputs of every product, fp32 sums and
// state) and every output are those of window_fwd.cu (reference: python/hsn/train/compile.py:
// 1117-1193, python/hsn/model/hsn.py:1903-1980, python/hsn/model/cell.py:349-505); only the order
// of fp32 partial sums differs. Fixed orders everywhere: no atomics on values (one shared-memory
// atomicMax on a maximum, which no order can change).
//
// Every mbarrier wait is bounded (rows.cuh: ring_wait) and reports through the status word; the
// cluster barriers are hardware barriers that every thread of the cluster reaches the same number
// of times (all control flow around them depends on values that are identical in the cluster).
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "select.cuh"
#include "stage.cuh"
#include "host_util.h"
#include "rows.cuh"
#include "umma.cuh"

#include <type_traits>

using namespace hsnw;

namespace {

constexpr int kRowThreads = 384;      // + the producer warp (copies, records) and three issuer warps (tensor-core products)
constexpr int kMaxStages = 3;         // ring depth (2 when 3 slots do not fit beside a large state)
constexpr int kMaxK = 8;              // slots (register accumulators per slot)
constexpr int kMaxMR = 16;            // units
constexpr int kFrontCols = 256;       // merged front columns per block (2H / C with H = 128 C)
constexpr int kActOperand = 2 * 16 * 16 * 8;   // bytes of a unit's activations as a bf16 operand [128 / 8][16 slots][8]

struct RowsCtx {
    HsnwModel m;
    HsnwForward io;
    int C, Nc, Ks;            // blocks of a cluster, cells a block owns, slots a block owns (ceil(K / C))
    int gate_rows;            // 4d / C
    uint32_t bank_bytes;      // a unit's weights on the block's 128 hidden columns: three pieces, W1 (inputs 0..2d), W1 (2d..4d), W2
    uint32_t w1_bytes;        // one W1 piece (= the ring slot); the W2 piece is half of it
    uint32_t front_bytes;     // one front chunk
    uint32_t slot_bytes;      // ring slot
    uint32_t stages;          // ring depth
    const float* pre_s;       // [B*T, H]
    int* status;
};

__host__ __device__ inline size_t up16(size_t v) { return (v + 15) & ~static_cast<size_t>(15); }

// Offsets (bytes) of the dynamic shared memory's segments.
struct RowsSmem {
    size_t ring, h, vh, lh, age, cmax, wout, vt, gate, swh, sw_head, sw_tail, norm_w, cand_w, fb2, gate_b, score_b,
        fb1p, score_all, unit_all, age_all, q, q_after, ue, rowterm, hold, big, msg, rms, graph, b2, gacc, inbox_front,
        inbox_f, inbox_delta, in_scal, in_pre, in_z, upd, cell_of, unit_of, ulist, umask, cand, total;
};
__host__ __device__ inline RowsSmem rows_smem(const HsnwModel& m, int C, uint32_t slot_bytes, uint32_t stages) {
    RowsSmem L;
    const size_t d = m.d, N = m.N, K = m.K, M = m.M, D = m.D, S = m.S, Nc = N / C, Ks = (K + C - 1) / C;
    size_t o = 0;
    auto take = [&o](size_t bytes) {
        const size_t at = o;
        o += up16(bytes);
        return at;
    };
    L.ring = take(static_cast<size_t>(stages) * slot_bytes + 1024);   // + room to start on a 1024-byte boundary (swizzled tiles)
    L.h = take(4 * Nc * d);
    L.vh = take(2 * Nc * d);            // bf16: the values are bf16 in this mode
    L.lh = take(4 * Nc * M);
    L.age = take(8 * Nc);
    L.cmax = take(4 * Nc);
    L.wout = take(2 * d * d);           // bf16
    L.vt = take(2 * d * d);             // bf16
    L.gate = take(2 * (4 * d / C) * d); // bf16, the block's input rows
    L.swh = take(4 * d * M);
    L.sw_head = take(4 * 2 * d * M);
    L.sw_tail = take(4 * (1 + S) * M);
    L.norm_w = take(4 * 4 * d);
    L.cand_w = take(4 * d);
    L.fb2 = take(4 * 2 * d);
    L.gate_b = take(4 * d);
    L.score_b = take(4 * 2 * kMaxMR);   // score_b, then cost
    L.fb1p = take(4 * kFrontCols);      // the predictor's first-layer bias on the block's columns
    L.score_all = take(4 * N);
    L.unit_all = take(4 * N);
    L.age_all = take(8 * N);
    L.q = take(4 * d);
    L.q_after = take(4 * d);            // the summary after the position, before the next reset (for the tape)
    L.ue = take(4 * 2 * d);
    L.rowterm = take(4 * kMaxMR);
    L.hold = take(4 * K * d);           // the selected cells' rows
    {
        // sources [K D][d], then the pairs' inputs v [K][4d] over them; the front's act [256] and
        // partial sums [256 / d][2d] use the same bytes in phase A
        size_t big = 4 * K * D * d;
        if (2 * 16 * 4 * d > big) big = 2 * 16 * 4 * d;   // the pairs' inputs as a bf16 operand [4d/8][16][8]
        if (4 * (kFrontCols + 2 * kFrontCols) > big) big = 4 * 3 * kFrontCols;
        L.big = take(big);
    }
    L.msg = take(4 * K * d);
    L.rms = take(4 * K);
    L.graph = take(4 * N * D);          // every cell's sources and edge weights: (source << 16) | bf16 weight
    L.gacc = take(4 * (K * d > Nc * M ? K * d : Nc * M));   // phase D: the gate's partial sums; phases A-B: the cells' part of the logits
    L.inbox_front = take(4 * C * (2 * d + 4));
    L.inbox_f = take(4 * C * Ks * 2 * d);
    L.in_scal = take(4 * Nc * S + 16);
    L.in_pre = take(4 * kFrontCols);
    L.in_z = take(4 * d);
    L.upd = take(4 * Ks * 6 * d + 4 * Ks);  // F, gate_pre, y, -, hb per owned slot
    L.cell_of = take(4 * K);
    L.unit_of = take(4 * K);
    L.ulist = take(4 * (kMaxMR + 4));
    L.umask = take(4 * (kMaxMR + 4));
    // phase C's keys ([N] then [8] stale counts per warp and [K] flags) and phase E/F's inbox of the
    // slots' changes are adjacent: phase D's two activation operands (bf16 [16][16][8] each, 8 KB) use
    // the same bytes between them (C is over when D starts; E's stores come after the barrier that
    // ends D)
    L.cand = take(8 * N + 64);
    L.inbox_delta = take(4 * K * d);
    L.b2 = L.cand;
    if (L.inbox_delta + up16(4 * K * d) - L.cand < 2 * kActOperand) o = L.cand + 2 * kActOperand;
    L.total = o;
    return L;
}

// Optional phase timestamps for tuning (-DHSNW_TRACE): thread 0 of row 0's blocks, at the middle
// position, event i of block r at trace[r * 32 + i] (cycles of the SM's clock: reading the global timer takes about a microsecond, which back-to-back marks would show as phase time); the trace
// area follows the status word.
#ifdef HSNW_TRACE
// (kept in shared memory until the kernel ends: a global store here would make the next block barrier
// wait for it and distort the very phases being timed; the clock read takes a value just loaded from
// shared memory as an operand, because the assembler otherwise moves a clock read across a barrier)
#define RMARK(i)                                                                              \
    do {                                                                                      \
        if (tid == 0 && row == 0 && t == T / 2) {                                             \
            unsigned long long now;                                                           \
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);                     \
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");        \
            trace_s[(i)] = now;                                                               \
        }                                                                                     \
    } while (0)
#define UMARK(w, i, m)                                                                        \
    do {                                                                                      \
        if ((tid == 0 || tid == 128 || tid == 288) && row == 0 && t == T / 2 && (i) < 6) {    \
            unsigned long long now;                                                           \
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);                     \
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");        \
            utrace_s[(w)][(i)][(m)] = now;                                                    \
        }                                                                                     \
    } while (0)
#else
#define RMARK(i) do { } while (0)
#define UMARK(w, i, m) do { } while (0)
#endif

// The K + 1 largest of the unique, non-zero 32-bit keys a warp holds (PER a lane, 0 = none), in
// descending order: lane r returns the r-th largest (0 when there are fewer). K + 1 rounds of a
// warp-wide maximum (one redux instruction); the lane that holds the winner drops it.
template <int PER>
__device__ __forceinline__ uint32_t warp_top_keys(uint32_t (&key)[PER], int K, int lane) {
    uint32_t best = 0u;
#pragma unroll
    for (int s = 0; s < PER; ++s) best = max(best, key[s]);
    uint32_t kept = 0u;
    for (int r = 0; r <= K; ++r) {
        const uint32_t win = __reduce_max_sync(0xffffffffu, best);
        if (lane == r) kept = win;
        if (win != 0u && best == win) {
            best = 0u;
#pragma unroll
            for (int s = 0; s < PER; ++s) {
                if (key[s] == win) key[s] = 0u;
                best = max(best, key[s]);
            }
        }
    }
    return kept;
}

template <int D_>
__global__ void __launch_bounds__(kRowThreads, 1) k_rows_fwd(RowsCtx c) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ SelectShared S;
    __shared__ __align__(8) uint64_t full[kMaxStages], empty[kMaxStages];
    __shared__ int n_units_s;    // units some valid slot runs this position
    __shared__ int hmax_local;   // bits of max |h| over the block's cells after the last position
    __shared__ int failed_s;     // a ring wait ran out
    __shared__ __align__(8) uint64_t bar_d1[2], bar_d2;   // a unit's first product (two accumulator pairs in turn); the position's second products
    __shared__ __align__(8) uint64_t bar_sp[2];           // a unit's second product has read its activation buffer
    __shared__ __align__(8) uint64_t bar_v;               // the position's cell inputs are written (the first products' operand)
    __shared__ __align__(8) uint64_t bar_act[2];          // a unit's activations are written (the second product's operand, two buffers in turn)
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t in_bar;   // the next position's inputs (bulk copies by the producer)
    __shared__ uint64_t next_key_s;   // the (K + 1)-th best key of the position's scored order
#ifdef HSNW_TRACE
    __shared__ unsigned long long trace_s[64];
    __shared__ unsigned long long utrace_s[3][6][8];
#ifdef HSNW_TRACE
    if (threadIdx.x < 144) (&utrace_s[0][0][0])[threadIdx.x] = 0ull;
#endif
#endif

    cg::cluster_group cl = cg::this_cluster();
    const int C = c.C, r = static_cast<int>(cl.block_rank());
    const int row = blockIdx.x / C;
    constexpr int d = D_;   // compile time: the index arithmetic of every phase divides by it
    const int N = c.m.N, K = c.m.K, M = c.m.M, D = c.m.D, Sn = c.m.S, H = c.m.H;
    const int T = c.io.T, Nc = c.Nc, Ks = c.Ks, grows = c.gate_rows;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool producer = warp == kConsumers / 32;
    const bool issuer = warp > kConsumers / 32;          // three warps that issue the tensor-core products
    const int issue_role = warp - kConsumers / 32 - 1;   // 0, 1: a W1 piece each; 2: W2
    const bool tape = c.io.tape_state != 0;
    const bool rec = c.io.rec_c != nullptr;
    const int stride_in = 2 * d + 4;   // a block's line of the front inbox: u part, z_hat part, max |h|

    const uint32_t kStages = c.stages;   // 2 or 3: a ring index by a constant division or a mask, never a runtime division
    const bool three = kStages == 3u;
    auto ring_slot = [&](uint32_t g) { return three ? g % 3u : g & 1u; };
    auto ring_round = [&](uint32_t g) { return three ? g / 3u : g >> 1; };
    const int cmask = c.C - 1, cshift = __ffs(c.C) - 1;   // the cluster size is a power of two
    const RowsSmem L = rows_smem(c.m, C, c.slot_bytes, kStages);
    unsigned char* ring = dyn + L.ring + ((1024u - (smem_addr(dyn + L.ring) & 1023u)) & 1023u);
    float* h_s = reinterpret_cast<float*>(dyn + L.h);
    uint16_t* vh_s = reinterpret_cast<uint16_t*>(dyn + L.vh);
    float* lh_s = reinterpret_cast<float*>(dyn + L.lh);
    int64_t* age_s = reinterpret_cast<int64_t*>(dyn + L.age);
    int* cmax_s = reinterpret_cast<int*>(dyn + L.cmax);
    uint16_t* wout = reinterpret_cast<uint16_t*>(dyn + L.wout);
    uint16_t* vt = reinterpret_cast<uint16_t*>(dyn + L.vt);
    uint16_t* gate = reinterpret_cast<uint16_t*>(dyn + L.gate);
    float* swh = reinterpret_cast<float*>(dyn + L.swh);
    float* sw_head = reinterpret_cast<float*>(dyn + L.sw_head);
    float* sw_tail = reinterpret_cast<float*>(dyn + L.sw_tail);
    float* norm_w = reinterpret_cast<float*>(dyn + L.norm_w);
    float* cand_w = reinterpret_cast<float*>(dyn + L.cand_w);
    float* fb2 = reinterpret_cast<float*>(dyn + L.fb2);
    float* gate_b = reinterpret_cast<float*>(dyn + L.gate_b);
    float* score_b = reinterpret_cast<float*>(dyn + L.score_b);
    float* fb1p = reinterpret_cast<float*>(dyn + L.fb1p);
    float* score_all = reinterpret_cast<float*>(dyn + L.score_all);
    int* unit_all = reinterpret_cast<int*>(dyn + L.unit_all);
    int64_t* age_all = reinterpret_cast<int64_t*>(dyn + L.age_all);
    float* q_s = reinterpret_cast<float*>(dyn + L.q);
    float* q_after = reinterpret_cast<float*>(dyn + L.q_after);
    float* ue = reinterpret_cast<float*>(dyn + L.ue);
    float* rowterm = reinterpret_cast<float*>(dyn + L.rowterm);
    float* hold = reinterpret_cast<float*>(dyn + L.hold);
    float* big = reinterpret_cast<float*>(dyn + L.big);
    float* msg = reinterpret_cast<float*>(dyn + L.msg);
    float* rms = reinterpret_cast<float*>(dyn + L.rms);
    uint16_t* b2 = reinterpret_cast<uint16_t*>(dyn + L.b2);
    uint32_t* graph = reinterpret_cast<uint32_t*>(dyn + L.graph);
    float* gacc = reinterpret_cast<float*>(dyn + L.gacc);
    float* part_s = gacc;   // [Nc][M] between phase A and phase B
    float* inbox_front = reinterpret_cast<float*>(dyn + L.inbox_front);
    float* inbox_f = reinterpret_cast<float*>(dyn + L.inbox_f);
    float* inbox_delta = reinterpret_cast<float*>(dyn + L.inbox_delta);
    float* in_scal = reinterpret_cast<float*>(dyn + L.in_scal);
    float* in_pre = reinterpret_cast<float*>(dyn + L.in_pre);
    float* in_z = reinterpret_cast<float*>(dyn + L.in_z);
    float* upd = reinterpret_cast<float*>(dyn + L.upd);
    int* cell_of = reinterpret_cast<int*>(dyn + L.cell_of);
    int* unit_of = reinterpret_cast<int*>(dyn + L.unit_of);
    int* ulist = reinterpret_cast<int*>(dyn + L.ulist);
    uint64_t* cand = reinterpret_cast<uint64_t*>(dyn + L.cand);
    int* umask = reinterpret_cast<int*>(dyn + L.umask);
    float* Fk = upd;
    float* gp = upd + Ks * d;
    float* ys = upd + 2 * Ks * d;
    float* hnew = upd + 3 * Ks * d;
    float* hb = upd + 4 * Ks * d;
    float* dl = upd + 5 * Ks * d;
    float* scale = upd + 6 * Ks * d;

    const int cell0 = r * Nc;                 // the block's first cell
    // cell n lives in block n / Nc at row n % Nc: a multiply-high by ceil(2^32 / Nc), exact for n Nc < 2^32
    const uint32_t nc_magic = 0xffffffffu / static_cast<uint32_t>(Nc) + 1u;
    auto owner_of = [&](int n) { return static_cast<int>(__umulhi(static_cast<uint32_t>(n), nc_magic)); };
    const uint32_t md_magic = 0xffffffffu / static_cast<uint32_t>(M + d) + 1u;   // o / (M + d) the same way
    const int pre_cols = max(0, min(kFrontCols, H - r * kFrontCols));  // its columns that belong to S
    const unsigned char* bank = static_cast<const unsigned char*>(c.m.rows_bank);
    const unsigned char* front = static_cast<const unsigned char*>(c.m.rows_front);

    // ---- once per window: barriers, the resident weights, the block's cells and their derived state
    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&bar_d1[0], 2);   // one arrival per W1 piece's chain
        mbar_init(&bar_d1[1], 2);
        mbar_init(&bar_sp[0], 1);
        mbar_init(&bar_sp[1], 1);
        mbar_init(&bar_d2, 1);
        mbar_init(&bar_v, 1);
        mbar_init(&bar_act[0], kConsumers / 32);   // one arrival per compute warp
        mbar_init(&bar_act[1], kConsumers / 32);
        mbar_init(&in_bar, 1);
        hmax_local = 0;
        n_units_s = 0;
        failed_s = 0;
    }
    for (int e = tid; e < d * d; e += kRowThreads) {
        wout[e] = bf16_bits(c.m.wout_t[e]);
        vt[e] = bf16_bits(c.m.v_t[e]);
    }
    for (int e = tid; e < grows * d; e += kRowThreads) gate[e] = bf16_bits(c.m.gate_t[static_cast<int64_t>(r) * grows * d + e]);
    for (int e = tid; e < d * M; e += kRowThreads) swh[e] = c.m.score_w_t[2 * d * M + e];
    for (int e = tid; e < 2 * d * M; e += kRowThreads) sw_head[e] = c.m.score_w_t[e];
    for (int e = tid; e < (1 + Sn) * M; e += kRowThreads) sw_tail[e] = c.m.score_w_t[3 * d * M + e];
    for (int e = tid; e < 4 * d; e += kRowThreads) norm_w[e] = c.m.norm_w[e];
    for (int e = tid; e < d; e += kRowThreads) {
        cand_w[e] = c.m.cand_w[e];
        gate_b[e] = c.m.gate_b[e];
    }
    for (int e = tid; e < 2 * d; e += kRowThreads) fb2[e] = c.m.f_b2[e];
    for (int e = tid; e < M; e += kRowThreads) {
        score_b[e] = c.m.score_b[e];
        S.cost[e] = c.m.cost[e];
    }
    for (int e = tid; e < kFrontCols; e += kRowThreads) fb1p[e] = c.m.f_b1[r * kFrontCols + e];
    if (warp == 0) tmem_alloc(&tmem_slot, 512);
    for (int e = tid; e < N * D; e += kRowThreads)
        graph[e] = (static_cast<uint32_t>(c.m.pad_src[e]) << 16) | bf16_bits(c.m.edge_w[e]);
    const bool cut0 = c.io.reset[static_cast<int64_t>(row) * T] != 0;
    {
        const float* h0 = c.io.h0 + (static_cast<int64_t>(row) * N + cell0) * d;
        for (int e = tid; e < Nc * d; e += kRowThreads) h_s[e] = cut0 ? 0.0f : h0[e];
        const int64_t* a0 = c.io.age0 + static_cast<int64_t>(row) * N + cell0;
        for (int n = tid; n < Nc; n += kRowThreads) age_s[n] = cut0 ? 0 : a0[n];
        for (int x = tid; x < d; x += kRowThreads) q_s[x] = cut0 ? 0.0f : c.io.q0[static_cast<int64_t>(row) * d + x];
        // the first position's inputs
        const int64_t rt0 = static_cast<int64_t>(row) * T;
        for (int e = tid; e < Nc * Sn; e += kRowThreads) in_scal[e] = c.io.scalars[(rt0 * N + cell0) * Sn + e];
        for (int e = tid; e < pre_cols; e += kRowThreads) in_pre[e] = c.pre_s[rt0 * H + r * kFrontCols + e];
        for (int x = tid; x < d; x += kRowThreads) in_z[x] = c.io.z[rt0 * d + x];
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    // completed phases of the per-unit barriers before this position (bar_d1, bar_act and bar_sp complete once per
    // unit, the even-numbered units of a position on [0], the odd ones on [1]), and of bar_d2
    uint32_t units_even = 0, units_odd = 0, d2_phase = 0;
    for (int o = tid; o < Nc * (M + d); o += kRowThreads) {
        const int cell = o / (M + d), w = o - cell * (M + d);
        const float* hr = h_s + cell * d;
        float sum = 0.0f;
        if (w < M) {
            for (int x = 0; x < d; ++x) sum += bf16r(hr[x]) * swh[x * M + w];
            lh_s[cell * M + w] = sum;
        } else {
            for (int x = 0; x < d; ++x) sum += bf16r(hr[x]) * bf16_value(vt[x * d + (w - M)]);
            vh_s[cell * d + (w - M)] = bf16_bits(sum);
        }
    }
    for (int n = tid; n < Nc; n += kRowThreads) {
        int top = 0;
        for (int x = 0; x < d; ++x) top = max(top, __float_as_int(fabsf(h_s[n * d + x])));
        cmax_s[n] = top;
    }
    if (tape) {
        const int64_t rec0 = static_cast<int64_t>(row) * (T + 1);
        float* th = c.io.tape_h + (rec0 * N + cell0) * d;
        for (int e = tid; e < Nc * d; e += kRowThreads) th[e] = h_s[e];
        for (int n = tid; n < Nc; n += kRowThreads) c.io.tape_age[rec0 * N + cell0 + n] = age_s[n];
        if (r == 0)
            for (int x = tid; x < d; x += kRowThreads) c.io.tape_q[rec0 * d + x] = q_s[x];
    }
    uint32_t g_issue = 0, g_use = 0;   // copies issued (producer) / consumed (compute warps), in ring order
    if (producer && lane == 0) {
        for (int part = 0; part < 2; ++part) {
            const uint32_t slot = ring_slot(g_issue);
            mbar_expect_tx(&full[slot], c.front_bytes);
            bulk_g2s(ring + slot * c.slot_bytes, front + (static_cast<size_t>(r) * 2 + part) * c.front_bytes, c.front_bytes, &full[slot]);
            ++g_issue;
        }
    }
    cl.sync();

    // The part of a cell's logit for unit j that does not depend on the row's (u, eps): the state's part,
    // the age term and the scalars, summed in the scorer's order (the row term and the bias are added to
    // it in phase B, so the sum is the one the whole scorer makes).
    const float age_div = static_cast<float>(c.m.age_max);
    auto cell_part = [&](int i, int j) {
        float acc = lh_s[i * M + j];
        acc += bf16r(static_cast<float>(age_s[i]) / age_div) * sw_tail[j];
        for (int sI = 0; sI < Sn; ++sI) acc += bf16r(in_scal[i * Sn + sI]) * sw_tail[(1 + sI) * M + j];
        return acc;
    };
    const uint32_t m_magic = M > 1 ? magic_of(M) : 0u;

    for (int t = 0; t < T; ++t) {
        const int64_t rt = static_cast<int64_t>(row) * T + t;
        const bool last = t + 1 == T;
        const bool clear = !last && c.io.reset[rt + 1] != 0;
        // ---------------- A: the front MLPs on the block's columns
        RMARK(0);
        if (!producer && !issuer) {
            if (t > 0) ring_wait(&in_bar, static_cast<uint32_t>(t - 1) & 1u, c.status, &failed_s);
            if (tid < d) ue[tid] = bf16r(q_s[tid]);
            consumer_sync();
            float* act = big;                     // [256]
            float* fpart = big + kFrontCols;      // [256 / d][2d]
            {
                const uint32_t slot = ring_slot(g_use);
                ring_wait(&full[slot], ring_round(g_use) & 1u, c.status, &failed_s);
                const uint16_t* w1c = reinterpret_cast<const uint16_t*>(ring + slot * c.slot_bytes);
                const int col = tid, colg = r * kFrontCols + col;
                const float sum = dot_bf16w(ue, 1, w1c + col, kFrontCols, d);
                const float pre = colg >= H ? fb1p[col] : in_pre[col];
                act[col] = bf16r(gelu_erf(bf16r(sum + pre)));
            }
            consumer_sync();
            if (tid == 0) mbar_arrive(&empty[ring_slot(g_use)]);
            {
                const uint32_t slot = ring_slot(g_use + 1);
                ring_wait(&full[slot], ring_round(g_use + 1) & 1u, c.status, &failed_s);
                const uint16_t* w2c = reinterpret_cast<const uint16_t*>(ring + slot * c.slot_bytes);
                const int x = tid % d, grp = tid / d;
                const bool is_p = r * kFrontCols + grp * d >= H;
                const float sum = dot_bf16w(act + grp * d, 1, w2c + grp * d * d + x, d, d);
                fpart[grp * 2 * d + x] = is_p ? 0.0f : sum;
                fpart[grp * 2 * d + d + x] = is_p ? sum : 0.0f;
            }
            consumer_sync();
            if (tid == 0) mbar_arrive(&empty[ring_slot(g_use + 1)]);
            if (tid < 2 * d) {
                float tot = 0.0f;
                for (int grp = 0; grp < kFrontCols / d; ++grp) tot += fpart[grp * 2 * d + tid];
                for (int p = 0; p < C; ++p) peer(cl, inbox_front, p)[r * stride_in + tid] = tot;
            }
            if (tid == 0) peer(cl, inbox_front, 0)[r * stride_in + 2 * d] = __int_as_float(hmax_local);
        }
        g_use += 2;
        RMARK(1);
        cl.sync();   // 1
        RMARK(2);
        if (producer && t > 0) {
            // the previous position's summary and ages for the tape: they are final since that position's
            // phase F and stay until this position's
            const int64_t rp = rt - 1;
            const bool cleared = c.io.reset[rt] != 0;
            if (r == 0) {
                for (int x = lane; x < d; x += 32) {
                    c.io.qs[rp * d + x] = q_after[x];
                    if (tape) c.io.tape_q[(static_cast<int64_t>(row) * (T + 1) + t) * d + x] = cleared ? 0.0f : q_after[x];
                }
            }
            if (tape)
                for (int n = lane; n < Nc; n += 32) c.io.tape_age[(static_cast<int64_t>(row) * (T + 1) + t) * N + cell0 + n] = age_s[n];
        }
        // ---------------- B: u, eps, the scorer on the block's cells
        if (!producer && !issuer) {
            if (tid < 2 * d) {
                float sum = 0.0f;
                for (int p = 0; p < C; ++p) sum += inbox_front[p * stride_in + tid];
                const float out = bf16r(sum + fb2[tid]);
                ue[tid] = tid < d ? out : in_z[tid - d] - out;
            }
            if (tid == 0) hmax_local = 0;   // phase A sent it; phase F of this position takes the next maximum
            if (r == 0 && tid == 0 && t > 0 && c.io.h_max) {
                int mx = 0;
                for (int p = 0; p < C; ++p) mx = max(mx, __float_as_int(inbox_front[p * stride_in + 2 * d]));
                c.io.h_max[rt - 1] = __int_as_float(mx);
            }
            // the block's cells' part of the logits (everything but the row's term), a (cell, unit) pair a thread
            for (int o = tid; o < Nc * M; o += kConsumers) {
                const int i = M > 1 ? div_magic(o, m_magic) : o;
                part_s[o] = cell_part(i, o - i * M);
            }
            consumer_sync();
            RMARK(14);
            for (int j = warp; j < M; j += kConsumers / 32) {
                float sum = 0.0f;
                for (int x = lane; x < 2 * d; x += 32) sum += bf16r(ue[x]) * sw_head[x * M + j];
                sum = warp_sum(sum);
                if (lane == 0) rowterm[j] = sum;
            }
            consumer_sync();
            RMARK(15);
            const float lambda = c.m.lambda_cost;
            // four threads per cell, each with the units sub, sub + 4, ...; the quad then keeps the
            // first maximiser (the higher score, the lower unit on a tie)
            for (int i0 = 0; i0 < Nc; i0 += kConsumers / 4) {
                const int i = i0 + (tid >> 2), sub = tid & 3;
                float best = -INFINITY;
                int arg = 0;
                int64_t ag = 0;
                if (i < Nc) {
                    ag = age_s[i];
#pragma unroll
                    for (int jj = 0; jj < kMaxMR / 4; ++jj) {
                        const int j = sub + 4 * jj;
                        if (j < M) {
                            const float logit = bf16r(part_s[i * M + j] + rowterm[j] + score_b[j]);
                            if (c.io.logits) c.io.logits[(rt * N + cell0 + i) * M + j] = logit;
                            const float sc = lambda > 0.0f ? __fsub_rn(logit, __fmul_rn(lambda, S.cost[j])) : logit;
                            if (jj == 0 || sc > best) {
                                best = sc;
                                arg = j;
                            }
                        }
                    }
                }
#pragma unroll
                for (int w = 1; w < 4; w <<= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, w);
                    const int oa = __shfl_xor_sync(0xffffffffu, arg, w);
                    if (ob > best || (ob == best && oa < arg)) {
                        best = ob;
                        arg = oa;
                    }
                }
                if (i < Nc && sub < C) {   // thread `sub` of the quad writes block sub's copy
                    peer(cl, score_all, sub)[cell0 + i] = best;
                    peer(cl, unit_all, sub)[cell0 + i] = arg;
                    peer(cl, age_all, sub)[cell0 + i] = ag;
                }
                if (i < Nc && C > 4 && sub == 0) {
                    for (int p = 4; p < C; ++p) {
                        peer(cl, score_all, p)[cell0 + i] = best;
                        peer(cl, unit_all, p)[cell0 + i] = arg;
                        peer(cl, age_all, p)[cell0 + i] = ag;
                    }
                }
            }
        }
        RMARK(3);
        cl.sync();   // 2
        RMARK(4);
        // ---------------- C: the decision (every block, on identical inputs). A cell's place in
        // the scored order is the number of cells with a larger key, counted by the cell's thread
        // against all keys: no rounds, no sort. One warp then finishes (budget, threshold, probes).
        uint64_t* keys = cand;
        int* stale_w = reinterpret_cast<int*>(cand + N);     // [8] cells older than age_max, per warp
        int* old_rank = stale_w + 8;                          // [K] the same flag for the K best
        if (!producer && !issuer && !c.io.forced) {
            int n_old = 0;
            if (c.m.lambda_cost == 0.0f) {
                // the scores are bf16 values here (rounded logits, no cost term): the low half of
                // their order word carries nothing, so (score's high half, 0xffff - index) is a
                // 32-bit key with the same order, unique per cell. A thread holds the keys of the cells
                // tid, tid + 256, ...; every warp finds its K + 1 best by rounds of a warp-wide
                // maximum, the warps' lists meet in shared memory and warp 0 takes the K + 1 best of
                // those the same way: lane r then holds the cell of rank r.
                uint32_t* wtop = reinterpret_cast<uint32_t*>(keys);   // [8][K + 1]
                const int64_t age_max = static_cast<int64_t>(c.m.age_max);
                auto own_keys = [&](auto per) {
                    constexpr int PER = decltype(per)::value;
                    uint32_t key[PER];
                    int old = 0;
#pragma unroll
                    for (int sI = 0; sI < PER; ++sI) {
                        const int i = tid + sI * kConsumers;
                        key[sI] = 0u;
                        if (i < N) {
                            key[sI] = (float_order(score_all[i]) & 0xffff0000u) | (0xffffu - static_cast<uint32_t>(i));
                            old += age_all[i] > age_max ? 1 : 0;
                        }
                    }
                    const uint32_t kept = warp_top_keys<PER>(key, K, lane);
                    if (lane <= K) wtop[warp * (K + 1) + lane] = kept;
                    old = __reduce_add_sync(0xffffffffu, old);
                    if (lane == 0) stale_w[warp] = old;
                };
                if (N <= kConsumers) own_keys(std::integral_constant<int, 1>{});
                else if (N <= 2 * kConsumers) own_keys(std::integral_constant<int, 2>{});
                else if (N <= 4 * kConsumers) own_keys(std::integral_constant<int, 4>{});
                else own_keys(std::integral_constant<int, 8>{});
                RMARK(32);
                consumer_sync();
                RMARK(33);
                if (warp == 0) {
                    const int n_cand = (kConsumers / 32) * (K + 1);   // at most 72
                    uint32_t cand3[3];
#pragma unroll
                    for (int sI = 0; sI < 3; ++sI) cand3[sI] = lane + 32 * sI < n_cand ? wtop[lane + 32 * sI] : 0u;
                    const uint32_t kept = warp_top_keys<3>(cand3, K, lane);
                    const int cell = static_cast<int>(0xffffu - (kept & 0xffffu));
                    if (lane < K && kept != 0u) {
                        S.order[lane] = cell;
                        old_rank[lane] = age_all[cell] > age_max ? 1 : 0;
                    }
                    if (lane == K) next_key_s = kept != 0u ? pack_key(score_all[cell], cell) : 0ull;
                    __syncwarp();
                }
                n_old = -1;   // the counts are in place
            } else {
                for (int i = tid; i < N; i += kConsumers) keys[i] = pack_key(score_all[i], i);
                if (tid == 0) next_key_s = 0ull;
                consumer_sync();
                for (int i = tid; i < N; i += kConsumers) {
                    const uint64_t mine = keys[i];
                    int rank = 0;
#pragma unroll 8
                    for (int j = 0; j < N; ++j) rank += keys[j] > mine ? 1 : 0;
                    const bool old = age_all[i] > static_cast<int64_t>(c.m.age_max);
                    n_old += old ? 1 : 0;
                    if (rank < K) {
                        S.order[rank] = i;
                        old_rank[rank] = old ? 1 : 0;
                    } else if (rank == K) {
                        next_key_s = mine;
                    }
                }
            }
            if (n_old >= 0) {
                n_old = __reduce_add_sync(0xffffffffu, n_old);
                if (lane == 0) stale_w[warp] = n_old;
                consumer_sync();
            }
        }
        RMARK(16);
        if (warp == 0) {
            if (!c.io.forced) {
                SelectParams P;
                P.N = N; P.M = M; P.K = K; P.age_max = c.m.age_max; P.probes = c.m.probes;
                P.reserved = 0; P.fixed_units = 0;
                P.overhead = c.m.cell_overhead; P.shared_cost = c.m.shared_cost; P.limit = c.m.limit;
                // the budget: costs summed in slot order, every lane follows the same running sum
                const int cidx = lane < K ? S.order[lane] : 0;
                const int u = unit_all[cidx];
                const float cost = P.overhead + S.cost[u];
                float running = 0.0f, mine_cum = 0.0f;
                for (int i = 0; i < K; ++i) {
                    running += __shfl_sync(0xffffffffu, cost, i);
                    if (lane == i) mine_cum = running;
                }
                const bool ok = lane < K && P.shared_cost + mine_cum <= P.limit;
                const unsigned okmask = __ballot_sync(0xffffffffu, ok);
                const int n_valid = __popc(okmask);
                if (lane < K) {
                    S.out_cell[lane] = ok ? cidx : 0;
                    S.out_unit[lane] = ok ? u : 0;
                    S.out_flag[lane] = ok ? 1 : 0;
                }
                if (lane == 0) {
                    const bool any = n_valid > 0;
                    const float low = any ? score_all[S.order[n_valid - 1]] : INFINITY;
                    float high;
                    if (n_valid < K) high = score_all[S.order[n_valid]];
                    else high = next_key_s ? score_all[key_cell(next_key_s)] : -INFINITY;
                    S.theta = 0.5f * (low + high);
                    S.n_valid = n_valid;
                }
                int n_force = 0;
                if (P.probes) {
                    const int total_old = __reduce_add_sync(0xffffffffu, lane < kConsumers / 32 ? stale_w[lane] : 0);
                    const int chosen_old = __popc(__ballot_sync(0xffffffffu, lane < n_valid && old_rank[lane] != 0));
                    const int n_stale = total_old - chosen_old;
                    n_force = n_stale < n_valid ? n_stale : n_valid;
                }
                __syncwarp();
                // a row with stale cells to refresh takes the one-warp routine from the scored order on
                if (n_force > 0) select_finish_warp(P, score_all, unit_all, age_all, S, next_key_s);
                RMARK(17);
            } else {
                for (int k = lane; k < K; k += 32) {
                    const bool ok = c.io.valid[rt * K + k] != 0;
                    S.out_cell[k] = ok ? static_cast<int>(c.io.cells[rt * K + k]) : 0;
                    S.out_unit[k] = ok ? static_cast<int>(c.io.units[rt * K + k]) : 0;
                    S.out_flag[k] = ok ? 1 : 0;
                }
            }
            __syncwarp();
            int my_unit = -1;
            for (int k = lane; k < K; k += 32) {   // K <= 32: lane k holds slot k
                const bool ok = (S.out_flag[k] & 1) != 0;
                cell_of[k] = ok ? S.out_cell[k] : -1;
                my_unit = ok ? S.out_unit[k] : -1;
                unit_of[k] = my_unit;
            }
            // the units in use, ascending, and each one's slots as a bit mask: the set of units by one
            // warp-wide OR, a unit's place = the number of smaller units in the set, its slots = the
            // lanes that hold the same unit
            const unsigned in_use = __reduce_or_sync(0xffffffffu, my_unit >= 0 ? 1u << my_unit : 0u);
            const unsigned same = __match_any_sync(0xffffffffu, my_unit);
            if (my_unit >= 0 && (same & ((1u << lane) - 1u)) == 0u) {   // the unit's first slot writes its entry
                const int at = __popc(in_use & ((1u << my_unit) - 1u));
                ulist[at] = my_unit;
                umask[at] = static_cast<int>(same);
            }
            const int n = __popc(in_use);
            if (lane == 0) n_units_s = n;
            RMARK(18);
        }
#ifdef HSNW_TRACE
        if (lane == 0 && row == 0 && t == T / 2) {
            unsigned long long now;
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");
            trace_s[48 + warp] = now;
        }
#endif
        __syncthreads();
#ifdef HSNW_TRACE
        if (lane == 0 && row == 0 && t == T / 2) {
            unsigned long long now;
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");
            trace_s[36 + warp] = now;   // when each warp leaves the barrier
        }
#endif
        RMARK(5);
        const int n_units = n_units_s;
        // ---------------- D
        if (producer) {
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                if (!last) {
                    // the next position's inputs (their buffers were last read before this position's decision)
                    const uint32_t b_scal = static_cast<uint32_t>(sizeof(float)) * Nc * Sn, b_pre = static_cast<uint32_t>(sizeof(float)) * pre_cols;
                    const uint32_t b_z = static_cast<uint32_t>(sizeof(float)) * d;
                    mbar_expect_tx(&in_bar, b_scal + b_pre + b_z);
                    bulk_g2s(in_scal, c.io.scalars + ((rt + 1) * N + cell0) * Sn, b_scal, &in_bar);
                    if (pre_cols > 0) bulk_g2s(in_pre, c.pre_s + (rt + 1) * H + r * kFrontCols, b_pre, &in_bar);
                    bulk_g2s(in_z, c.io.z + (rt + 1) * d, b_z, &in_bar);
                }
                const int n_bank = n_units * 3;
                const int total = n_bank + (last ? 0 : 2);
                auto request = [&](int i, uint32_t slot) {   // the position's piece i into its slot
                    const unsigned char* from;
                    uint32_t bytes;
                    if (i < n_bank) {
                        const int ui = i / 3, piece = i - 3 * ui;
                        const int j = ulist[ui];
                        from = bank + (static_cast<size_t>(j) * C + r) * c.bank_bytes + piece * c.w1_bytes;
                        bytes = piece == 2 ? c.w1_bytes / 2 : c.w1_bytes;
                    } else {
                        from = front + (static_cast<size_t>(r) * 2 + (i - n_bank)) * c.front_bytes;
                        bytes = c.front_bytes;
                    }
                    mbar_expect_tx(&full[slot], bytes);
                    bulk_g2s(ring + slot * c.slot_bytes, from, bytes, &full[slot]);
                };
                if (three) {
                    // Three slots: every third piece shares a slot (a piece kind each within a position), and the
                    // slots are served independently, whichever is handed back first: a unit's W2 slot is handed
                    // back only after its epilogue, and requests in ring order would hold the next units' W1
                    // pieces behind it (measured with forced decisions: 1.2 us a unit in ring order, 0.8 this
                    // way). Per slot the pieces still go in ring order.
                    const uint32_t g_first = g_issue;
                    int next[3] = {0, 1, 2};   // the next piece (index in the position) of the slot (g_first + k) % 3
                    int remaining = total;
                    uint32_t idle = 0;
                    while (remaining > 0 && !failed_s) {
                        bool progress = false;
                        int oldest = -1;
#pragma unroll
                        for (int k = 0; k < 3; ++k) {
                            const int i = next[k];
                            if (i >= total) continue;
                            const uint32_t g = g_first + static_cast<uint32_t>(i), slot = ring_slot(g);
                            if (g >= kStages) {
                                uint32_t done;
                                asm volatile(
                                    "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                                    : "=r"(done)
                                    : "r"(smem_addr(&empty[slot])), "r"((ring_round(g) - 1u) & 1u)
                                    : "memory");
                                if (!done) {
                                    // (where to sleep if nothing moves: a first-layer piece's slot comes back
                                    // long before a second-layer piece's)
                                    if (oldest < 0 || (next[oldest] % 3 == 2 && i % 3 != 2)) oldest = k;
                                    continue;
                                }
                            }
                            request(i, slot);
                            next[k] = i + 3;
                            --remaining;
                            progress = true;
                        }
                        if (!progress && oldest >= 0) {
                            // nothing was handed back: sleep on the oldest outstanding piece's slot for a moment
                            const uint32_t g = g_first + static_cast<uint32_t>(next[oldest]);
                            uint32_t done;
                            asm volatile(
                                "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                                : "=r"(done)
                                : "r"(smem_addr(&empty[ring_slot(g)])), "r"((ring_round(g) - 1u) & 1u), "r"(1000u)
                                : "memory");
                            if (++idle > (1u << 20)) {   // bounded like every wait of the pipeline
                                failed_s = 1;
                                if (c.status) atomicExch(c.status, 1);
                            }
                        }
                    }
                    g_issue = g_first + static_cast<uint32_t>(total);
                } else {
                    for (int i = 0; i < total; ++i) {
                        const uint32_t slot = ring_slot(g_issue);
                        if (g_issue >= kStages) ring_wait(&empty[slot], (ring_round(g_issue) - 1u) & 1u, c.status, &failed_s);
                        request(i, slot);
                        ++g_issue;
                    }
                }
            }
            __syncwarp();
            if (r == 0 && c.io.us)   // u: in place since phase B, until the next position's phase A
                for (int x = lane; x < d; x += 32) c.io.us[rt * d + x] = ue[x];
            if (r == 0 && !c.io.forced) {   // the decision's record
                for (int k = lane; k < K; k += 32) {
                    const bool ok = (S.out_flag[k] & 1) != 0;
                    c.io.cells[rt * K + k] = S.out_cell[k];
                    c.io.units[rt * K + k] = S.out_unit[k];
                    c.io.valid[rt * K + k] = static_cast<uint8_t>(ok ? 1 : 0);
                    c.io.refreshed[rt * K + k] = static_cast<uint8_t>((S.out_flag[k] >> 1) & 1);
                }
                if (lane == 0) c.io.theta[rt] = S.theta;
            }
        } else if (issuer) {
            // The units' two layers on the streamed weights, on the tensor cores. A unit's weights on the
            // block's 128 hidden columns arrive as three pieces, each a ring slot of its own: W1's rows for
            // the inputs [0, 2d) and [2d, 4d) (A tiles [128 columns][2d]), then W2 ([d outputs][128
            // columns]). Each piece has its own issuer warp (a product costs its issuing warp about 70
            // cycles of instructions, twice the tensor pipe's time for it: one warp issuing a unit's 24
            // products was the unit's critical path). Warps 0 and 1: D1a, D1b [128 columns, 16 slots] =
            // a W1 piece x its half of the inputs^T (the epilogue adds the two); the piece's slot is
            // handed back when its products have run. Warp 2: D2 [d outputs, 16 slots] += W2 x
            // activations^T, accumulating over the position's units (rows d..127 of D2 come from the
            // bytes after the tile and are never read). Each product is issued as soon as its operands
            // are in place: a first-layer chain of unit i waits for the piece and, from the third unit on,
            // for the epilogue of unit i - 2 (which read the accumulators it overwrites); a second-layer
            // chain for the unit's activations and its piece.
            const uint16_t* vop = reinterpret_cast<const uint16_t*>(big);
            const uint32_t idesc = umma_idesc_bf16(128, 16);
            constexpr int steps_piece = (2 * d) >> 4;       // K = 16 products of one W1 piece
            const uint32_t g0 = g_use;
            auto unit_parity = [&](int i) { return (((i & 1) ? units_odd : units_even) + static_cast<uint32_t>(i >> 1)) & 1u; };
            // (A slot's barrier tells two consecutive rounds apart, no more: a warp may wait for a slot's
            // round only if it also consumed, or waited for, the round before. With three slots every piece
            // kind has a slot and a warp of its own. With two the kinds rotate through the slots, so one
            // warp issues everything in ring order: first layer, second layer, unit after unit.)
            auto first_piece = [&](int i, int piece) {
                UMARK(2, i, 0);
                if (i >= 2) ring_wait(&bar_act[i & 1], unit_parity(i - 2), c.status, &failed_s);
                const uint32_t g = g0 + 3 * i + piece, slot = ring_slot(g);
                ring_wait(&full[slot], ring_round(g) & 1u, c.status, &failed_s);
                tcgen05_fence_after();
                UMARK(2, i, 1);
                const unsigned char* tile = ring + slot * c.slot_bytes;
                const uint32_t acc = taddr + 32 * (i & 1) + 16 * piece;   // D1a, D1b of the unit's parity
                if (d == 64)   // (a piece is two 128-byte-swizzled K-blocks of 64 inputs, 128 rows each)
                    umma_chain_sw128<steps_piece>(acc, umma_desc_sw128(tile), (128 * 128) >> 4,
                                                  umma_desc(vop + piece * steps_piece * 2 * 16 * 8, 16), umma_kstep(16), idesc, false);
                else
                    umma_chain_fixed<steps_piece>(acc, umma_desc(tile, 128), umma_desc(vop + piece * steps_piece * 2 * 16 * 8, 16),
                                                  idesc, umma_kstep(128), umma_kstep(16), false);
                umma_commit(&empty[slot]);   // the piece is spent when these products have read it
                umma_commit(&bar_d1[i & 1]);
                UMARK(2, i, 2);
            };
            auto second_layer = [&](int i) {
                UMARK(2, i, 3);
                ring_wait(&bar_act[i & 1], unit_parity(i), c.status, &failed_s);
                UMARK(2, i, 4);
                const uint32_t g = g0 + 3 * i + 2, slot = ring_slot(g);
                ring_wait(&full[slot], ring_round(g) & 1u, c.status, &failed_s);
                tcgen05_fence_after();
                UMARK(2, i, 5);
                const unsigned char* tile = ring + slot * c.slot_bytes;
                if (d == 64)   // (two K-blocks of 64 hidden columns, d rows each)
                    umma_chain_sw128<8>(taddr + 256, umma_desc_sw128(tile), (64 * 128) >> 4,
                                        umma_desc(b2 + (i & 1) * (kActOperand / 2), 16), umma_kstep(16), idesc, i > 0);
                else
                    umma_chain_fixed<8>(taddr + 256, umma_desc(tile, d), umma_desc(b2 + (i & 1) * (kActOperand / 2), 16), idesc,
                                        umma_kstep(d), umma_kstep(16), i > 0);
                umma_commit(&empty[slot]);
                umma_commit(&bar_sp[i & 1]);
                if (i + 1 == n_units) umma_commit(&bar_d2);
                UMARK(2, i, 6);
            };
            if (issue_role < 2) ring_wait(&bar_v, static_cast<uint32_t>(t) & 1u, c.status, &failed_s);
            if (three) {
                for (int i = 0; i < n_units; ++i) {
                    if (issue_role < 2) first_piece(i, issue_role);
                    else second_layer(i);
                }
            } else if (issue_role == 0) {
                for (int i = 0; i < n_units; ++i) {
                    first_piece(i, 0);
                    first_piece(i, 1);
                    second_layer(i);
                }
            }
            tcgen05_fence_before();
        } else {
            RMARK(24);
            // Every value comes from another block's shared memory (a few hundred cycles each): all the loads
            // of a thread's elements are issued before the first use, four edges at a time, instead of one
            // after the other.
            for (int e0 = tid; e0 < K * d; e0 += 2 * kConsumers) {
                const float* hp[2];
                const uint16_t* vp[2][4];
                float ew[2][4];
                float hv[2], sum[2] = {0.0f, 0.0f};
                uint16_t vv[2][4];
                int cellv[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int e = e0 + u * kConsumers;
                    const int k = e < K * d ? e / d : 0, x = e < K * d ? e - k * d : 0;
                    const int cell = S.out_cell[k];
                    cellv[u] = cell;
                    const int co = owner_of(cell);
                    hp[u] = peer(cl, h_s, co) + (cell - co * Nc) * d + x;
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) hv[u] = *hp[u];
                for (int j0 = 0; j0 < D; j0 += 4) {   // edge order
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int e = e0 + u * kConsumers;
                        const int x = e < K * d ? e % d : 0;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const uint32_t edge = j0 + jj < D ? graph[cellv[u] * D + j0 + jj] : 0u;
                            const int sc = static_cast<int>(edge >> 16);
                            const int so = owner_of(sc);
                            vp[u][jj] = peer(cl, vh_s, so) + (sc - so * Nc) * d + x;
                            ew[u][jj] = bf16_lo(edge);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) vv[u][jj] = *vp[u][jj];
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj)
                            if (j0 + jj < D) sum[u] += bf16_value(vv[u][jj]) * ew[u][jj];
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int e = e0 + u * kConsumers;
                    if (e < K * d) {
                        hold[e] = hv[u];
                        msg[e] = bf16r(sum[u]);
                    }
                }
            }
            // rows 8..15 of the two activation operands (their bytes belong to other phases' data)
            for (int e = tid; e < 2 * 16 * 8; e += kConsumers) {
                const int which = e >> 7, p = (e >> 3) & 15, k = 8 + (e & 7);
                reinterpret_cast<uint4*>(b2 + which * (kActOperand / 2))[p * 16 + k] = make_uint4(0u, 0u, 0u, 0u);
            }
            consumer_sync();
            RMARK(22);
            for (int k = warp; k < K; k += kConsumers / 32) {
                float sq = 0.0f;
                for (int jx = lane; jx < 4 * d; jx += 32) {
                    const int blk = jx / d, x = jx - blk * d;
                    const float v = blk == 0 ? ue[x] : blk == 1 ? ue[d + x] : blk == 2 ? hold[k * d + x] : msg[k * d + x];
                    sq += v * v;
                }
                sq = warp_sum(sq);
                if (lane == 0) rms[k] = rsqrtf(sq / static_cast<float>(4 * d) + c.m.norm_eps);
            }
            consumer_sync();
            RMARK(23);
            RMARK(6);
            // the pairs' inputs as the tensor cores' B operand: bf16 [4d/8][16 slots][8] (slots K..15 stay zero)
            uint16_t* vop = reinterpret_cast<uint16_t*>(big);
            for (int e = tid; e < K * 4 * d; e += kConsumers) {
                const int k = e / (4 * d), jx = e - k * 4 * d;
                const int blk = jx / d, x = jx - blk * d;
                const float val = blk == 0 ? ue[x] : blk == 1 ? ue[d + x] : blk == 2 ? hold[k * d + x] : msg[k * d + x];
                vop[((jx >> 3) * 16 + k) * 8 + (jx & 7)] = bf16_bits(val * rms[k] * norm_w[jx]);
            }
            for (int e = tid; e < (4 * d / 8) * 16; e += kConsumers)   // the front phase used the padded slots' bytes
                if ((e & 15) >= K) reinterpret_cast<uint4*>(vop)[e] = make_uint4(0u, 0u, 0u, 0u);
            fence_async_smem();   // the operand written above, before the tensor cores read it
            consumer_sync();
            if (tid == 0) mbar_arrive(&bar_v);   // the issuer warp starts the units' first layers
            RMARK(7);
            // The epilogues of the units' first layers (the issuer warp runs the products): a unit's epilogue
            // adds the bias, rounds, records, applies the activation for the slots that run the unit (zero
            // for the others) and writes the bf16 operand of the second product. All eight warps read D1:
            // warp w the columns 32 (w % 4) .. and the slots 4 (w / 4) .. 4 (w / 4) + 3, and go on to the
            // next unit without a block barrier (a warp's arrival on the operand's barrier says its part is
            // written); before the first accumulator is ready they compute the gate's partial sums.
            RMARK(30);
            const int hc = lane + 32 * (warp & 3);            // the thread's hidden column of the block (TMEM lane)
            const int sh = warp >> 2;                         // its half of the slots: 4 sh .. 4 sh + 3
            float bias_next = n_units > 0 ? c.m.b1[ulist[0] * H + r * 128 + hc] : 0.0f;   // a unit ahead
            {
                // the gate's partial sum over the block's input rows (under the first unit's first layer)
                const int x = tid % d, grp = tid / d, ngrp = kConsumers / d;
                for (int k = grp; k < K; k += ngrp) {
                    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
                    if (cell_of[k] >= 0) {
                        // the slot's inputs r grows .. of the operand: 8 consecutive inputs are one 16-byte unit
                        for (int xi = 0; xi < grows; xi += 8) {
                            const int jx = r * grows + xi;
                            const uint4 vv = *reinterpret_cast<const uint4*>(vop + ((jx >> 3) * 16 + k) * 8);
                            const uint16_t* g = gate + xi * d + x;
                            s0 += bf16_lo(vv.x) * bf16_value(g[0]);
                            s1 += bf16_hi(vv.x) * bf16_value(g[d]);
                            s2 += bf16_lo(vv.y) * bf16_value(g[2 * d]);
                            s3 += bf16_hi(vv.y) * bf16_value(g[3 * d]);
                            s0 += bf16_lo(vv.z) * bf16_value(g[4 * d]);
                            s1 += bf16_hi(vv.z) * bf16_value(g[5 * d]);
                            s2 += bf16_lo(vv.w) * bf16_value(g[6 * d]);
                            s3 += bf16_hi(vv.w) * bf16_value(g[7 * d]);
                        }
                    }
                    gacc[k * d + x] = (s0 + s1) + (s2 + s3);
                }
            }
            float hid_keep[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int i = 0; i < n_units; ++i) {
                const unsigned mask = static_cast<unsigned>(umask[i]);
                UMARK(tid == 0 ? 0 : 1, i, 0);
                {
                    const float bias = bias_next;
                    if (i + 1 < n_units) bias_next = c.m.b1[ulist[i + 1] * H + r * 128 + hc];
                    uint16_t* b2i = b2 + (i & 1) * (kActOperand / 2);
                    const uint32_t parity = (((i & 1) ? units_odd : units_even) + static_cast<uint32_t>(i >> 1)) & 1u;
                    // (the buffer's previous tenant, unit i - 2: its second product has read it)
                    if (i >= 2) ring_wait(&bar_sp[i & 1], parity ^ 1u, c.status, &failed_s);
                    ring_wait(&bar_d1[i & 1], parity, c.status, &failed_s);
                    tcgen05_fence_after();
                    if (i == 0) RMARK(25);
                    UMARK(tid == 0 ? 0 : 1, i, 2);
                    float acc[8];
                    tmem_ld4x2(tmem_addr(taddr, 32 * (warp & 3), 32 * (i & 1) + 4 * sh), acc);   // D1a, D1b: the thread's four slots
                    UMARK(tid == 0 ? 0 : 1, i, 3);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int k = 4 * sh + q;
                        float a = 0.0f;
                        hid_keep[q] = 0.0f;
                        if (mask & (1u << k)) {
                            const float hid = bf16r((acc[q] + acc[4 + q]) + bias);
                            hid_keep[q] = hid;
                            a = gelu_erf(hid);
                        }
                        b2i[((hc >> 3) * 16 + k) * 8 + (hc & 7)] = bf16_bits(a);
                    }
                    fence_async_smem();
                    tcgen05_fence_before();
                    if (i == 0) RMARK(26);
                    UMARK(tid == 0 ? 0 : 1, i, 4);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_act[i & 1]);   // this warp's activations are written
                UMARK(tid == 0 ? 0 : 1, i, 5);
                if (rec) {
                    // the record of the pre-activations goes out after the barrier: a barrier waits
                    // for the stores its threads have in flight
                    const int colg = r * 128 + hc;
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (mask & (1u << (4 * sh + q))) static_cast<uint16_t*>(c.io.rec_hidden)[(rt * K + 4 * sh + q) * H + colg] = bf16_bits(hid_keep[q]);
                }
                if (i == 0) RMARK(27);
            }
            const int n_chunks = 3 * n_units;
            consumer_sync();   // (the gate's partial sums are written)
            RMARK(8);
            // the block's partial of every slot's second layer from the accumulator, and the gate's
            // partial, to the slots' owners
            if (sh == 0 && 32 * warp < d) {   // the outputs x < d sit in the accumulator's lanes 0 .. d - 1
                float acc[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
                if (n_chunks > 0) {
                    ring_wait(&bar_d2, d2_phase & 1u, c.status, &failed_s);
                    tcgen05_fence_after();
                    tmem_ld8(tmem_addr(taddr, 32 * warp, 256), acc);
                }
                RMARK(28);
                if (hc < d) {
#pragma unroll
                    for (int k = 0; k < kMaxK; ++k)
                        if (k < K) peer(cl, inbox_f, k & cmask)[(r * Ks + (k >> cshift)) * 2 * d + hc] = acc[k];
                }
            }
            if (n_chunks > 0) ++d2_phase;
            for (int e = tid; e < K * d; e += kConsumers) {
                const int k = e / d, x = e - k * d;
                peer(cl, inbox_f, k & cmask)[(r * Ks + (k >> cshift)) * 2 * d + d + x] = gacc[e];
            }
            tcgen05_fence_before();
        }
        g_use += 3 * n_units;
        units_even += static_cast<uint32_t>((n_units + 1) >> 1);
        units_odd += static_cast<uint32_t>(n_units >> 1);
#ifdef HSNW_TRACE
        if (warp >= 8 && lane == 0 && row == 0 && t == T / 2) {
            unsigned long long now;
            const int pin = *reinterpret_cast<volatile int*>(&failed_s);
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(now) : "r"(pin) : "memory");
            trace_s[58 + warp - 8] = now;   // when the producer and the issuers reach the barrier
        }
#endif
        RMARK(9);
        cl.sync();   // 3
        RMARK(10);

        // ---------------- E: the update of the block's slots (k = kl C + r)
        if (!producer && !issuer) {
            for (int e = tid; e < Ks * d; e += kConsumers) {
                const int kl = e / d, x = e - kl * d, k = kl * C + r;
                const bool ok = k < K && cell_of[k] >= 0;
                float F = 0.0f, G = 0.0f;
                for (int p = 0; p < C; ++p) {   // the blocks' partial sums in rank order
                    F += inbox_f[(p * Ks + kl) * 2 * d + x];
                    G += inbox_f[(p * Ks + kl) * 2 * d + d + x];
                }
                Fk[e] = ok ? bf16r(F + c.m.b2[unit_of[k] * d + x]) : 0.0f;
                gp[e] = ok ? bf16r(G + gate_b[x]) : 0.0f;
            }
            consumer_sync();
            RMARK(19);
            for (int e = tid; e < Ks * d; e += kConsumers) {
                const int kl = e / d, x = e - kl * d;
                ys[e] = bf16r(dot_bf16w(Fk + kl * d, 1, wout + x, d, d));
            }
            consumer_sync();
            RMARK(20);
            for (int kl = warp; kl < Ks; kl += kConsumers / 32) {
                float sq = 0.0f;
                for (int x = lane; x < d; x += 32) sq += ys[kl * d + x] * ys[kl * d + x];
                sq = warp_sum(sq);
                if (lane == 0) scale[kl] = rsqrtf(sq / static_cast<float>(d) + c.m.cand_eps);
            }
            consumer_sync();
            RMARK(21);
            for (int e = tid; e < Ks * d; e += kConsumers) {
                const int kl = e / d, x = e - kl * d, k = kl * C + r;
                if (k >= K) continue;
                const bool ok = cell_of[k] >= 0;
                float value = 0.0f, change = 0.0f, cv = 0.0f, bv = 0.0f;
                if (ok) {
                    const float old = hold[k * d + x];
                    cv = tanhf(ys[e] * scale[kl] * cand_w[x]);
                    bv = sigmoid_f(gp[e]);
                    value = (1.0f - bv) * old + bv * cv;
                    change = value - old;
                }
                hnew[e] = value;
                hb[e] = bf16r(value);
                Fk[e] = cv;   // F is spent: the candidate and the gate for the record, which the producer warp writes
                dl[e] = bv;
                for (int p = 0; p < C; ++p) peer(cl, inbox_delta, p)[k * d + x] = change;
                if (ok) {   // also before a reset: the position's max |h| and a padded slot's h_sel read it
                    const int cell = cell_of[k];
                    const int co = owner_of(cell);
                    peer(cl, h_s, co)[(cell - co * Nc) * d + x] = value;
                }
            }
            consumer_sync();
            {
                // the written cells' maxima, at their owners (their logit parts and V h follow in phase F)
                for (int kl = warp; kl < Ks; kl += kConsumers / 32) {
                    const int k = kl * C + r;
                    if (k >= K || cell_of[k] < 0) continue;
                    int top = 0;
                    for (int x = lane; x < d; x += 32) top = max(top, __float_as_int(fabsf(hnew[kl * d + x])));
                    for (int w = 16; w > 0; w >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, w));
                    const int co = owner_of(cell_of[k]);
                    if (lane == 0) peer(cl, cmax_s, co)[cell_of[k] - co * Nc] = top;
                }
            }
        }
        RMARK(11);
        cl.sync();   // 4
        RMARK(12);
        // ---------------- F: summary, ages, the tape's next record, the next reset
        if (producer) {
            // the position's records and the tape's next state record, from shared memory, by the warp
            // that takes part in no block barrier of the compute warps: its stores delay nobody. The
            // values stay where they are until the next position's phases D and E, which begin two
            // cluster barriers after this warp is done.
            if (rec) {
                for (int kl = 0; kl < Ks; ++kl) {
                    const int k = kl * C + r;
                    if (k >= K) continue;
                    const bool ok = cell_of[k] >= 0;
                    for (int x = lane; x < d; x += 32) {
                        const int e = kl * d + x;
                        const int64_t at = (rt * K + k) * d + x;
                        c.io.rec_c[at] = Fk[e];
                        c.io.rec_b[at] = dl[e];
                        c.io.rec_y[at] = ys[e];
                        c.io.rec_gate_pre[at] = gp[e];
                        c.io.rec_h_old[at] = hold[k * d + x];
                        c.io.rec_m[at] = msg[k * d + x];
                        if (ok) c.io.h_sel[at] = hnew[e];
                    }
                    if (lane == 0) c.io.rec_rms[rt * K + k] = rms[k];
                }
            } else {
                for (int kl = 0; kl < Ks; ++kl) {
                    const int k = kl * C + r;
                    if (k >= K || cell_of[k] < 0) continue;
                    for (int x = lane; x < d; x += 32) c.io.h_sel[(rt * K + k) * d + x] = hnew[kl * d + x];
                }
            }
            if (tape) {
                float4* dst = reinterpret_cast<float4*>(c.io.tape_h + ((static_cast<int64_t>(row) * (T + 1) + t + 1) * N + cell0) * d);
                const float4* from = reinterpret_cast<const float4*>(h_s);
                const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int e = lane; e < (Nc * d) >> 2; e += 32) dst[e] = clear ? zero4 : from[e];   // a reset: zeros, whatever the compute warps do to h_s meanwhile
            }
        }
        if (!producer && !issuer) {
            // no barrier in this phase unless the next position resets: every part reads what the
            // cluster barrier above published and writes its own data
            if (tid >= 96 && !clear) {
                // the written cells' logit parts and V h, at their owners, by the five warps that have
                // nothing else to do here; the next position reads them after its cluster barriers
                for (int o = tid - 96; o < Ks * (M + d); o += 160) {
                    const int kl = static_cast<int>(__umulhi(static_cast<uint32_t>(o), md_magic)), w = o - kl * (M + d), k = kl * C + r;
                    if (k >= K || cell_of[k] < 0) continue;
                    const int cell = cell_of[k], owner = owner_of(cell), cc = cell - owner * Nc;
                    const float* hr = hb + kl * d;
                    if (w < M) peer(cl, lh_s, owner)[cc * M + w] = dot4(hr, 1, swh + w, M, d);
                    else peer(cl, vh_s, owner)[cc * d + (w - M)] = bf16_bits(dot_bf16w(hr, 1, vt + (w - M), d, d));
                }
            }
            RMARK(31);
            for (int x = tid; x < d; x += kConsumers) {
                float sum = 0.0f;
                for (int k = 0; k < K; ++k) sum += inbox_delta[k * d + x];   // slot order
                const float after = q_s[x] + sum / static_cast<float>(N);
                q_after[x] = after;   // the producer warp writes qs and the tape's q after the next cluster barrier
                q_s[x] = clear ? 0.0f : after;
            }
            if (r == 0) {
                // a padded slot reads cell 0 after the position (reference compile.py: the tape's h_sel)
                for (int e = tid; e < K * d; e += kConsumers) {
                    const int k = e / d, x = e - k * d;
                    if (cell_of[k] < 0) c.io.h_sel[(rt * K + k) * d + x] = h_s[x];
                }
            }
            RMARK(34);
            {
                int top = 0;
                for (int n = tid; n < Nc; n += kConsumers) top = max(top, cmax_s[n]);
                for (int w = 16; w > 0; w >>= 1) top = max(top, __shfl_xor_sync(0xffffffffu, top, w));
                if (lane == 0 && top > 0) atomicMax(&hmax_local, top);   // a maximum: any order gives the same bits
            }
            RMARK(35);
            for (int n = tid; n < Nc; n += kConsumers) {
                int64_t a = age_s[n] + 1;
                for (int k = 0; k < K; ++k)
                    if (cell_of[k] == cell0 + n) a = 0;
                if (clear) a = 0;
                age_s[n] = a;   // the tape's ages likewise
            }
            if (clear) {
                consumer_sync();   // the reads of the state above are over
                for (int e = tid; e < Nc * d; e += kConsumers) {
                    h_s[e] = 0.0f;
                    vh_s[e] = 0;
                }
                for (int e = tid; e < Nc * M; e += kConsumers) lh_s[e] = 0.0f;
                for (int n = tid; n < Nc; n += kConsumers) cmax_s[n] = 0;
                consumer_sync();
            }
        }
        RMARK(13);
    }
    // the last position's max |h|, and the state the window ends in
    if (!producer && !issuer) consumer_sync();   // (every warp's share of the maximum is in)
    if (tid == 0) peer(cl, inbox_front, 0)[r * stride_in + 2 * d] = __int_as_float(hmax_local);
    cl.sync();
    if (producer) {
        const int64_t rp = static_cast<int64_t>(row) * T + T - 1;
        if (r == 0) {
            for (int x = lane; x < d; x += 32) {
                c.io.qs[rp * d + x] = q_after[x];
                if (tape) c.io.tape_q[(static_cast<int64_t>(row) * (T + 1) + T) * d + x] = q_after[x];
            }
        }
        if (tape)
            for (int n = lane; n < Nc; n += 32) c.io.tape_age[(static_cast<int64_t>(row) * (T + 1) + T) * N + cell0 + n] = age_s[n];
    }
    if (!producer && !issuer) {
        if (r == 0 && tid == 0) {
            if (c.io.h_max) {
                int mx = 0;
                for (int p = 0; p < C; ++p) mx = max(mx, __float_as_int(inbox_front[p * stride_in + 2 * d]));
                c.io.h_max[static_cast<int64_t>(row) * T + T - 1] = __int_as_float(mx);
            }
            int last_reset = 0;
            for (int s = 0; s < T; ++s)
                if (c.io.reset[static_cast<int64_t>(row) * T + s]) last_reset = s + 1;
            c.io.pos[row] = last_reset > 0 ? T + 1 - last_reset : c.io.pos[row] + T;
        }
        if (!tape) {
            float* h0 = c.io.h0 + (static_cast<int64_t>(row) * N + cell0) * d;
            for (int e = tid; e < Nc * d; e += kConsumers) h0[e] = h_s[e];
            int64_t* a0 = c.io.age0 + static_cast<int64_t>(row) * N + cell0;
            for (int n = tid; n < Nc; n += kConsumers) a0[n] = age_s[n];
            if (r == 0)
                for (int x = tid; x < d; x += kConsumers) c.io.q0[static_cast<int64_t>(row) * d + x] = q_s[x];
        }
    }
    tcgen05_fence_before();
    __syncthreads();
#ifdef HSNW_TRACE
    if (row == 0 && tid < 64) reinterpret_cast<unsigned long long*>(c.status + 64)[r * 64 + tid] = trace_s[tid];
    if (row == 0 && tid < 144) reinterpret_cast<unsigned long long*>(c.status + 64)[256 + r * 144 + tid] = (&utrace_s[0][0][0])[tid];
#endif
    if (warp == 0) tmem_dealloc(taddr, 512);
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// Host side: when the model and the window fit, hsnw_window_forward runs this kernel instead of
// the phases. Returns HSNW_OK when launched, HSNW_DECLINED when the shape does not fit (the caller runs
// the phases), a negative error code otherwise (the caller passes it on).
// ------------------------------------------------------------------------------------------------
static bool rows_shape(const HsnwModel& m, RowsCtx* c) {
    if (!m.prod_bf16 || m.phases_only || !m.rows_bank || !m.rows_front) return false;
    if (m.H % 128) return false;
    const int C = m.H / 128;
    if (C != 1 && C != 2 && C != 4 && C != 8) return false;
    if (m.N % C || m.N / C < 2 || (4 * m.d) % C || m.N > 2048) return false;   // (a block owns at least two cells: n / Nc is a multiply-high)
    if (m.d != 16 && m.d != 32 && m.d != 64) return false;
    if (m.K > kMaxK || m.M > kMaxMR || m.K < 1 || m.S > 16 || m.S < 1) return false;
    if (((m.N / C) * m.S) % 4) return false;   // the position's scalars of a block's cells move as one 16-byte aligned bulk copy
    c->C = C;
    c->Nc = m.N / C;
    c->Ks = (m.K + C - 1) / C;
    c->gate_rows = 4 * m.d / C;
    c->w1_bytes = static_cast<uint32_t>(512 * m.d);
    c->bank_bytes = static_cast<uint32_t>(1280 * m.d);
    c->front_bytes = static_cast<uint32_t>(512 * m.d);
    c->slot_bytes = c->w1_bytes;
    return true;
}

int hsnw_rows_forward(const HsnwModel* model, const HsnwForward* io, const float* pre_s, int* status, cudaStream_t stream) {
    RowsCtx c;
    if (!rows_shape(*model, &c)) return HSNW_DECLINED;
    if ((reinterpret_cast<uintptr_t>(io->scalars) | reinterpret_cast<uintptr_t>(io->z) | reinterpret_cast<uintptr_t>(pre_s)) & 15) return HSNW_DECLINED;
    c.stages = kMaxStages;
    RowsSmem L = rows_smem(*model, c.C, c.slot_bytes, c.stages);
    if (L.total + 2048 > hsnw_max_shared()) {
        c.stages = 2;
        L = rows_smem(*model, c.C, c.slot_bytes, c.stages);
        if (L.total + 2048 > hsnw_max_shared()) return HSNW_DECLINED;
    }
    c.m = *model;
    c.io = *io;
    c.pre_s = pre_s;
    c.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(io->B) * c.C, 1, 1);
    cfg.blockDim = dim3(kRowThreads, 1, 1);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(c.C);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void (*kernel)(RowsCtx) = model->d == 64 ? k_rows_fwd<64> : model->d == 32 ? k_rows_fwd<32> : k_rows_fwd<16>;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        return HSNW_DECLINED;   // no cluster of this size and shared memory fits the device
    }
    hsnw_profile_mark(HSNW_K_ROWS_FWD, stream);
    if (cudaLaunchKernelEx(&cfg, kernel, c) != cudaSuccess) return hsnw_check_launch("window_forward (row clusters)");
    return hsnw_check_launch("window_forward (row clusters)");
}

void hsnw_rows_set_attributes() {
    if (!hsnw_opt_in(reinterpret_cast<const void*>(k_rows_fwd<64>), "rows_fwd<64>")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_rows_fwd<32>), "rows_fwd<32>")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_rows_fwd<16>), "rows_fwd<16>"))
        hsnw_attribute_failed();
}
