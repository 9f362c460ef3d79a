// The router's hard decision for one batch row, by the whole thread block that owns the row.
//
// Follows Router.select with mode "topk" (reference python/hsn/model/router.py:1263-1417):
//   _topk       :1640-1648  descending by score, equal scores in index order (a stable sort);
//                           the unit of a cell is the first maximiser of its scores
//   _truncate   :1650-1657  the longest prefix of the slots whose cumulative cost fits the limit
//   _ste_threshold :1771-1786, the refresh probes of _post_process :1788-1850
// and keeps the contract of the reference kernel hsn_win_select (kernels/cuda/hsn_window.cu:533-562).
//
// Method: a cell's (score, index) pair is packed into one 64-bit key whose unsigned order is
// "higher score first, then lower index", so all keys differ. Slot r takes the largest key below
// slot r-1's: K rounds of a warp-shuffle maximum (lanes fold 64-bit keys with shuffles, the
// warps' maxima are folded by the first warp). No rank counting, no sort, no atomics: the result
// does not depend on thread scheduling. The probes use the same rounds on (age, index) keys.
#pragma once
#include "common.cuh"

namespace hsnw {

constexpr int kMaxSlots = 64;   // K of a row
constexpr int kMaxUnits = 64;   // M

struct SelectParams {
    int N, M, K;
    int age_max;
    int probes;
    int reserved;      // amendment A8: cells 0..reserved-1 hold the first slots
    int fixed_units;   // and slot k < reserved runs unit k mod M
    float overhead, shared_cost, limit;
};

// Shared-memory working set of a decision (the [N]-sized arrays are the caller's).
struct SelectShared {
    uint64_t red[33];
    float cost[kMaxUnits];
    int order[kMaxSlots];      // the scored decision's cells, slot by slot
    int out_cell[kMaxSlots];
    int out_unit[kMaxSlots];
    int out_flag[kMaxSlots];   // bit 0 valid, bit 1 refreshed
    int n_valid;
    float theta;
};

// score[N], unit[N]: shared memory, filled by the caller (score_i = max_j(logit_ij - lambda c_j),
// unit_i its first maximiser); age_row: the row's ages (global or shared; read only with probes).
// Every thread of the block calls this; the results are in S.out_* / S.theta after the trailing
// barrier.
__device__ __forceinline__ void select_row(const SelectParams& P, const float* score, const int* unit,
                                           const int64_t* age_row, SelectShared& S) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int N = P.N, K = P.K, F = P.reserved;
    uint64_t prev = ~0ull;
    for (int r = 0; r < K; ++r) {
        if (r < F) {
            if (tid == 0) S.order[r] = r;
            continue;
        }
        uint64_t best = 0ull;
        for (int i = F + tid; i < N; i += nt) {
            const uint64_t key = pack_key(score[i], i);
            if (key < prev && key > best) best = key;
        }
        best = block_max_u64(best, S.red);
        if (tid == 0) S.order[r] = best ? key_cell(best) : 0;
        prev = best;
    }
    __syncthreads();
    if (tid == 0) {
        // the budget: the longest prefix that fits, the costs summed in slot order
        float cumulative = 0.0f;
        int n_valid = 0;
        for (int k = 0; k < K; ++k) {
            const int c = S.order[k];
            const int u = (P.fixed_units && k < F) ? k % P.M : unit[c];
            cumulative += P.overhead + S.cost[u];
            const bool ok = P.shared_cost + cumulative <= P.limit;
            S.out_cell[k] = ok ? c : 0;
            S.out_unit[k] = ok ? u : 0;
            S.out_flag[k] = ok ? 1 : 0;
            n_valid += ok ? 1 : 0;
        }
        S.n_valid = n_valid;
    }
    __syncthreads();
    const int n_valid = S.n_valid;
    const bool any_scored = n_valid > F;
    const int last = any_scored ? S.order[n_valid - 1] : 0;
    const float lowest_in = any_scored ? score[last] : INFINITY;
    const uint64_t in_key = any_scored ? pack_key(score[last], last) : ~0ull;
    // the straight-through threshold: midway between the lowest selected (scored slots only) and
    // the highest unselected score
    float high = -INFINITY;
    int stale = 0;
    for (int i = tid; i < N; i += nt) {
        const bool chosen = i < F ? i < n_valid : (any_scored && pack_key(score[i], i) >= in_key);
        if (!chosen) {
            high = fmaxf(high, score[i]);
            if (P.probes && age_row[i] > static_cast<int64_t>(P.age_max)) ++stale;
        }
    }
    high = block_max_float(high, S.red);
    if (tid == 0) S.theta = 0.5f * (lowest_in + high);
    if (P.probes) {
        // the stalest unselected cells (equal ages in index order) take the valid scored slots
        // from the last one backwards
        const int n_stale = block_sum_int(stale, S.red);
        const int scored = any_scored ? n_valid - F : 0;
        const int n_force = n_stale < scored ? n_stale : scored;
        uint64_t before = ~0ull;
        for (int j = 0; j < n_force; ++j) {
            uint64_t best = 0ull;
            for (int i = tid; i < N; i += nt) {
                const bool chosen = i < F ? i < n_valid : (any_scored && pack_key(score[i], i) >= in_key);
                const int64_t ag = age_row[i];
                if (!chosen && ag > static_cast<int64_t>(P.age_max)) {
                    const uint64_t key = pack_key(static_cast<float>(ag), i);
                    if (key < before && key > best) best = key;
                }
            }
            best = block_max_u64(best, S.red);
            before = best;
            if (tid == 0) {
                const int pick = key_cell(best), k = n_valid - 1 - j;
                S.out_cell[k] = pick;
                S.out_unit[k] = unit[pick];
                S.out_flag[k] |= 2;
            }
        }
        __syncthreads();
        if (tid == 0 && n_force > 0) {
            // a row the probes pushed over the limit keeps its scored decision
            float spent = 0.0f;
            for (int k = 0; k < K; ++k)
                spent += (S.out_flag[k] & 1) ? P.overhead + S.cost[S.out_unit[k]] : 0.0f;
            if (P.shared_cost + spent > P.limit) {
                for (int k = 0; k < K; ++k) {
                    const bool ok = (S.out_flag[k] & 1) != 0;
                    const int c = S.order[k];
                    const int u = (P.fixed_units && k < F) ? k % P.M : unit[c];
                    S.out_cell[k] = ok ? c : 0;
                    S.out_unit[k] = ok ? u : 0;
                    S.out_flag[k] &= 1;
                }
            }
        }
    }
    __syncthreads();
}

// The same decision by ONE warp (no reserved cells), for rows of up to a few thousand cells: the
// whole selection then needs no block barrier. Lane l owns the cells l, l + 32, ...; it keeps its
// best remaining key, the warp takes the maximum with two redux instructions (the score half,
// then the index half among the lanes that hold that score), and only the winner's lane rescans
// its cells. Called by every lane of one warp; the other warps wait at the caller's barrier.
__device__ __forceinline__ uint64_t warp_argmax_key(uint64_t mine) {
    const uint32_t hi = __reduce_max_sync(0xffffffffu, static_cast<uint32_t>(mine >> 32));
    const uint32_t lo = __reduce_max_sync(0xffffffffu, static_cast<uint32_t>(mine >> 32) == hi ? static_cast<uint32_t>(mine) : 0u);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

// The rest of the decision once the scored order is known (S.order[0..K) and next_key, the
// (K + 1)-th best key or 0): the budget prefix, the threshold, the probes. One warp.
__device__ __forceinline__ void select_finish_warp(const SelectParams& P, const float* score, const int* unit,
                                                   const int64_t* age_row, SelectShared& S, uint64_t next_key) {
    const int lane = threadIdx.x & 31;
    const int N = P.N, K = P.K;
    __syncwarp();
    int n_valid = 0;
    if (lane == 0) {
        float cumulative = 0.0f;
        for (int k = 0; k < K; ++k) {
            const int c = S.order[k];
            const int u = unit[c];
            cumulative += P.overhead + S.cost[u];
            const bool ok = P.shared_cost + cumulative <= P.limit;
            S.out_cell[k] = ok ? c : 0;
            S.out_unit[k] = ok ? u : 0;
            S.out_flag[k] = ok ? 1 : 0;
            n_valid += ok ? 1 : 0;
        }
        S.n_valid = n_valid;
    }
    n_valid = __shfl_sync(0xffffffffu, n_valid, 0);
    __syncwarp();
    const bool any = n_valid > 0;
    const int last = any ? S.order[n_valid - 1] : 0;
    const uint64_t in_key = any ? pack_key(score[last], last) : ~0ull;
    // the highest unselected score: the first slot the budget cut, else the (K + 1)-th best
    float high;
    if (n_valid < K) high = score[S.order[n_valid]];
    else high = next_key ? score[key_cell(next_key)] : -INFINITY;
    if (lane == 0) S.theta = 0.5f * ((any ? score[last] : INFINITY) + high);
    if (P.probes) {
        int stale = 0;
        uint64_t oldest = 0ull;
        for (int i = lane; i < N; i += 32) {
            const bool chosen = any && pack_key(score[i], i) >= in_key;
            const int64_t ag = age_row[i];
            if (!chosen && ag > static_cast<int64_t>(P.age_max)) {
                ++stale;
                const uint64_t key = pack_key(static_cast<float>(ag), i);
                oldest = key > oldest ? key : oldest;
            }
        }
        const int n_stale = __reduce_add_sync(0xffffffffu, stale);
        const int n_force = n_stale < n_valid ? n_stale : n_valid;
        for (int j = 0; j < n_force; ++j) {
            const uint64_t win = warp_argmax_key(oldest);
            const int pick = key_cell(win);
            if (lane == 0) {
                const int k = n_valid - 1 - j;
                S.out_cell[k] = pick;
                S.out_unit[k] = unit[pick];
                S.out_flag[k] |= 2;
            }
            if ((pick & 31) == lane) {
                uint64_t best = 0ull;
                for (int i = lane; i < N; i += 32) {
                    const bool chosen = any && pack_key(score[i], i) >= in_key;
                    const int64_t ag = age_row[i];
                    if (!chosen && ag > static_cast<int64_t>(P.age_max)) {
                        const uint64_t key = pack_key(static_cast<float>(ag), i);
                        if (key < win && key > best) best = key;
                    }
                }
                oldest = best;
            }
        }
        __syncwarp();
        if (lane == 0 && n_force > 0) {
            float spent = 0.0f;
            for (int k = 0; k < K; ++k)
                spent += (S.out_flag[k] & 1) ? P.overhead + S.cost[S.out_unit[k]] : 0.0f;
            if (P.shared_cost + spent > P.limit) {
                for (int k = 0; k < K; ++k) {
                    const bool ok = (S.out_flag[k] & 1) != 0;
                    const int c = S.order[k];
                    S.out_cell[k] = ok ? c : 0;
                    S.out_unit[k] = ok ? unit[c] : 0;
                    S.out_flag[k] &= 1;
                }
            }
        }
    }
    __syncwarp();
}

__device__ __forceinline__ void select_row_warp(const SelectParams& P, const float* score, const int* unit,
                                                const int64_t* age_row, SelectShared& S) {
    const int lane = threadIdx.x & 31;
    const int N = P.N, K = P.K;
    // the scored decision: K + 1 rounds (the extra one is the highest unselected score)
    uint64_t mine = 0ull;
    for (int i = lane; i < N; i += 32) {
        const uint64_t key = pack_key(score[i], i);
        mine = key > mine ? key : mine;
    }
    uint64_t next_key = 0ull;
    for (int r = 0; r <= K; ++r) {
        const uint64_t win = warp_argmax_key(mine);
        if (r < K) {
            if (lane == 0) S.order[r] = win ? key_cell(win) : 0;
        } else {
            next_key = win;
        }
        if (win && (key_cell(win) & 31) == lane) {  // the winner's lane moves on to its next best
            uint64_t best = 0ull;
            for (int i = lane; i < N; i += 32) {
                const uint64_t key = pack_key(score[i], i);
                if (key < win && key > best) best = key;
            }
            mine = best;
        }
    }
    select_finish_warp(P, score, unit, age_row, S, next_key);
}

// The same scored order found by several warps: each warp first reduces the cells first, first +
// stride, ... (first = its first thread's index in the group, stride = the group's thread count)
// to its K + 1 best keys (select_candidates_warp, all warps at once), then ONE warp merges the
// warps' candidates (select_merge_warp) and finishes. cand: [warps][K + 1] keys in shared memory.
__device__ __forceinline__ void select_candidates_warp(int N, int K, const float* score, uint64_t* cand_row, int first,
                                                       int stride) {
    const int lane = threadIdx.x & 31;
    uint64_t mine = 0ull;
    for (int i = first + lane; i < N; i += stride) {
        const uint64_t key = pack_key(score[i], i);
        mine = key > mine ? key : mine;
    }
    for (int r = 0; r <= K; ++r) {
        const uint64_t win = warp_argmax_key(mine);
        if (lane == 0) cand_row[r] = win;
        if (win && mine == win) {   // keys are unique: exactly one lane holds the winner
            uint64_t best = 0ull;
            for (int i = first + lane; i < N; i += stride) {
                const uint64_t key = pack_key(score[i], i);
                if (key < win && key > best) best = key;
            }
            mine = best;
        }
    }
}
__device__ __forceinline__ void select_merge_warp(const SelectParams& P, const float* score, const int* unit,
                                                  const int64_t* age_row, const uint64_t* cand, int n_cand,
                                                  SelectShared& S) {
    const int lane = threadIdx.x & 31;
    const int K = P.K;
    uint64_t mine = 0ull;
    for (int i = lane; i < n_cand; i += 32) mine = cand[i] > mine ? cand[i] : mine;
    uint64_t next_key = 0ull;
    for (int r = 0; r <= K; ++r) {
        const uint64_t win = warp_argmax_key(mine);
        if (r < K) {
            if (lane == 0) S.order[r] = win ? key_cell(win) : 0;
        } else {
            next_key = win;
        }
        if (win && mine == win) {
            uint64_t best = 0ull;
            for (int i = lane; i < n_cand; i += 32)
                if (cand[i] < win && cand[i] > best) best = cand[i];
            mine = best;
        }
    }
    select_finish_warp(P, score, unit, age_row, S, next_key);
}

}  // namespace hsnw
