// The trainer's per-step passes over lists of tensors (include/hsn_trainer_b200.h). Each pass is
// elementwise and HBM bound (AdamW: 16 bytes read, 12 written an element), so the layout is chosen
// for the memory system: the tensors of a launch are cut into runs of 1024 elements, a block takes
// a run at a time (grid-stride over the launch's runs, a few blocks an SM), a thread four
// consecutive elements as one 16-byte access per operand wherever the tensor's addresses and the
// run's end allow it, single elements otherwise. The tensor of a run is found once per run by a
// search over the launch's (at most 40) run counts in shared memory.
//
// Arithmetic: every step is one explicitly rounded operation (__fmul_rn, __fadd_rn, ... are never
// contracted), and a fused multiply-add stands exactly where PyTorch's CUDA kernels have one:
//   lerp(s, e, w) = fma(w, e - s, s) for |w| < 0.5, else fma(-(e - s), 1 - w, e);
//   addcmul(x, a, b, c) = fma(c, a * b, x), fma(a, b, x) for c = 1;
//   addcdiv(x, a, b, c) = fma(c, a / b, x), x + a / b for c = 1
// (reference kernels/cuda/hsn_trainer.cu:9-18 names the ATen sources).
#include "../../include/hsn_trainer_b200.h"
#include "../../include/hsn_window_b200.h"
#include "host_util.h"

#include <cstring>

namespace {

constexpr int kRun = 1024;       // elements of a run
constexpr int kThreads = 256;    // four elements a thread

__device__ __forceinline__ float lerp_rn(float self, float end, float w) {
    const float diff = __fsub_rn(end, self);
    return fabsf(w) < 0.5f ? __fmaf_rn(w, diff, self) : __fmaf_rn(-diff, __fsub_rn(1.0f, w), end);
}
__device__ __forceinline__ float addcmul_rn(float x, float a, float b, float c) {
    return c == 1.0f ? __fmaf_rn(a, b, x) : __fmaf_rn(c, __fmul_rn(a, b), x);
}
__device__ __forceinline__ float addcdiv_rn(float x, float a, float b, float c) {
    const float q = __fdiv_rn(a, b);
    return c == 1.0f ? __fadd_rn(x, q) : __fmaf_rn(c, q, x);
}

// An operation: READ / WRITE are bit masks of the rows it loads and stores as fp32 elements;
// apply() turns the loaded values x[row] of element o of tensor j into the stored ones.
struct AdamW {
    static constexpr int READ = 0xf, WRITE = 0xd;
    const HsnTrainArgs& a;
    __device__ void tensor(int, int64_t) {}
    __device__ void apply(float (&x)[4], int64_t) const {
        const float g = x[1];
        float p = x[0];
        if (a.i[1]) p = __fmul_rn(p, a.f[0]);
        const float m = lerp_rn(x[2], g, a.f[1]);
        const float v = addcmul_rn(__fmul_rn(x[3], a.f[2]), g, g, a.f[3]);
        const float den = __fadd_rn(__fmul_rn(__fsqrt_rn(v), a.f[4]), a.f[5]);
        x[0] = addcdiv_rn(p, m, den, a.f[6]);
        x[2] = m;
        x[3] = v;
    }
};
struct AdamWUnits {   // stacked [M, ...] tensors: the unit of element o is o / (elements / M)
    static constexpr int READ = 0xf, WRITE = 0xd;
    const HsnTrainArgs& a;
    uint32_t per_unit = 1;
    __device__ void tensor(int, int64_t count) { per_unit = static_cast<uint32_t>(count / a.i[2]); }
    __device__ void apply(float (&x)[4], int64_t o) const {
        const int unit = static_cast<int>(static_cast<uint32_t>(o) / per_unit);
        const float g = a.u[0][unit] != 0.0f ? x[1] : 0.0f;
        float p = x[0];
        if (a.i[1]) p = __fmul_rn(p, a.u[1][unit]);
        const float m = lerp_rn(x[2], g, a.u[2][unit]);
        const float v = addcmul_rn(__fmul_rn(x[3], a.u[3][unit]), g, g, a.f[3]);
        const float den = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), a.u[4][unit]), a.f[5]);
        x[0] = addcdiv_rn(p, __fmul_rn(m, a.u[5][unit]), den, -1.0f);
        x[2] = m;
        x[3] = v;
    }
};
struct Lerp {
    static constexpr int READ = 0x3, WRITE = 0x1;
    const HsnTrainArgs& a;
    __device__ void tensor(int, int64_t) {}
    __device__ void apply(float (&x)[4], int64_t) const { x[0] = lerp_rn(x[0], x[1], a.f[0]); }
};
struct Scale64 {   // grad = f32(f64(grad) * coefficient), the coefficient one float64 on the device
    static constexpr int READ = 0x1, WRITE = 0x1;
    const HsnTrainArgs& a;
    double coefficient = 0.0;
    __device__ void tensor(int, int64_t) { coefficient = *static_cast<const double*>(a.p[1][0]); }
    __device__ void apply(float (&x)[4], int64_t) const { x[0] = static_cast<float>(__dmul_rn(static_cast<double>(x[0]), coefficient)); }
};
struct Copy {
    static constexpr int READ = 0x2, WRITE = 0x1;
    const HsnTrainArgs& a;
    __device__ void tensor(int, int64_t) {}
    __device__ void apply(float (&x)[4], int64_t) const { x[0] = x[1]; }
};
struct LimitSquares {
    static constexpr int READ = 0x3, WRITE = 0xc;
    const HsnTrainArgs& a;
    __device__ void tensor(int, int64_t) {}
    __device__ void apply(float (&x)[4], int64_t) const {
        const float delta = __fsub_rn(x[0], x[1]);
        x[2] = __fmul_rn(x[1], x[1]);
        x[3] = __fmul_rn(delta, delta);
    }
};
struct LimitProject {   // param' = old + (param - old) scale where the tensor's group is clipped
    static constexpr int READ = 0x3, WRITE = 0x5;
    const HsnTrainArgs& a;
    float scale = 1.0f;
    bool clipped = false;
    __device__ void tensor(int j, int64_t) {
        const float* group = static_cast<const float*>(a.p[3][j]);
        scale = group[0];
        clipped = group[1] != 0.0f;
    }
    __device__ void apply(float (&x)[4], int64_t) const {
        if (clipped) x[0] = __fadd_rn(x[1], __fmul_rn(__fsub_rn(x[0], x[1]), scale));
        const float applied = __fsub_rn(x[0], x[1]);
        x[2] = __fmul_rn(applied, applied);
    }
};

template <class Op>
__global__ void __launch_bounds__(kThreads) k_table(const __grid_constant__ HsnTrainArgs a) {
    __shared__ int64_t run_end[HSN_TR_TENSORS];   // runs of the tensors 0 .. j, cumulative
    __shared__ int wide[HSN_TR_TENSORS];          // every operand of the tensor starts on a 16-byte boundary
    const int n = a.i[0], tid = threadIdx.x;
    if (tid < n) {
        bool ok = true;
        for (int r = 0; r < HSN_TR_ROWS; ++r)
            if ((Op::READ | Op::WRITE) >> r & 1) ok = ok && (reinterpret_cast<uintptr_t>(a.p[r][tid]) & 15) == 0;
        wide[tid] = ok ? 1 : 0;
    }
    if (tid == 0) {
        int64_t runs = 0;
        for (int j = 0; j < n; ++j) {
            const int64_t count = a.end[j] - (j ? a.end[j - 1] : 0);
            runs += (count + kRun - 1) / kRun;
            run_end[j] = runs;
        }
    }
    __syncthreads();
    const int64_t total = run_end[n - 1];
    Op op{a};
    int at = -1;   // the tensor the operation is set up for
    for (int64_t run = blockIdx.x; run < total; run += gridDim.x) {
        int lo = 0, hi = n - 1;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (run_end[mid] > run) hi = mid;
            else lo = mid + 1;
        }
        const int j = lo;
        const int64_t count = a.end[j] - (j ? a.end[j - 1] : 0);
        if (j != at) {
            op.tensor(j, count);
            at = j;
        }
        const int64_t o = (run - (j ? run_end[j - 1] : 0)) * kRun + 4 * tid;
        if (o >= count) continue;
        float x[4][4];   // [element][row]
        if (wide[j] && o + 4 <= count) {
#pragma unroll
            for (int r = 0; r < HSN_TR_ROWS; ++r)
                if (Op::READ >> r & 1) {
                    const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(a.p[r][j]) + o);
                    x[0][r] = v.x; x[1][r] = v.y; x[2][r] = v.z; x[3][r] = v.w;
                }
#pragma unroll
            for (int e = 0; e < 4; ++e) op.apply(x[e], o + e);
#pragma unroll
            for (int r = 0; r < HSN_TR_ROWS; ++r)
                if (Op::WRITE >> r & 1)
                    *reinterpret_cast<float4*>(static_cast<float*>(a.p[r][j]) + o) = make_float4(x[0][r], x[1][r], x[2][r], x[3][r]);
        } else {
            for (int e = 0; e < 4 && o + e < count; ++e) {
#pragma unroll
                for (int r = 0; r < HSN_TR_ROWS; ++r)
                    if (Op::READ >> r & 1) x[0][r] = static_cast<const float*>(a.p[r][j])[o + e];
                op.apply(x[0], o + e);
#pragma unroll
                for (int r = 0; r < HSN_TR_ROWS; ++r)
                    if (Op::WRITE >> r & 1) static_cast<float*>(a.p[r][j])[o + e] = x[0][r];
            }
        }
    }
}

template <class Op>
int launch(const HsnTrainArgs& a, int64_t runs, cudaStream_t stream) {
    const int64_t cap = static_cast<int64_t>(hsnw_sm_count_current()) * 8;   // eight resident blocks an SM
    const unsigned grid = static_cast<unsigned>(runs < cap ? runs : cap);
    k_table<Op><<<grid, kThreads, 0, stream>>>(a);
    return hsnw_check_launch("launch_table");
}

}  // namespace

namespace {

// One thread: four consecutive elements of the rank's shard (the shard is a multiple of four elements and
// every buffer 16-byte aligned: checked on the host). Loads from the peers' gradients are issued together,
// then summed in rank order.
__global__ void __launch_bounds__(kThreads) k_exchange_adamw(const __grid_constant__ HsnwExchange x) {
    constexpr int U = 2;   // quads a thread has in flight: the peers' memory is microseconds away
    const int64_t quads = x.shard >> 2;
    const int64_t base = static_cast<int64_t>(x.rank) * x.shard;
    const float inv = 1.0f / static_cast<float>(x.world);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t q0 = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; q0 < quads; q0 += U * stride) {
        float4 part[U][HSN_EX_RANKS], p4[U], m4[U], v4[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t e = 4 * (q0 + u * stride);
            if (q0 + u * stride >= quads) continue;
#pragma unroll
            for (int k = 0; k < HSN_EX_RANKS; ++k)
                if (k < x.world) part[u][k] = *reinterpret_cast<const float4*>(x.grads[k] + base + e);
            p4[u] = *reinterpret_cast<const float4*>(x.params[x.rank] + base + e);
            m4[u] = *reinterpret_cast<const float4*>(x.exp_avg + e);
            v4[u] = *reinterpret_cast<const float4*>(x.exp_avg_sq + e);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t e = 4 * (q0 + u * stride);
            if (q0 + u * stride >= quads) continue;
            float g[4] = {part[u][0].x, part[u][0].y, part[u][0].z, part[u][0].w};
#pragma unroll
            for (int k = 1; k < HSN_EX_RANKS; ++k)
                if (k < x.world) {   // rank order: every rank computes the same bits
                    g[0] = __fadd_rn(g[0], part[u][k].x);
                    g[1] = __fadd_rn(g[1], part[u][k].y);
                    g[2] = __fadd_rn(g[2], part[u][k].z);
                    g[3] = __fadd_rn(g[3], part[u][k].w);
                }
            float p[4] = {p4[u].x, p4[u].y, p4[u].z, p4[u].w}, m[4] = {m4[u].x, m4[u].y, m4[u].z, m4[u].w},
                  v[4] = {v4[u].x, v4[u].y, v4[u].z, v4[u].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float gi = x.average ? __fmul_rn(g[i], inv) : g[i];
                if (x.weight_decay_on) p[i] = __fmul_rn(p[i], x.f[0]);
                m[i] = lerp_rn(m[i], gi, x.f[1]);
                v[i] = addcmul_rn(__fmul_rn(v[i], x.f[2]), gi, gi, x.f[3]);
                const float den = __fadd_rn(__fmul_rn(__fsqrt_rn(v[i]), x.f[4]), x.f[5]);
                p[i] = addcdiv_rn(p[i], m[i], den, x.f[6]);
            }
            *reinterpret_cast<float4*>(x.exp_avg + e) = make_float4(m[0], m[1], m[2], m[3]);
            *reinterpret_cast<float4*>(x.exp_avg_sq + e) = make_float4(v[0], v[1], v[2], v[3]);
            const float4 out = make_float4(p[0], p[1], p[2], p[3]);
#pragma unroll
            for (int k = 0; k < HSN_EX_RANKS; ++k)
                if (k < x.world) *reinterpret_cast<float4*>(x.params[k] + base + e) = out;
        }
    }
}

}  // namespace

extern "C" int hsnw_exchange_adamw(const HsnwExchange* exchange, void* stream_) {
    if (!exchange) return hsnw_fail(HSNW_E_ARG, "exchange_adamw: null argument");
    const HsnwExchange& x = *exchange;
    if (x.world < 1 || x.world > HSN_EX_RANKS || x.rank < 0 || x.rank >= x.world) return hsnw_fail(HSNW_E_ARG, "exchange_adamw: world must be 1..8 and rank inside it");
    if (x.shard < 4 || x.shard % 4) return hsnw_fail(HSNW_E_ARG, "exchange_adamw: the shard must be a positive multiple of 4 elements");
    uintptr_t bits = reinterpret_cast<uintptr_t>(x.exp_avg) | reinterpret_cast<uintptr_t>(x.exp_avg_sq);
    if (!x.exp_avg || !x.exp_avg_sq) return hsnw_fail(HSNW_E_ARG, "exchange_adamw: the moments are missing");
    for (int k = 0; k < x.world; ++k) {
        if (!x.grads[k] || !x.params[k]) return hsnw_fail(HSNW_E_ARG, "exchange_adamw: a rank's buffer is missing");
        bits |= reinterpret_cast<uintptr_t>(x.grads[k]) | reinterpret_cast<uintptr_t>(x.params[k]);
    }
    if (bits & 15) return hsnw_fail(HSNW_E_ARG, "exchange_adamw: every buffer must start on a 16-byte boundary");
    const int64_t blocks = (x.shard / 4 + kThreads - 1) / kThreads;
    const int64_t cap = static_cast<int64_t>(hsnw_sm_count_current()) * 8;
    k_exchange_adamw<<<static_cast<unsigned>(blocks < cap ? blocks : cap), kThreads, 0, static_cast<cudaStream_t>(stream_)>>>(x);
    return hsnw_check_launch("exchange_adamw");
}

extern "C" int hsnw_launch_table(const char* name, const HsnTrainArgs* args, void* stream_) {
    if (!name || !args) return hsnw_fail(HSNW_E_ARG, "launch_table: null argument");
    const HsnTrainArgs& a = *args;
    const int n = a.i[0];
    if (n < 1 || n > HSN_TR_TENSORS) return hsnw_fail(HSNW_E_ARG, "launch_table: i[0] must be 1..40 tensors");
    int64_t runs = 0, before = 0;
    for (int j = 0; j < n; ++j) {
        if (a.end[j] <= before) return hsnw_fail(HSNW_E_ARG, "launch_table: end[] must increase (no empty tensors)");
        runs += (a.end[j] - before + kRun - 1) / kRun;
        before = a.end[j];
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int need = 0;   // rows that must be addresses of every tensor
    int rc;
    if (!std::strcmp(name, "hsn_tr_adamw")) need = 0xf;
    else if (!std::strcmp(name, "hsn_tr_adamw_units")) need = 0xf;
    else if (!std::strcmp(name, "hsn_tr_lerp")) need = 0x3;
    else if (!std::strcmp(name, "hsn_tr_scale64")) need = 0x1;
    else if (!std::strcmp(name, "hsn_tr_copy")) need = 0x3;
    else if (!std::strcmp(name, "hsn_tr_limit_squares")) need = 0xf;
    else if (!std::strcmp(name, "hsn_tr_limit_project")) need = 0xf;
    else return hsnw_fail(HSNW_E_NAME, "launch_table: no trainer kernel of that name");
    for (int r = 0; r < HSN_TR_ROWS; ++r)
        for (int j = 0; j < n; ++j)
            if ((need >> r & 1) && !a.p[r][j]) return hsnw_fail(HSNW_E_ARG, "launch_table: a row the kernel reads is null");
    if (!std::strcmp(name, "hsn_tr_adamw")) rc = launch<AdamW>(a, runs, stream);
    else if (!std::strcmp(name, "hsn_tr_adamw_units")) {
        if (a.i[2] < 1 || a.i[2] > HSN_TR_UNITS) return hsnw_fail(HSNW_E_ARG, "launch_table: i[2] must be 1..64 units");
        before = 0;
        for (int j = 0; j < n; ++j) {
            if ((a.end[j] - before) % a.i[2]) return hsnw_fail(HSNW_E_ARG, "launch_table: a unit tensor's elements must divide by its units");
            before = a.end[j];
        }
        rc = launch<AdamWUnits>(a, runs, stream);
    } else if (!std::strcmp(name, "hsn_tr_lerp")) rc = launch<Lerp>(a, runs, stream);
    else if (!std::strcmp(name, "hsn_tr_scale64")) {
        if (!a.p[1][0]) return hsnw_fail(HSNW_E_ARG, "launch_table: scale64 needs its coefficient at p[1][0]");
        rc = launch<Scale64>(a, runs, stream);
    } else if (!std::strcmp(name, "hsn_tr_copy")) rc = launch<Copy>(a, runs, stream);
    else if (!std::strcmp(name, "hsn_tr_limit_squares")) rc = launch<LimitSquares>(a, runs, stream);
    else rc = launch<LimitProject>(a, runs, stream);
    return rc;
}
