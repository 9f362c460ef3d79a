// The window's epilogue on the device: the decoder D([q_t; u_t]) = fc2(act(fc1(.))) over all the
// window's (or the serving step's) rows at once (reference python/hsn/model/hsn.py:2374-2390,
// python/hsn/model/encoder.py:128-206: MLP2 with biases, exact-erf GELU; under autocast every
// linear's operands, bias and output are bfloat16, its sums float32).
//
// Two dense layers over R = B T rows: with bf16 products each is a tcgen05 tile product, a 128 x 128
// output tile per block, K in chunks of 128 staged as K-major core-matrix planes (both operands are
// converted to bfloat16 while they are staged; the weights are nn.Linear's [out, in], so a plane of 8
// inputs is 32 contiguous bytes of a weight row), the chunks' products accumulating in tensor memory;
// the epilogue adds the bias, rounds, applies the activation for the first layer. With fp32 products
// a CUDA-core kernel (sums in input order).
#include "../../include/hsn_window_b200.h"
#include "common.cuh"
#include "stage.cuh"
#include "host_util.h"
#include "umma.cuh"

using namespace hsnw;

namespace {

constexpr int kChunk = 128;   // inputs staged at a time: 2 x 32 KB of operands

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&pair);
}

// out[r, c] = f(sum_k x[r, k] w[c, k] + b[c]); x = [in0 | in1] (in1 may be null: d1 = 0)
// BN: the columns of a block's tile (128; 32 when there are few rows, so that a serving step still fills the SMs)
template <bool GELU, int BN>
__global__ void __launch_bounds__(128) k_linear_tc(const float* in0, int d0, const float* in1, int d1, const float* w, const float* bias,
                                                   int64_t rows, int n_out, float* out, int* status) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int K = d0 + d1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * 128;
    const int c0 = blockIdx.y * BN;
    uint4* As = reinterpret_cast<uint4*>(dyn);
    uint4* Bs = As + (kChunk / 8) * 128;
    if (tid == 0) mbar_init(&bar, 1);
    if (warp == 0) tmem_alloc(&tmem_slot, BN);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t taddr = tmem_slot;
    const uint32_t idesc = umma_idesc_bf16(128, BN);
    int phase = 0;
    for (int k0 = 0; k0 < K; k0 += kChunk, ++phase) {
        const int kc_n = min(kChunk, ((K - k0) + 15) & ~15) >> 3;   // planes of this chunk (whole K = 16 steps)
        for (int idx = tid; idx < kc_n * 128; idx += 128) {
            const int r = idx & 127, kc = idx >> 7;
            const int k = k0 + kc * 8;           // eight consecutive inputs; d0 is a multiple of 8
            const int64_t row = r0 + r;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
            if (row < rows && k < K) {
                const float* src = k < d0 ? in0 + row * d0 + k : in1 + row * d1 + (k - d0);
                const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
            As[idx] = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
        }
        for (int idx = tid; idx < kc_n * BN; idx += 128) {
            const int r = idx % BN, kc = idx / BN;
            const int k = k0 + kc * 8;
            const int col = c0 + r;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
            if (col < n_out && k < K) {
                const float* src = w + static_cast<int64_t>(col) * K + k;
                const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
            Bs[idx] = make_uint4(pack2(v[0], v[1]), pack2(v[2], v[3]), pack2(v[4], v[5]), pack2(v[6], v[7]));
        }
        fence_async_smem();
        __syncthreads();
        if (tid < 32) {   // the whole first warp, converged after the barrier: one elected lane issues
            tcgen05_fence_after();
            umma_chain(taddr, umma_desc(As, 128), umma_desc(Bs, BN), idesc, kc_n >> 1, umma_kstep(128), umma_kstep(BN), k0 > 0);
            umma_commit(&bar);
        }
        mbar_wait(&bar, phase & 1, status);   // the products have read the operands: the next chunk may be staged
        tcgen05_fence_after();
    }
    const int64_t row = r0 + warp * 32 + lane;
    for (int cb = 0; cb < BN; cb += 8) {
        float acc[8];
        tmem_ld8(tmem_addr(taddr, warp * 32, cb), acc);
        if (row < rows) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int col = c0 + cb + i;
                if (col < n_out) {
                    float y = bf16r(acc[i] + bf16r(bias[col]));
                    if (GELU) y = bf16r(gelu_erf(y));
                    out[row * n_out + col] = y;
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, BN);
}

// fp32 products: a block takes 8 rows (staged in shared memory), a warp an output at a time with its lanes
// along the weight row; the sum of a row's products in lane-strided partial sums, then a shuffle tree.
template <bool GELU>
__global__ void __launch_bounds__(256) k_linear_f32(const float* in0, int d0, const float* in1, int d1, const float* w, const float* bias,
                                                    int64_t rows, int n_out, float* out) {
    extern __shared__ __align__(16) unsigned char dyn[];
    float* x = reinterpret_cast<float*>(dyn);   // [8][K]
    const int K = d0 + d1, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * 8;
    for (int e = tid; e < 8 * K; e += 256) {
        const int r = e / K, k = e - r * K;
        const int64_t row = r0 + r;
        x[e] = row < rows ? (k < d0 ? in0[row * d0 + k] : in1[row * d1 + (k - d0)]) : 0.0f;
    }
    __syncthreads();
    for (int col = warp; col < n_out; col += 8) {
        const float* wr = w + static_cast<int64_t>(col) * K;
        float sum[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        for (int k = lane; k < K; k += 32) {
            const float wv = wr[k];
#pragma unroll
            for (int r = 0; r < 8; ++r) sum[r] += x[r * K + k] * wv;
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float total = warp_sum(sum[r]);
            if (lane == 0 && r0 + r < rows) {
                float y = total + bias[col];
                if (GELU) y = gelu_erf(y);
                out[(r0 + r) * n_out + col] = y;
            }
        }
    }
}

size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace

extern "C" int64_t hsnw_decode_scratch_bytes(const HsnwDecoder* dec, int64_t rows) {
    if (!dec || rows < 1 || dec->H < 1) return 0;
    return static_cast<int64_t>(256 + up256(sizeof(float) * static_cast<size_t>(rows) * dec->H));
}

extern "C" int hsnw_window_decode(const HsnwDecoder* dec, const float* qs, const float* us, int64_t rows, float* logits, void* scratch,
                                  int64_t scratch_bytes, void* stream_) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (!dec || !qs || !logits || rows < 1) return hsnw_fail(HSNW_E_ARG, "window_decode: null or empty");
    if (dec->d_q < 1 || dec->d_u < 0 || dec->H < 1 || dec->V < 1 || !dec->w1 || !dec->b1 || !dec->w2 || !dec->b2 || (dec->d_u > 0 && !us))
        return hsnw_fail(HSNW_E_ARG, "window_decode: sizes or weights missing");
    if (!scratch || scratch_bytes < hsnw_decode_scratch_bytes(dec, rows) || (reinterpret_cast<uintptr_t>(scratch) & 255))
        return hsnw_fail(HSNW_E_ARG, "window_decode: scratch too small or not 256-byte aligned (hsnw_decode_scratch_bytes)");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int* status = static_cast<int*>(scratch);
    float* hidden = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + 256);
    if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) return hsnw_check_launch("window_decode");
    const int K1 = dec->d_q + dec->d_u;
    if (dec->prod_bf16) {
        // 16-byte loads of eight consecutive inputs: both parts and the hidden width in multiples of 8, aligned rows
        if (dec->d_q % 8 || dec->d_u % 8 || dec->H % 8
            || ((reinterpret_cast<uintptr_t>(qs) | reinterpret_cast<uintptr_t>(us) | reinterpret_cast<uintptr_t>(dec->w1)
                 | reinterpret_cast<uintptr_t>(dec->w2)) & 15))
            return hsnw_fail(HSNW_E_UNSUPPORTED, "window_decode: bf16 products need widths in multiples of 8 and 16-byte aligned operands");
        const size_t shared = static_cast<size_t>(2) * (kChunk / 8) * 128 * 16;
        const unsigned row_tiles = static_cast<unsigned>((rows + 127) / 128);
        hsnw_profile_mark(HSNW_K_DECODE, stream);
        // few rows (a serving step): 32-column tiles, four times the blocks
        if (row_tiles * ((dec->H + 127) / 128) >= 64)
            k_linear_tc<true, 128><<<dim3(row_tiles, (dec->H + 127) / 128), 128, shared, stream>>>(qs, dec->d_q, us, dec->d_u, dec->w1, dec->b1,
                                                                                                   rows, dec->H, hidden, status);
        else
            k_linear_tc<true, 32><<<dim3(row_tiles, (dec->H + 31) / 32), 128, shared, stream>>>(qs, dec->d_q, us, dec->d_u, dec->w1, dec->b1, rows,
                                                                                                dec->H, hidden, status);
        if (int rc = hsnw_check_launch("window_decode")) return rc;
        hsnw_profile_mark(HSNW_K_DECODE, stream);
        if (row_tiles * ((dec->V + 127) / 128) >= 64)
            k_linear_tc<false, 128><<<dim3(row_tiles, (dec->V + 127) / 128), 128, shared, stream>>>(hidden, dec->H, nullptr, 0, dec->w2, dec->b2,
                                                                                                    rows, dec->V, logits, status);
        else
            k_linear_tc<false, 32><<<dim3(row_tiles, (dec->V + 31) / 32), 128, shared, stream>>>(hidden, dec->H, nullptr, 0, dec->w2, dec->b2, rows,
                                                                                                 dec->V, logits, status);
        return hsnw_check_launch("window_decode");
    }
    const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
    if (sizeof(float) * 8 * static_cast<size_t>(K1 > dec->H ? K1 : dec->H) > 48 * 1024)
        return hsnw_fail(HSNW_E_UNSUPPORTED, "window_decode: fp32 products take layers of at most 1536 inputs");
    hsnw_profile_mark(HSNW_K_DECODE, stream);
    k_linear_f32<true><<<blocks, 256, sizeof(float) * 8 * K1, stream>>>(qs, dec->d_q, us, dec->d_u, dec->w1, dec->b1, rows, dec->H, hidden);
    if (int rc = hsnw_check_launch("window_decode")) return rc;
    hsnw_profile_mark(HSNW_K_DECODE, stream);
    k_linear_f32<false><<<blocks, 256, sizeof(float) * 8 * dec->H, stream>>>(hidden, dec->H, nullptr, 0, dec->w2, dec->b2, rows, dec->V, logits);
    return hsnw_check_launch("window_decode");
}

void hsnw_decode_set_attributes() {
    if (!hsnw_opt_in(reinterpret_cast<const void*>(k_linear_tc<true, 128>), "linear_tc<gelu>")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_linear_tc<false, 128>), "linear_tc")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_linear_tc<true, 32>), "linear_tc<gelu, 32>")
        || !hsnw_opt_in(reinterpret_cast<const void*>(k_linear_tc<false, 32>), "linear_tc<32>"))
        hsnw_attribute_failed();
}
