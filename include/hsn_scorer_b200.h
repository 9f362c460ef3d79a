/* hsn_scorer_b200: the replay's scorer logits over every cell of every window position, and the gradients of the
 * scorer's weight and bias, behind the same C ABI as hsn_window_b200.h (error codes, hsnw_prepare, hsnw_last_error
 * are that header's).
 *
 * Reference interface replaced (path inside the reference project):
 *   python/hsn/train/split.py:305-342     _scorer_logits(scorer, u, eps, h, age, scalars)   -> hsnw_scorer_logits
 *   autograd's backward of it w.r.t. scorer.net.weight / .bias (the features are constants of the replay:
 *   h is the recorded state, u and eps are detached; split.py:628-631)                       -> hsnw_scorer_logits_backward
 * for the linear scorer without an address gate and without excluded features (the cases the reference's own
 * fast path covers, minus A12).
 *
 * logits[r, n, :] = W[:, 2d:3d] h[r, n] + W[:, 3d:] [age[r, n] / age_max; scalars[r, n]] + b + W[:, :2d] [u[r]; eps[r]]
 * without the [R, N, 3d + 1 + S] feature tensor: the recorded state (R N d floats, 0.5 GB for a B32 T256 N256 d64
 * window) is read once per call.
 *
 * prod_bf16 = 1 is the function under bfloat16 autocast: each of the three maps reads bfloat16 operands, sums in
 * float32 and rounds its output to bfloat16, the outputs are added in float32; in the backward every gradient
 * block is rounded to bfloat16 and widened. prod_bf16 = 0: float32 throughout. Tensors are float32 in both.
 */
#ifndef HSN_SCORER_B200_H
#define HSN_SCORER_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* weight [n_units, 3 d + 1 + n_scalars] and bias [n_units] as nn.Linear holds them, float32 on the device.
 * d a multiple of 4, at most 128; at most 8 units; at most 15 scalars. */
typedef struct HsnwScorer {
    int32_t d, n_cells, n_units, n_scalars;
    int32_t prod_bf16;
    float age_max;
    const float *weight, *bias;
} HsnwScorer;

/* Bytes of device scratch for `rows` window positions (256-byte aligned); backward != 0: the backward call's. */
int64_t hsnw_scorer_scratch_bytes(const HsnwScorer* scorer, int64_t rows, int backward);

/* u, eps [rows, d], h [rows, n_cells, d], age [rows, n_cells] int64, scalars [rows, n_cells, n_scalars]
 * -> logits [rows, n_cells, n_units]. The first int32 of `scratch` is the call's status word (0, or 1 after a
 * bounded device-side wait gave up: discard the results). */
int hsnw_scorer_logits(const HsnwScorer* scorer, const float* u, const float* eps, const float* h, const int64_t* age,
                       const float* scalars, int64_t rows, float* logits, void* scratch, int64_t scratch_bytes, void* stream);

/* d_weight [n_units, 3 d + 1 + n_scalars] and d_bias [n_units] (overwritten) for the cotangent d_logits
 * [rows, n_cells, n_units]. Sums run in a fixed order: the same bits every run. */
int hsnw_scorer_logits_backward(const HsnwScorer* scorer, const float* u, const float* eps, const float* h, const int64_t* age,
                                const float* scalars, int64_t rows, const float* d_logits, float* d_weight, float* d_bias,
                                void* scratch, int64_t scratch_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif
