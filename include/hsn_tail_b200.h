/* hsn_tail_b200: the end of the replay's cell pass over every slot of every window position (W_out, the candidate
 * norm, the weighted tanh) and its backward, behind the same C ABI as hsn_window_b200.h (error codes, hsnw_prepare,
 * hsnw_last_error are that header's).
 *
 * Reference interface replaced (path inside the reference project):
 *   python/hsn/model/cell.py:719-721   y = W_out(unit_out).to(dtype); pre = cand_norm(y);
 *                                      c = tanh(alpha[..., None] * pre)           -> hsnw_tail_forward
 *   python/hsn/model/cell.py:723       record["y"] = y                             (the forward's second output)
 *   autograd's backward of those three lines w.r.t. unit_out, alpha, W_out.weight and cand_norm.weight
 *                                                                                  -> hsnw_tail_backward
 * for model.cand_norm = rms (cell.py:210-211: nn.RMSNorm(d, eps)); the branch without the norm (cell.py:714-717)
 * is not taken here (HSNW_E_ARG when norm_weight is null).
 *
 * It sits between the grouped unit pass (hsn_units_b200.h: its `out` is this `unit_out`, this `d_unit_out` its
 * `d_out`) and the state-gradient sweep (hsn_window_b200.h: its `dc` is this `d_c`).
 *
 * prod_bf16 = 1 is the pass under bfloat16 autocast: the linear reads bfloat16 operands, sums in float32 and rounds
 * y to bfloat16; norm and tanh in float32; in the backward d_y is rounded to bfloat16 where it crosses the cast and
 * both of the linear's products are rounded to bfloat16. unit_out and d_unit_out are then bfloat16 tensors (as the
 * unit pass holds them), else float32; everything else is float32.
 */
#ifndef HSN_TAIL_B200_H
#define HSN_TAIL_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* w_out [d, d] as nn.Linear holds it ([out, in], no bias) and the norm's gain norm_weight [d], float32 on the
 * device. d is 16, 32, 64 or 128. */
typedef struct HsnwTail {
    int32_t d;
    int32_t prod_bf16;
    float norm_eps;
    int32_t reserved;
    const float *w_out, *norm_weight;
} HsnwTail;

/* Bytes of device scratch of the backward call for `slots` slots (256-byte aligned). The forward takes none. */
int64_t hsnw_tail_scratch_bytes(const HsnwTail* tail, int64_t slots);

/* unit_out [slots, d], alpha [slots] -> y [slots, d] (the record), c [slots, d]. */
int hsnw_tail_forward(const HsnwTail* tail, const void* unit_out, const float* alpha, int64_t slots, float* y, float* c,
                      void* stream);

/* For the cotangent d_c [slots, d] of c, with y the forward's: d_unit_out [slots, d], d_alpha [slots],
 * d_w_out [d, d], d_norm_weight [d] (all overwritten). Sums run in a fixed order: the same bits every run. */
int hsnw_tail_backward(const HsnwTail* tail, const void* unit_out, const float* alpha, const float* y, const float* d_c,
                       int64_t slots, void* d_unit_out, float* d_alpha, float* d_w_out, float* d_norm_weight,
                       void* scratch, int64_t scratch_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif
