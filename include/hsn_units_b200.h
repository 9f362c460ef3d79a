/* hsn_units_b200: the replay's grouped unit pass, forward and backward, behind the same C ABI as
 * hsn_window_b200.h (error codes, hsnw_prepare, hsnw_last_error are that header's).
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   python/hsn/model/units.py:356-414     UnitBank.forward_grouped(v, unit_idx, record=)  -> hsnw_units_forward
 *   the autograd backward of that pass (per present unit: addmm, activation, addmm)       -> hsnw_units_backward
 *   python/hsn/model/cell.py:716          its call in PDGCell.replay_sparse, every pair of a window at once
 *   python/hsn/train/split.py:588-762     SplitWindow._replay, the caller of replay_sparse
 *
 * For P pairs (v_p [d_in], unit_p): pre_p = v_p W1[u] + b1[u], out_p = gelu(pre_p) W2[u] + b2[u] (exact-erf
 * GELU), both in the pairs' input order; `pre` is what the reference hands out as record["hidden"]. The
 * backward returns, for a cotangent d_out of out, d_v and the gradients of the four stacked parameters
 * (zero for a unit no pair chose).
 *
 * prod_bf16 = 1 is the pass under bfloat16 autocast: every product reads bfloat16 operands, sums in float32 and
 * rounds its output to bfloat16 (the weight gradients and bias sums too, which are then widened to float32);
 * pre, out and d_out are bfloat16 tensors. prod_bf16 = 0: float32 throughout, pre, out, d_out float32.
 * v and d_v are float32 in both (under autocast the cell norm's output is float32 and addmm casts it).
 */
#ifndef HSN_UNITS_B200_H
#define HSN_UNITS_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The unit bank's stacked parameters in the reference's layouts (units.py:211-214), float32 on the device:
 * w1 [n_units, d_in, hidden], b1 [n_units, hidden], w2 [n_units, hidden, d_out], b2 [n_units, d_out].
 * d_in, hidden, d_out in multiples of 8; at most 256 units. */
typedef struct HsnwUnits {
    int32_t n_units, d_in, hidden, d_out;
    int32_t prod_bf16;
    int32_t reserved;
    const float *w1, *b1, *w2, *b2;
} HsnwUnits;

/* Bytes of device scratch a call over `pairs` pairs needs (256-byte aligned; backward != 0: hsnw_units_backward's,
 * which holds d_pre [pairs, hidden] and the weight gradients' partial tiles). 0 for sizes the calls refuse. */
int64_t hsnw_units_scratch_bytes(const HsnwUnits* units, int64_t pairs, int backward);

/* v [pairs, d_in] float32, unit_idx [pairs] int64 -> pre [pairs, hidden], out [pairs, d_out] (bfloat16 or float32,
 * see prod_bf16). All launches go to `stream`; nothing is read by the host. The first int32 of `scratch` is the
 * call's status word once the stream has run: 0, 1 (a bounded device-side wait gave up: discard the results) or
 * 2 (a unit index outside [0, n_units): its pair was skipped; the reference raises IndexError). */
int hsnw_units_forward(const HsnwUnits* units, const float* v, const int64_t* unit_idx, int64_t pairs, void* pre, void* out,
                       void* scratch, int64_t scratch_bytes, void* stream);

/* The backward of hsnw_units_forward for the cotangent d_out [pairs, d_out] (out's type) with `pre` that call's:
 * d_v [pairs, d_in], d_w1, d_b1, d_w2, d_b2 in the parameters' shapes, all float32, overwritten. The weight
 * gradients are summed in a fixed order (segments of the sorted pairs, in order): the same bits every run. */
int hsnw_units_backward(const HsnwUnits* units, const float* v, const int64_t* unit_idx, int64_t pairs, const void* pre,
                        const void* d_out, float* d_v, float* d_w1, float* d_b1, float* d_w2, float* d_b2, void* scratch,
                        int64_t scratch_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif
