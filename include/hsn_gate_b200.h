/* hsn_gate_b200: the cell norm and the gate of the replay's cell pass over every slot of every window position, and
 * their backward, behind the same C ABI as hsn_window_b200.h (error codes, hsnw_prepare, hsnw_last_error are that
 * header's).
 *
 * Reference interface replaced (path inside the reference project):
 *   python/hsn/model/cell.py:707-709   v = self.norm(v_raw); gate_pre = self.gate(v).to(dtype);
 *                                      b = torch.sigmoid(gate_pre)                  -> hsnw_gate_forward
 *   python/hsn/model/cell.py:727-733   record["gate_pre"], record["rms"]             (outputs of the forward)
 *   autograd's backward of those lines w.r.t. v_raw, norm.weight, gate.weight and gate.bias, with the unit pass's
 *   gradient of v added                                                             -> hsnw_gate_backward
 * for model.cell_norm = rms (cell.py: nn.RMSNorm(4 d)).
 *
 * It sits before the grouped unit pass (hsn_units_b200.h: this `v` is its `v`, its `d_v` this `d_v_units`); `b` goes
 * to the state recurrence, whose reverse sweep returns `db` (hsn_window_b200.h), this `d_b`.
 *
 * Products in bfloat16 only (prod_bf16 = 1, the pass under bfloat16 autocast: the norm in float32; the gate reads v,
 * its weight and bias as bfloat16, sums in float32 and rounds to bfloat16; in the backward d_gate_pre is rounded to
 * bfloat16 where it crosses the cast and the linear's two products and the bias sum are rounded to bfloat16).
 * prod_bf16 = 0 and d = 128 return HSNW_E_UNSUPPORTED: the caller keeps the reference's lines. Tensors are float32.
 */
#ifndef HSN_GATE_B200_H
#define HSN_GATE_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* norm_weight [4 d], gate_w [d, 4 d] as nn.Linear holds it, gate_b [d], float32 on the device. d is 16, 32 or 64. */
typedef struct HsnwGate {
    int32_t d;
    int32_t prod_bf16;
    float norm_eps;
    int32_t reserved;
    const float *norm_weight, *gate_w, *gate_b;
} HsnwGate;

/* Bytes of device scratch for `slots` slots (256-byte aligned); backward != 0: the backward call's (the blocks'
 * shares of the parameter gradients). The forward keeps nothing between launches: 256 bytes. */
int64_t hsnw_gate_scratch_bytes(const HsnwGate* gate, int64_t slots, int backward);

/* v_raw [slots, 4 d] -> v [slots, 4 d], rms [slots], gate_pre [slots, d], b [slots, d]. */
int hsnw_gate_forward(const HsnwGate* gate, const float* v_raw, int64_t slots, float* v, float* rms, float* gate_pre, float* b,
                      void* scratch, int64_t scratch_bytes, void* stream);

/* For the cotangents d_v_units [slots, 4 d] of v (the unit pass's) and d_b [slots, d] of b, with gate_pre the
 * forward's: d_v_raw [slots, 4 d], d_norm_weight [4 d], d_gate_w [d, 4 d], d_gate_b [d] (all overwritten). Sums run
 * in a fixed order: the same bits every run. */
int hsnw_gate_backward(const HsnwGate* gate, const float* v_raw, const float* gate_pre, const float* d_v_units, const float* d_b,
                       int64_t slots, float* d_v_raw, float* d_norm_weight, float* d_gate_w, float* d_gate_b,
                       void* scratch, int64_t scratch_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif
