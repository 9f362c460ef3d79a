/* hsn_messages_b200: the messages and the gathered inputs of the replay's cell pass over every slot of every window
 * position, and their backward, behind the same C ABI as hsn_window_b200.h (error codes, hsnw_prepare,
 * hsnw_last_error are that header's).
 *
 * Reference interface replaced (path inside the reference project):
 *   python/hsn/model/cell.py:698-705   index = graph._pad_src[cells]; sources = self.V(h_const.gather(1, index));
 *                                      m = (sources * edge_weights[..., None]).sum(dim=2);
 *                                      v_raw = native_ops.gather_concat(u, eps, h_const, m, cells)   -> hsnw_messages_forward
 *   autograd's backward of those lines w.r.t. u, eps, V.weight and the padded edge weights
 *   (graph._padded_weights(), python/hsn/model/graph.py:222-246; the state is a constant there)      -> hsnw_messages_backward
 *
 * It sits before the cell norm and the gate (hsn_gate_b200.h: this `v_raw` is its `v_raw`, its `d_v_raw` this one's).
 * The edge weights' normalisation (softmax or sigmoid of graph.edge_logit over [N, D] values) stays with the caller:
 * `edge_w` is its result, `d_edge_w` the gradient to send back through it.
 *
 * Products in bfloat16 only (prod_bf16 = 1, the pass under bfloat16 autocast: V reads bfloat16 operands, sums in
 * float32 and rounds to bfloat16; the weights are cast to bfloat16, every product w_j sources_j is a bfloat16 value,
 * their sum over j is rounded once; in the backward d_m is rounded to bfloat16, the products are bfloat16 values and
 * d_V a bfloat16 product). A cell's shares of d_edge_w are summed in float32 in slot order and rounded once, where the
 * reference adds them one by one into a bfloat16 tensor. prod_bf16 = 0, d = 128 and more than 4 in-neighbours return
 * HSNW_E_UNSUPPORTED: the caller keeps the reference's lines. Tensors are float32, indices int64.
 */
#ifndef HSN_MESSAGES_B200_H
#define HSN_MESSAGES_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* v_w [d, d] as nn.Linear holds it (no bias), edge_w [n_cells, degree] (zero on padding) and pad_src
 * [n_cells, degree] (the in-neighbours; 0 on padding), on the device. d is 16, 32 or 64; degree 1..4; k slots a row. */
typedef struct HsnwMessages {
    int32_t d, n_cells, degree, k;
    int32_t prod_bf16, reserved;
    const float *v_w, *edge_w;
    const int64_t* pad_src;
} HsnwMessages;

/* Bytes of device scratch of the backward call for `rows` window positions (256-byte aligned). The forward takes none. */
int64_t hsnw_messages_scratch_bytes(const HsnwMessages* msg, int64_t rows);

/* u, eps [rows, d], h [rows, n_cells, d], cells [rows, k] (a padded slot holds cell 0) -> v_raw [rows, k, 4 d]. */
int hsnw_messages_forward(const HsnwMessages* msg, const float* u, const float* eps, const float* h, const int64_t* cells,
                          int64_t rows, float* v_raw, void* stream);

/* For the cotangent d_v_raw [rows, k, 4 d]: d_u, d_eps [rows, d], d_edge_w [n_cells, degree], d_v_w [d, d] (all
 * overwritten). Sums run in a fixed order: the same bits every run. */
int hsnw_messages_backward(const HsnwMessages* msg, const float* h, const int64_t* cells, const float* d_v_raw, int64_t rows,
                           float* d_u, float* d_eps, float* d_edge_w, float* d_v_w, void* scratch, int64_t scratch_bytes,
                           void* stream);

#ifdef __cplusplus
}
#endif
#endif
