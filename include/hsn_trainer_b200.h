/* hsn_trainer_b200: the trainer's per-step passes after backward() (AdamW on ordinary and on
 * stacked unit tensors, the float64 clip's scaling, the update caps, the weight average) as one
 * launch over a list of tensors each, behind the same C ABI as hsn_window_b200.h.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   kernels/include/hsn_trainer_launch.h:11-29       HsnTrainArgs, kept bit for bit (3760 bytes)
 *   python/hsn/kernels/window_ext.cpp:155-213         launch_table   -> hsnw_launch_table
 *   kernels/cuda/hsn_trainer.cu:71-182                the seven kernels launched by name, each with
 *                                                     the rows / i[] / f[] / u[][] of its namesake
 * Every kernel computes, bit for bit, what the sequence of PyTorch CUDA kernels it replaces
 * computes (python/hsn/train/lazy_adam.py:462-486, :573-627, weight_ema.py, grad_norm.py,
 * update_limit.py): one explicitly rounded operation per PyTorch operation, a fused multiply-add
 * exactly where PyTorch's kernels have one (lerp, addcmul, addcdiv).
 */
#ifndef HSN_TRAINER_B200_H
#define HSN_TRAINER_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HSN_TR_ROWS 4
#define HSN_TR_TENSORS 40
#define HSN_TR_INTS 8
#define HSN_TR_FLOATS 8
#define HSN_TR_DOUBLES 2
#define HSN_TR_COEFS 6
#define HSN_TR_UNITS 64
/* A launch walks a list of tensors as one index space: tensor j holds the elements
 * [end[j-1], end[j]) (end[-1] = 0), p[r][j] is the device address of its r-th operand (a row a
 * kernel does not read stays null). i[0] is the number of tensors, i[1..] sizes and flags, f[]
 * float scalars, g[] double scalars, u[c][m] per-unit coefficients of stacked unit tensors. */
typedef struct HsnTrainArgs {
    void* p[HSN_TR_ROWS][HSN_TR_TENSORS];
    int64_t end[HSN_TR_TENSORS];
    double g[HSN_TR_DOUBLES];
    int32_t i[HSN_TR_INTS];
    float f[HSN_TR_FLOATS];
    float u[HSN_TR_COEFS][HSN_TR_UNITS];
} HsnTrainArgs;

/* Launch the trainer kernel `name` over the tensors of `args` on `stream`. Names and slots:
 *   hsn_tr_adamw          rows 0 param, 1 grad, 2 exp_avg, 3 exp_avg_sq; i1 weight decay on;
 *                         f0 1 - lr wd, f1 1 - beta1, f2 beta2, f3 1 - beta2,
 *                         f4 1 / sqrt(1 - beta2^t), f5 eps, f6 -lr / (1 - beta1^t)
 *   hsn_tr_adamw_units    the same rows; i1 weight decay on, i2 M; f3 1 - beta2, f5 eps;
 *                         u0 active, u1 decay, u2 lerp weight, u3 second-moment factor,
 *                         u4 sqrt(1 - beta2^t), u5 lr / (1 - beta1^t), per unit
 *   hsn_tr_lerp           rows 0 self (in place), 1 end; f0 weight
 *   hsn_tr_scale64        row 0 grad (in place); p[1][0] one float64 on the device
 *   hsn_tr_copy           rows 0 dst, 1 src
 *   hsn_tr_limit_squares  rows 0 param, 1 old, 2 old^2 (out), 3 (param - old)^2 (out)
 *   hsn_tr_limit_project  rows 0 param (in place), 1 old, 2 (param' - old)^2 (out),
 *                         3 the tensor's group: [scale, clipped] as two floats on the device
 * The grid is the library's own (a block takes runs of 1024 elements of one tensor, 16 bytes a
 * thread where the addresses allow). Returns 0, HSNW_E_NAME, HSNW_E_ARG or HSNW_E_CUDA. */
int hsnw_launch_table(const char* name, const HsnTrainArgs* args, void* stream);

/* The gradient exchange fused with the optimiser step, for data-parallel ranks of one box whose gradient
 * and parameter buffers are mapped into each other's address spaces (peer memory over NVLink): ONE
 * kernel per rank that, for the rank's shard of a flat parameter vector, reads every rank's gradients
 * of the shard from that rank's memory, sums them in rank order (a fixed order: every rank computes the
 * same bits), averages, applies hsn_tr_adamw's step to the shard's parameters and moments, and writes the
 * new parameters into every rank's parameter buffer. That is reduce-scatter, AdamW and all-gather with
 * the transfers inside the arithmetic's loop instead of two collectives around a kernel. No counterpart
 * in the reference (its trainer all-reduces, then steps: scripts and python/hsn/train/loop.py).
 * The caller orders the ranks around the launch: every rank's gradients are complete before any rank's
 * kernel starts, and no rank reads its parameters before every rank's kernel has ended (two barriers on
 * the stream; hsn_b200/parallel.py uses a one-element NCCL all-reduce for each). */
#define HSN_EX_RANKS 8
typedef struct HsnwExchange {
    int32_t world, rank;        /* 1..8 ranks; this rank */
    int32_t average;            /* 1: divide the sum by world (multiply by 1 / world) */
    int32_t weight_decay_on;
    int64_t shard;              /* elements per rank; rank r owns [r shard, (r + 1) shard) of the flat vector */
    const float* grads[HSN_EX_RANKS];   /* every rank's gradient buffer [world shard], as mapped on this rank */
    float* params[HSN_EX_RANKS];        /* every rank's parameter buffer [world shard], as mapped on this rank */
    float* exp_avg;             /* [shard] this rank's moments */
    float* exp_avg_sq;
    float f[HSN_TR_FLOATS];     /* hsn_tr_adamw's f0 .. f6 */
} HsnwExchange;
int hsnw_exchange_adamw(const HsnwExchange* exchange, void* stream);

#ifdef __cplusplus
}
#endif
#endif
