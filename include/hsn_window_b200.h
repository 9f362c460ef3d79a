/* hsn_window_b200: the HSN TBPTT window path as hand-written sm_100a CUDA behind a C ABI.
 *
 * Plain pointers and sizes only: no torch types, no C++ in the signatures. Every pointer named
 * "device" is an address in the caller's current CUDA context on the device given to
 * hsnw_prepare. No entry point synchronises the device or the stream (except hsnw_prepare),
 * and none allocates device memory: outputs and scratch are the caller's.
 * Every function returns 0 on success and a negative HSNW_E_* code otherwise;
 * hsnw_last_error() then holds a message (thread-local).
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   kernels/include/hsn_window_launch.h:9-16        HsnWinArgs, kept bit for bit
 *   python/hsn/kernels/window_ext.cpp:41-56          prepare        -> hsnw_prepare
 *   python/hsn/kernels/window_ext.cpp:105-115        launch         -> hsnw_launch
 *   python/hsn/kernels/window_ext.cpp:117-127        launch_views   -> hsnw_launch (views are plain
 *                                                                      addresses here)
 *   python/hsn/kernels/window_ext.cpp:129-153        loop           -> hsnw_loop
 *   kernels/cuda/hsn_window.cu:59,124,563,792,1014,1183,1334  the kernels launched by name
 *   python/hsn/train/compile.py:1037-1213 (the folded forward sweep), python/hsn/train/
 *   state_sweep.py:359-384 (the reverse sweep's loop), python/hsn/train/compile.py:1913-2006
 *   (the serving step)                               -> hsnw_window_forward / _backward /
 *                                                       hsnw_stream_step
 */
#ifndef HSN_WINDOW_B200_H
#define HSN_WINDOW_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HSNW_OK 0
#define HSNW_E_ARG (-1)        /* a size, flag or pointer the entry point does not take */
#define HSNW_E_UNSUPPORTED (-2) /* a shape beyond a kernel's limits (message says which) */
#define HSNW_E_CUDA (-3)       /* the CUDA runtime reported an error */
#define HSNW_E_NAME (-4)       /* hsnw_launch: no kernel of that name */
#define HSNW_E_STATE (-5)      /* hsnw_prepare was not called on this device */

/* The launch descriptor of the kernels launched by name: the reference's own
 * (kernels/include/hsn_window_launch.h:9-16), same field order and sizes (544 bytes). Each
 * kernel's p[] / i[] / f[] slots are the reference kernel's of the same name. */
#define HSN_WIN_POINTERS 48
#define HSN_WIN_INTS 32
#define HSN_WIN_FLOATS 8
typedef struct HsnWinArgs {
    void* p[HSN_WIN_POINTERS];
    int32_t i[HSN_WIN_INTS];
    float f[HSN_WIN_FLOATS];
} HsnWinArgs;

/* Library version (major * 10000 + minor * 100 + patch). */
int hsnw_version(void);
/* The calling thread's last error message ("" if none). */
const char* hsnw_last_error(void);
/* Which kernels served the calling thread's last successful hsnw_window_forward / hsnw_stream_* /
 * hsnw_window_backward call: "rows" (one persistent thread-block cluster per row) or "phases" (the
 * batch-synchronous kernels, a few launches per position); "" before the first call. The row
 * kernels are taken when the model's shape fits them; an error of their launch is returned to the
 * caller, never hidden behind the other kernels. No counterpart in the reference. */
const char* hsnw_last_path(void);
/* Make `device` ready: checks that it is an sm_100 part, opts the kernels in to large dynamic
 * shared memory and records the SM count. Idempotent; the only call that may synchronise.
 * Replaces window_ext.cpp:41-56 (there: cuModuleLoad of a fatbin per context). */
int hsnw_prepare(int device);
/* 1 when hsnw_prepare succeeded for `device`. */
int hsnw_prepared(int device);
/* The number of SMs of a prepared device (0 otherwise). */
int hsnw_sm_count(int device);

/* One launch of the kernel `name` with `grid` blocks of `block` threads and `shared` bytes of
 * dynamic shared memory on `stream` (a cudaStream_t; NULL: the default stream).
 * Names: hsn_win_select, hsn_win_cell_update, hsn_win_recurrence, hsn_win_recurrence_dense, and the
 * reverse sweep's three per-position glue kernels hsn_win_back_head, hsn_win_back_mid,
 * hsn_win_back_tail (hsn_window.cu:1014-1427; their slots are window.py:1181-1290's, and the two
 * products between them stay the caller's; the whole sweep as one call is hsnw_window_backward).
 * Any other name returns HSNW_E_NAME.
 * grid <= 0 launches nothing (window_ext.cpp:96). Capturable in a CUDA graph. */
int hsnw_launch(const char* name, const HsnWinArgs* args, int64_t grid, int block, int shared,
                void* stream);
/* `steps` rounds of the kernels names[0..count) in order; round t runs them with
 * args->i[slot] = t (window_ext.cpp:129-153). */
int hsnw_loop(const char* const* names, int count, const int64_t* grids, const int* blocks,
              const int* shareds, const HsnWinArgs* args, int64_t steps, int slot, void* stream);
/* The launch shape this library wants for a by-name kernel at the sizes in `args` (the
 * reference's Python wrappers hard-code theirs, window.py:38-53,1151-1162): fills grid, block,
 * shared. Returns HSNW_E_UNSUPPORTED with a reason when the kernel cannot take the shape. */
int hsnw_launch_shape(const char* name, const HsnWinArgs* args, int64_t* grid, int* block,
                      int* shared);

/* ------------------------------------------------------------------------------------------------
 * Whole-window entry points.
 * Sizes: B rows, T positions, N cells, d state width, K slots, H hidden width, M units,
 * D padded in-degree, S scorer scalars per cell, dc context width.
 * ---------------------------------------------------------------------------------------------- */

/* The window's weights on the device, fp32, in the layouts the kernels read ("_t": transposed to
 * input-major so that consecutive threads read consecutive outputs). With prod_bf16 the values
 * must already be rounded to bfloat16 (the host rounds them once per window, as the reference's
 * SweepTwin.refresh does, compile.py:776-840); the kernels then round the products' other
 * operand and their outputs to bfloat16 and accumulate in fp32. */
typedef struct HsnwModel {
    int32_t N, d, K, H, M, D, S, dc;
    int32_t prod_bf16;      /* 0: fp32 products; 1: bf16 operands, fp32 accumulation */
    int32_t probes;         /* refresh probes on (router.py:1788-1850) */
    int32_t age_max;
    int32_t phases_only;    /* 1: never use the per-row cluster kernel (hsnw_window_forward picks it when it fits) */
    float lambda_cost, cell_overhead, shared_cost, limit; /* limit = budget * (1 + 1e-5) */
    float norm_eps, cand_eps;
    const float* s_w1zc_t;  /* [d + dc, H]  shared.fc1 rows of z, then of ctx */
    const float* f_w1q_t;   /* [d, 2H]      shared.fc1 rows of q | predictor.fc1 */
    const float* f_b1;      /* [2H]         shared.fc1.bias | predictor.fc1.bias */
    const float* f_w2_t;    /* [2H, d]      shared.fc2 (rows 0..H) ; predictor.fc2 (rows H..2H) */
    const float* f_b2;      /* [2d]         shared.fc2.bias | predictor.fc2.bias */
    const float* score_w_t; /* [3d + 1 + S, M] */
    const float* score_b;   /* [M] */
    const float* v_t;       /* [d, d]   (V h)[x] = sum_i h[i] v_t[i][x] */
    const float* wout_t;    /* [d, d] */
    const float* gate_t;    /* [4d, d] */
    const float* gate_b;    /* [d] */
    const float* norm_w;    /* [4d] */
    const float* cand_w;    /* [d] */
    const float* w1;        /* [M, 4d, H] */
    const float* b1;        /* [M, H] */
    const float* w2;        /* [M, H, d] */
    const float* b2;        /* [M, d] */
    const int32_t* pad_src; /* [N, D] */
    const float* edge_w;    /* [N, D] (0 on padding) */
    const float* cost;      /* [M] */
    /* bf16 images of the unit bank for the tensor cores (prod_bf16 only; null: CUDA-core path).
     * Tiles of 128 rows in the K-major core-matrix layout [K/8][128][8] (hsn_b200/csrc/umma.cuh),
     * zero padded: umma_w1 [M][ceil(H/128)][4d/8][128][8] (rows: hidden columns, K: the cell input),
     * umma_gate [4d/8][128][8] (rows: the gate's outputs), umma_w2 [M][ceil(H/128)][16][128][8]
     * (rows: the unit's outputs, K: the 128 hidden columns of the block). */
    const void* umma_w1;
    const void* umma_gate;
    const void* umma_w2;
    /* the same for the reverse sweep's transposed products (null: CUDA-core path), nT = ceil(2d/128):
     * umma_bw_w2 [M][ceil(H/128)][d/8][128][8] (rows: hidden columns, K: the unit's outputs),
     * umma_bw_w1 [M][ceil(H/128)][nT][16][128][8] (rows: the 2d state columns of the cell input,
     * K: the block's hidden columns), umma_bw_gate [nT][d/8][128][8] (rows: state columns,
     * K: the gate's outputs). */
    const void* umma_bw_w2;
    const void* umma_bw_w1;
    const void* umma_bw_gate;
    /* bf16 images for the per-row cluster kernel (prod_bf16, H a multiple of 128; null: not used).
     * With C = H / 128 blocks of a row's cluster:
     * rows_bank [M][C]: a unit's weights on a block's 128 hidden columns as three K-major tiles, W1's
     *   rows of the inputs [0, 2d) as [2d/8][128][8] (element (input x, column c) at ((x/8) 128 + c) 8 +
     *   x%8), the same for the inputs [2d, 4d), then W2 as [16][d][8] (element (column c, output x) at
     *   ((c/8) d + x) 8 + c%8); with d = 64 the tiles are 128-byte-swizzled K-blocks of 64 instead;
     * rows_front [C][2] chunks: the block's 256 columns of the merged front first layer
     *   f_w1q_t as [d][256], then the same columns' rows of f_w2_t as [256][d]. */
    const void* rows_bank;
    const void* rows_front;
    /* the same for the reverse sweep's per-row cluster kernel: rows_bank_bw [M][C], first W2 as [d/8][128][8]
     * (element (column c, output x) at ((x/8) 128 + c) 8 + x%8), then the 2d state rows of W1 as
     * [16][2d][8] (element (state input i, column c) at ((c/8) 2d + i) 8 + c%8); 128-byte-swizzled
     * K-blocks of 64 instead with d = 64. */
    const void* rows_bank_bw;
} HsnwModel;

/* Inputs, tape and record of a forward sweep. Row-major, contiguous. Null = not wanted, for the
 * pointers marked optional.
 *   tape_state != 0: the reference's tape (compile.py:1196-1213): tape_h [B,T+1,N,d],
 *     tape_q [B,T+1,d], tape_age [B,T+1,N] (i64); record 0 is written from (h0, q0, age0) with
 *     reset[:,0] applied, record t+1 after position t (zeroed when reset[:,t+1]); the final
 *     state is record T.
 *   tape_state == 0 ("resident"): h0/q0/age0 are updated in place, no state tape is kept;
 *     tape_h/q/age are ignored.
 */
typedef struct HsnwForward {
    int32_t B, T;
    int32_t tape_state;
    int32_t forced;            /* 1: cells/units/valid are inputs (a recorded decision replayed) */
    const float* z;            /* [B,T,d] */
    const float* ctx;          /* [B,T,dc] */
    const float* scalars;      /* [B,T,N,S] */
    const uint8_t* reset;      /* [B,T] */
    float* h0;                 /* [B,N,d] start state (resident: updated in place) */
    float* q0;                 /* [B,d] */
    int64_t* age0;             /* [B,N] */
    int64_t* pos;              /* [B] in/out (compile.py:1194-1200) */
    float* tape_h;
    float* tape_q;
    int64_t* tape_age;
    int64_t* cells;            /* [B,T,K] */
    int64_t* units;            /* [B,T,K] */
    uint8_t* valid;            /* [B,T,K] */
    uint8_t* refreshed;        /* [B,T,K] */
    float* theta;              /* [B,T] */
    float* h_sel;              /* [B,T,K,d] */
    float* qs;                 /* [B,T,d] */
    float* h_max;              /* [B,T] */
    /* the round's values per slot, what the state-gradient sweep reads (optional as a group:
     * rec_c null = none): c, b, h_old, y, gate_pre, m [B,T,K,d]; rms [B,T,K]; hidden [B,T,K,H].
     * rec_hidden holds float32 with fp32 products and bfloat16 (2 bytes an element: the values are
     * bfloat16 anyway, and the reference's record holds them so under autocast) with prod_bf16. */
    float* rec_c;
    float* rec_b;
    float* rec_h_old;
    float* rec_y;
    float* rec_gate_pre;
    float* rec_m;
    float* rec_rms;
    void* rec_hidden;
    float* logits;             /* optional [B,T,N,M]: the scorer's logits (tests) */
    float* us;                 /* optional [B,T,d]: u_t, the shared path's output at every position (the
                                * decoder's second input beside qs; hsnw_window_decode) */
    /* hsnw_forward_scratch_bytes() bytes, 256-byte aligned. Its first int32 is the call's status word:
     * cleared when the call is enqueued, set to 1 by a device-side wait (an mbarrier of the TMA
     * pipeline) that gave up after its iteration limit; the results of such a call are not valid. */
    void* scratch;
    int64_t scratch_bytes;
} HsnwForward;

int64_t hsnw_forward_scratch_bytes(const HsnwModel* model, int32_t B, int32_t T);
/* The forward sweep of one window for B rows: per position the shared path, the scorer, the
 * router's decision, the gather of the selected cells and their messages, the executed unit,
 * the gated update with write-back and the next position's reset. */
int hsnw_window_forward(const HsnwModel* model, const HsnwForward* io, void* stream);
/* One position on a resident state: hsnw_window_forward with T = 1, tape_state = 0, always by the
 * batch-synchronous kernels, which leave every cell's derived values (its part of the scorer's
 * logits, V h, max |h|) in io->scratch. */
int hsnw_stream_step(const HsnwModel* model, const HsnwForward* io, void* stream);
/* The next call on the same resident state: like hsnw_stream_step (any T, tape_state = 0), but the
 * derived values are taken from io->scratch instead of being recomputed from the whole state (at
 * 512 streams of 1024 cells that recomputation is five times the step). The caller guarantees:
 * the same model weights, B, T and scratch as the previous hsnw_stream_step / hsnw_stream_continue
 * on this state, and h0 / q0 / age0 untouched in between. A stream whose reset[:,0] is set starts
 * from zeros as usual. When the scratch's last call was of another kind or size (the library marks
 * the scratch), the derived values are recomputed as in hsnw_stream_step. */
int hsnw_stream_continue(const HsnwModel* model, const HsnwForward* io, void* stream);

/* The reverse sweep of one window (state_gradient.py:357-485; full_cut != 0: split.py:128-174).
 * A [B,N,d] and R [B,d] are in/out: on entry the cotangent of the state after the last position
 * (zeros for a window whose final state is detached; the next window's result when windows are
 * chained), on return the cotangent of the state the window started from, already zeroed on the
 * rows whose column 0 resets. */
typedef struct HsnwBackward {
    int32_t B, T;
    int32_t full_cut;
    int32_t pad_;
    const float* c;            /* [B,T,K,d] */
    const float* b;
    const float* h_old;
    const float* y;            /* state gradient only, as are gate_pre, m, rms, hidden, units */
    const float* gate_pre;
    const float* m;
    const float* rms;          /* [B,T,K] */
    const void* hidden;        /* [B,T,K,H]: float32, or bfloat16 with prod_bf16 (as HsnwForward.rec_hidden) */
    const int64_t* cells;      /* [B,T,K] (0 on padded slots) */
    const int64_t* units;
    const uint8_t* valid;
    const uint8_t* reset;      /* [B,T] */
    const float* d_q_pre;      /* optional [B,T,d] */
    const float* d_q_post;     /* optional [B,T,d] */
    const float* d_h_sel;      /* optional [B,T,K,d] */
    float* dc;                 /* [B,T,K,d] out */
    float* db;
    float* A;                  /* [B,N,d] in/out */
    float* R;                  /* [B,d] in/out */
    /* hsnw_backward_scratch_bytes() bytes, 256-byte aligned (optional with full_cut). Its first int32
     * is the call's status word, as in HsnwForward: cleared when the call is enqueued, set to 1 by a
     * device-side wait that gave up. */
    void* scratch;
    int64_t scratch_bytes;
} HsnwBackward;

int64_t hsnw_backward_scratch_bytes(const HsnwModel* model, int32_t B, int32_t T);
int hsnw_window_backward(const HsnwModel* model, const HsnwBackward* io, void* stream);

/* No counterpart in the reference. hsnw_window_backward for a caller that has no device memory to
 * give as scratch and no way to get some: a host that only forwards buffers it was handed, or a
 * process whose own pool already holds all free device memory, so that one more allocation would
 * fail. Same arguments and results; io->scratch and io->scratch_bytes are ignored. The scratch is
 * an array built into the library, hsnw_static_scratch_bytes() = 8 MiB of device memory that
 * every GPU which loads the library keeps until the process ends. A window whose B x K pairs
 * need more is refused with HSNW_E_UNSUPPORTED (the message says how much); it fits the
 * reference shape (B 32, K 8, H 512, d 64: 2.4 MiB). The call allocates nothing, on the device or
 * the host, and calls no allocating routine.
 * The first call on a device looks the array's address up (cudaGetSymbolAddress, with that device
 * current): make that first call before any stream capture begins.
 * All calls on one device share the array, and it keeps the last call's contents. Only its status
 * word has to start at zero and is cleared by every call (every other value is written before it
 * is read within a call); but two calls that overlap on the GPU, e.g. on two streams, race on it:
 * order them. */
int64_t hsnw_static_scratch_bytes(void);
int hsnw_window_backward_static(const HsnwModel* model, const HsnwBackward* io, void* stream);

/* The window-invariant part of the shared path's first layer for every position:
 * out [B*T, H] = [z ; ctx] [B*T, d+dc] x s_w1zc_t + shared.fc1.bias, one dense product
 * (hsnw_window_forward calls it itself; exported for tests and measurements). */
int hsnw_front_projection(const HsnwModel* model, const float* z, const float* ctx, int64_t rows,
                          float* out, void* stream);

/* ---- the window's prologue -----------------------------------------------------------------------
 * From a window's token and context ids to what hsnw_window_forward reads per position: replaces the
 * inference side of HSN._window_prologue (python/hsn/model/hsn.py:1707-1860) for model.key_address
 * with one address byte (S = 9) or without it (S = 7), no reader, no word addresses:
 * z = E(byte_emb(x)) (python/hsn/model/encoder.py:74-128), ctx = ctx_emb(id), positions
 * (hsn.py:347-355) and Scorer.window_scalars (python/hsn/model/router.py:597-765). Weights are in
 * torch's nn.Linear layout [out, in]; with prod_bf16 the encoder's two linears round their operands
 * and outputs to bfloat16 (what bf16 autocast does), the address features stay float32. All pointers
 * are device addresses. A caller that uploads only ids (B T of each) thus never moves the
 * [B,T,N,S] scalars across the bus. */
typedef struct HsnwPrologue {
    int32_t B, T, V, d, H, dc, N, S;   /* V byte values, H the encoder's hidden width */
    int32_t prod_bf16;
    int32_t position_mode;             /* 0: the position as it is, 1: clamped to unroll - 1, 2: modulo unroll */
    int32_t ema_per_row;               /* 0: ema_* are [N], 1: [B,N] */
    int32_t bos;                       /* the byte that stands for "no previous byte" */
    float budget_frac, round_frac, n_context, unroll;
    const float* byte_emb;             /* [V,d] */
    const float* enc_w1;               /* [H,d] */
    const float* enc_b1;               /* [H] */
    const float* enc_w2;               /* [d,H] */
    const float* enc_b2;               /* [d] */
    const float* ctx_emb;              /* [context ids, dc] */
    const float* byte_codes;           /* [V,d]  (S = 9) */
    const float* cell_addresses;       /* [N,d]  (S = 9) */
    const float* ema_utility;
    const float* ema_selected;
    const int64_t* tokens;             /* [B,T] */
    const int64_t* ctx_ids;            /* [B,T] */
    const uint8_t* reset;              /* [B,T] */
    const int64_t* pos0;               /* [B] the session position the window starts at */
    const int64_t* prev_tokens;        /* optional [B]: the byte before the window (null: none, reads as bos) */
    float* z;                          /* [B,T,d] out */
    float* ctx;                        /* [B,T,dc] out */
    float* scalars;                    /* [B,T,N,S] out */
    int64_t* positions;                /* optional [B,T] out */
    void* scratch;                     /* hsnw_prologue_scratch_bytes() bytes, 256-byte aligned */
    int64_t scratch_bytes;
} HsnwPrologue;
int64_t hsnw_prologue_scratch_bytes(const HsnwPrologue* prologue);
int hsnw_window_prologue(const HsnwPrologue* prologue, void* stream);

/* ------------------------------------------------------------------------------------------------
 * The window's epilogue: the decoder D([q_t; u_t]) = fc2(act(fc1(.))) over rows (python/hsn/model/
 * hsn.py:2374-2390, python/hsn/model/encoder.py:175-182), for a window's B T positions or a serving
 * step's B rows. Weights in nn.Linear's layout, fp32 (with prod_bf16 already rounded to bfloat16);
 * qs [rows, d_q] and us [rows, d_u] are the forward sweep's outputs of those names. With prod_bf16 every
 * linear's operands, bias and output are bfloat16 values and its sums float32 (autocast); the
 * activation is the exact-erf GELU.
 * ---------------------------------------------------------------------------------------------- */
typedef struct HsnwDecoder {
    int32_t d_q, d_u, H, V;    /* widths of the two input parts, the hidden layer, the vocabulary */
    int32_t prod_bf16;
    int32_t reserved;
    const float* w1;           /* [H, d_q + d_u] */
    const float* b1;           /* [H] */
    const float* w2;           /* [V, H] */
    const float* b2;           /* [V] */
} HsnwDecoder;
int64_t hsnw_decode_scratch_bytes(const HsnwDecoder* decoder, int64_t rows);
/* logits [rows, V]. scratch: hsnw_decode_scratch_bytes() bytes, 256-byte aligned; its first int32 is the
 * call's status word (0, or 1 after a bounded device-side wait gave up). */
int hsnw_window_decode(const HsnwDecoder* decoder, const float* qs, const float* us, int64_t rows, float* logits,
                       void* scratch, int64_t scratch_bytes, void* stream);

/* ---- launch timing, for measurement runs --------------------------------------------------------
 * No counterpart in the reference (it times whole steps on the host, scripts/bench_window.py:60-110).
 * Between hsnw_profile_begin and hsnw_profile_end every kernel launch of the window entry points
 * is preceded by an event on its stream; hsnw_profile_end synchronises, and fills for each kernel
 * kind k < hsnw_profile_kinds() the summed time (ms, event to next event: the kernel and the gap
 * before the next launch) and the number of launches. One profile at a time, one host thread, one
 * stream. hsnw_profile_kind_name(k): "init" "pre" "front" "row" "unit" "update" "head" "mid"
 * "tail_head" (the batch-synchronous phases) "rows_fwd" "rows_bwd" (the per-row cluster kernels: one
 * launch a window) "prologue" (hsnw_window_prologue's three launches as one) "decode" (hsnw_window_decode's
 * two). */
int hsnw_profile_begin(void);
int hsnw_profile_kinds(void);
const char* hsnw_profile_kind_name(int kind);
int hsnw_profile_end(double* ms_by_kind, int64_t* launches_by_kind, int kinds);

/* ---- self-test of the bounded device-side waits --------------------------------------------------
 * No counterpart in the reference (its kernels have no waits). Every mbarrier wait of the window
 * kernels polls a bounded number of times, then gives up, sets the call's status word and lets the
 * kernel run to its end. This launches one small kernel whose barrier nothing ever completes and
 * fills words[0..4) (device, int32): [0] = 1 the ring wait of the row kernels ran out, [1] = 1 the
 * staging wait of the phase kernels ran out, [2] = 7 the kernel reached its end, [3] = 0 a wait after
 * the block's first time-out returned at once. Takes up to a few seconds; the context stays usable. */
int hsnw_selftest_wait_timeout(int32_t* words, void* stream);

#ifdef __cplusplus
}
#endif
#endif
