// Host-side helpers shared by the translation units of the library: the thread-local error
// message, the prepared-device check and launch-error capture.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

// Records `message` as the calling thread's last error and returns `code`.
int hsnw_fail(int code, const char* message);
// HSNW_OK when the current device was prepared, else HSNW_E_STATE.
int hsnw_require_prepared();
// The largest dynamic shared memory a block may take on the current (prepared) device.
size_t hsnw_max_shared();
// The number of SMs of the current (prepared) device, 0 when it is not prepared.
int hsnw_sm_count_current();
// cudaPeekAtLastError after a launch sequence: HSNW_OK or HSNW_E_CUDA with the runtime's message.
int hsnw_check_launch(const char* what);
// Opt `kernel` in to the largest dynamic shared memory its static shared memory leaves room for.
// Returns false (and records the message) when the runtime refuses.
bool hsnw_opt_in(const void* kernel, const char* name);
void hsnw_attribute_failed();
// Each translation unit opts its kernels in to large dynamic shared memory.
void hsnw_forward_set_attributes();
void hsnw_backward_set_attributes();
void hsnw_ops_set_attributes();
void hsnw_rows_set_attributes();
void hsnw_rows_bwd_set_attributes();
void hsnw_decode_set_attributes();
void hsnw_units_set_attributes();
void hsnw_scorer_set_attributes();
void hsnw_tail_set_attributes();
void hsnw_gate_set_attributes();
void hsnw_messages_set_attributes();
struct HsnwBackward;
struct HsnwModel;
struct HsnwForward;
// What the per-row cluster kernels answer when a shape does not fit them: not an error (every HSNW_E_*
// is negative and is passed on to the caller), the entry point then runs the batch-synchronous phases.
constexpr int HSNW_DECLINED = 1;
// The forward sweep by one persistent cluster per row (window_rows.cu): HSNW_OK when launched,
// HSNW_DECLINED when the shape does not fit that kernel, else a negative error code.
int hsnw_rows_forward(const HsnwModel* model, const HsnwForward* io, const float* pre_s, int* status, cudaStream_t stream);
// The reverse sweep by one persistent cluster per row (window_rows_bwd.cu): same return convention.
int hsnw_rows_backward(const HsnwModel* model, const HsnwBackward* io, int* status, cudaStream_t stream);
// Which kernels served the calling thread's last whole-window call (hsnw_last_path reports it).
enum HsnwPath { HSNW_PATH_NONE = 0, HSNW_PATH_ROWS = 1, HSNW_PATH_PHASES = 2 };
void hsnw_set_path(int path);

// Launch timing for measurement runs (hsnw_profile_begin / hsnw_profile_end): while it is on, every
// launch site records an event on its stream first; the time between two consecutive events is
// charged to the kernel launched between them. Off (the default) this is one predictable branch.
enum HsnwKernelKind {
    HSNW_K_INIT = 0, HSNW_K_PRE, HSNW_K_FRONT, HSNW_K_ROW, HSNW_K_UNIT, HSNW_K_UPDATE,
    HSNW_K_HEAD, HSNW_K_MID, HSNW_K_TAIL_HEAD, HSNW_K_ROWS_FWD, HSNW_K_ROWS_BWD, HSNW_K_PROLOGUE, HSNW_K_DECODE, HSNW_K_UNITS_FWD, HSNW_K_UNITS_BWD,
    HSNW_K_SCORER_FWD, HSNW_K_SCORER_BWD, HSNW_K_TAIL_FWD, HSNW_K_TAIL_BWD, HSNW_K_GATE_FWD, HSNW_K_GATE_BWD, HSNW_K_MSG_FWD, HSNW_K_MSG_BWD, HSNW_K_KINDS
};
extern bool g_hsnw_profile_on;
void hsnw_profile_mark_slow(int kind, cudaStream_t stream);
inline void hsnw_profile_mark(int kind, cudaStream_t stream) {
    if (g_hsnw_profile_on) hsnw_profile_mark_slow(kind, stream);
}
