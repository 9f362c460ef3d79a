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
// cudaPeekAtLastError after a launch sequence: HSNW_OK or HSNW_E_CUDA with the runtime's message.
int hsnw_check_launch(const char* what);
// Each translation unit opts its kernels in to large dynamic shared memory.
void hsnw_forward_set_attributes();
void hsnw_backward_set_attributes();
void hsnw_ops_set_attributes();
