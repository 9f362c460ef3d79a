// A self-test of the bounded waits that every mbarrier wait of the window kernels goes through
// (rows.cuh: ring_wait; stage.cuh: mbar_wait): one small kernel waits on a barrier that nothing ever
// arrives at and nothing copies into. Both waits must give up after their iteration limits, set their
// error words and let the kernel run to its end, leaving the context usable. Nothing faults, traps or
// spins without a limit; no copy is in flight.
#include "../../include/hsn_window_b200.h"
#include "host_util.h"
#include "rows.cuh"

namespace {

__global__ void k_wait_runs_out(int* words) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int failed;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        failed = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        ring_wait(&bar, 0, words, &failed);       // phase 0 never completes: runs out, words[0] = 1
        ring_wait(&bar, 0, words + 3, &failed);   // after a time-out the block's later waits return at once: words[3] stays 0
        mbar_wait(&bar, 0, words + 1);            // the staging wait of the phase kernels: words[1] = 1
    }
    __syncthreads();
    if (threadIdx.x == 0) words[2] = 7;           // the kernel reached its end
}

}  // namespace

extern "C" int hsnw_selftest_wait_timeout(int* words, void* stream) {
    if (int rc = hsnw_require_prepared()) return rc;
    if (!words) return hsnw_fail(HSNW_E_ARG, "selftest_wait_timeout: null argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(words, 0, 4 * sizeof(int), s) != cudaSuccess) return hsnw_check_launch("selftest_wait_timeout");
    k_wait_runs_out<<<1, 32, 0, s>>>(words);
    return hsnw_check_launch("selftest_wait_timeout");
}
