// The C ABI's plumbing: error messages, device preparation and the launch of a kernel by name
// with the reference's launch descriptor (reference python/hsn/kernels/window_ext.cpp:41-153 does
// the same through the driver API on a fatbin; here the kernels are linked into the library).
#include "../../include/hsn_window_b200.h"
#include "host_util.h"

#include <mutex>
#include <vector>
#include <stdio.h>
#include <string.h>

extern "C" __global__ void hsn_win_select(HsnWinArgs a);
extern "C" __global__ void hsn_win_cell_update(HsnWinArgs a);
extern "C" __global__ void hsn_win_recurrence(HsnWinArgs a);
extern "C" __global__ void hsn_win_recurrence_dense(HsnWinArgs a);
extern "C" __global__ void hsn_win_back_head(HsnWinArgs a);
extern "C" __global__ void hsn_win_back_mid(HsnWinArgs a);
extern "C" __global__ void hsn_win_back_tail(HsnWinArgs a);

namespace {

constexpr int kMaxDevices = 64;
thread_local char last_error[512] = "";
thread_local int last_path = HSNW_PATH_NONE;
std::mutex prepare_mutex;
struct DeviceInfo {
    bool ready = false;
    int sm_count = 0;
    size_t max_shared = 0;
};
DeviceInfo devices[kMaxDevices];

struct Named {
    const char* name;
    void (*kernel)(HsnWinArgs);
};
const Named kKernels[] = {
    {"hsn_win_select", hsn_win_select},
    {"hsn_win_cell_update", hsn_win_cell_update},
    {"hsn_win_recurrence", hsn_win_recurrence},
    {"hsn_win_recurrence_dense", hsn_win_recurrence_dense},
    {"hsn_win_back_head", hsn_win_back_head},
    {"hsn_win_back_mid", hsn_win_back_mid},
    {"hsn_win_back_tail", hsn_win_back_tail},
};

const Named* find(const char* name) {
    if (!name) return nullptr;
    for (const Named& k : kKernels)
        if (strcmp(k.name, name) == 0) return &k;
    return nullptr;
}

int current_device() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) return -1;
    return device;
}

int round_up32(int v) { return (v + 31) & ~31; }

}  // namespace

int hsnw_fail(int code, const char* message) {
    snprintf(last_error, sizeof(last_error), "%s", message ? message : "");
    return code;
}

int hsnw_require_prepared() {
    const int device = current_device();
    if (device < 0 || device >= kMaxDevices || !devices[device].ready)
        return hsnw_fail(HSNW_E_STATE, "the current device is not prepared; call hsnw_prepare(device) first");
    return HSNW_OK;
}

size_t hsnw_max_shared() {
    const int device = current_device();
    return (device >= 0 && device < kMaxDevices) ? devices[device].max_shared : 0;
}

int hsnw_sm_count_current() {
    const int device = current_device();
    return (device >= 0 && device < kMaxDevices) ? devices[device].sm_count : 0;
}

int hsnw_check_launch(const char* what) {
    const cudaError_t status = cudaPeekAtLastError();
    if (status == cudaSuccess) return HSNW_OK;
    cudaGetLastError();
    char buffer[400];
    snprintf(buffer, sizeof(buffer), "%s: CUDA error: %s", what, cudaGetErrorString(status));
    return hsnw_fail(HSNW_E_CUDA, buffer);
}

bool hsnw_opt_in(const void* kernel, const char* name) {
    cudaFuncAttributes attr;
    cudaError_t status = cudaFuncGetAttributes(&attr, kernel);
    if (status == cudaSuccess) {
        const int room = static_cast<int>(hsnw_max_shared()) - static_cast<int>(attr.sharedSizeBytes);
        status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, room);
    }
    if (status == cudaSuccess) return true;
    cudaGetLastError();
    char buffer[300];
    snprintf(buffer, sizeof(buffer), "prepare: %s: %s", name, cudaGetErrorString(status));
    hsnw_fail(HSNW_E_CUDA, buffer);
    return false;
}

static bool attributes_ok = true;
void hsnw_attribute_failed() { attributes_ok = false; }

void hsnw_ops_set_attributes() {
    for (const Named& k : kKernels)
        if (!hsnw_opt_in(reinterpret_cast<const void*>(k.kernel), k.name)) hsnw_attribute_failed();
}

extern "C" int hsnw_version(void) { return 100; }

extern "C" const char* hsnw_last_error(void) { return last_error; }

void hsnw_set_path(int path) { last_path = path; }
extern "C" const char* hsnw_last_path(void) {
    return last_path == HSNW_PATH_ROWS ? "rows" : last_path == HSNW_PATH_PHASES ? "phases" : "";
}

extern "C" int hsnw_prepare(int device) {
    if (device < 0 || device >= kMaxDevices) return hsnw_fail(HSNW_E_ARG, "prepare: device out of range");
    std::lock_guard<std::mutex> lock(prepare_mutex);
    if (devices[device].ready) return HSNW_OK;
    int previous = -1;
    cudaGetDevice(&previous);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        cudaGetLastError();
        return hsnw_fail(HSNW_E_CUDA, "prepare: no such CUDA device");
    }
    if (prop.major != 10) {
        char buffer[160];
        snprintf(buffer, sizeof(buffer), "prepare: built for sm_100a only, device %d is sm_%d%d", device,
                 prop.major, prop.minor);
        return hsnw_fail(HSNW_E_UNSUPPORTED, buffer);
    }
    if (cudaSetDevice(device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) {
        cudaGetLastError();
        return hsnw_fail(HSNW_E_CUDA, "prepare: context initialisation failed");
    }
    devices[device].sm_count = prop.multiProcessorCount;
    devices[device].max_shared = prop.sharedMemPerBlockOptin;
    attributes_ok = true;
    hsnw_ops_set_attributes();
    hsnw_forward_set_attributes();
    hsnw_backward_set_attributes();
    hsnw_rows_set_attributes();
    hsnw_rows_bwd_set_attributes();
    hsnw_decode_set_attributes();
    hsnw_units_set_attributes();
    hsnw_scorer_set_attributes();
    hsnw_tail_set_attributes();
    hsnw_gate_set_attributes();
    hsnw_messages_set_attributes();
    const cudaError_t status = cudaGetLastError();
    if (previous >= 0 && previous != device) cudaSetDevice(previous);
    if (!attributes_ok) return HSNW_E_CUDA;  // the message names the kernel
    if (status != cudaSuccess) {
        char buffer[300];
        snprintf(buffer, sizeof(buffer), "prepare: %s", cudaGetErrorString(status));
        return hsnw_fail(HSNW_E_CUDA, buffer);
    }
    devices[device].ready = true;
    return HSNW_OK;
}

extern "C" int hsnw_prepared(int device) {
    return device >= 0 && device < kMaxDevices && devices[device].ready ? 1 : 0;
}

extern "C" int hsnw_sm_count(int device) {
    return hsnw_prepared(device) ? devices[device].sm_count : 0;
}

extern "C" int hsnw_launch(const char* name, const HsnWinArgs* args, int64_t grid, int block, int shared,
                           void* stream) {
    const Named* k = find(name);
    if (!k) return hsnw_fail(HSNW_E_NAME, "launch: no kernel of that name");
    if (!args) return hsnw_fail(HSNW_E_ARG, "launch: args is null");
    if (int rc = hsnw_require_prepared()) return rc;
    if (grid <= 0) return HSNW_OK;
    if (block < 32 || block > 1024 || (block & 31) || shared < 0 || static_cast<size_t>(shared) > hsnw_max_shared())
        return hsnw_fail(HSNW_E_ARG, "launch: block must be a multiple of 32 in [32, 1024] and shared within the device's limit");
    k->kernel<<<static_cast<unsigned>(grid), block, shared, static_cast<cudaStream_t>(stream)>>>(*args);
    return hsnw_check_launch(name);
}

extern "C" int hsnw_loop(const char* const* names, int count, const int64_t* grids, const int* blocks,
                         const int* shareds, const HsnWinArgs* args, int64_t steps, int slot, void* stream) {
    if (!names || !grids || !blocks || !shareds || !args || count < 1 || slot < 0 || slot >= HSN_WIN_INTS)
        return hsnw_fail(HSNW_E_ARG, "loop: invalid loop descriptor");
    HsnWinArgs local = *args;
    for (int64_t t = 0; t < steps; ++t) {
        local.i[slot] = static_cast<int32_t>(t);
        for (int k = 0; k < count; ++k)
            if (int rc = hsnw_launch(names[k], &local, grids[k], blocks[k], shareds[k], stream)) return rc;
    }
    return HSNW_OK;
}

extern "C" int hsnw_launch_shape(const char* name, const HsnWinArgs* a, int64_t* grid, int* block, int* shared) {
    if (!find(name)) return hsnw_fail(HSNW_E_NAME, "launch_shape: no kernel of that name");
    if (!a || !grid || !block || !shared) return hsnw_fail(HSNW_E_ARG, "launch_shape: null argument");
    const size_t cap = hsnw_max_shared() ? hsnw_max_shared() : 227 * 1024;
    size_t bytes = 0;
    *grid = a->i[0];
    if (strcmp(name, "hsn_win_select") == 0) {
        const int N = a->i[1], M = a->i[2], K = a->i[3];
        if (N < 1 || M < 1 || K < 1 || K > N) return hsnw_fail(HSNW_E_ARG, "select: need 1 <= K <= N and M >= 1");
        if (K > 64 || M > 64) return hsnw_fail(HSNW_E_UNSUPPORTED, "select: at most 64 slots and 64 units");
        *block = N >= 1024 ? 1024 : round_up32(N < 64 ? 64 : N);
        bytes = sizeof(float) * 2 * static_cast<size_t>(N);
    } else if (strcmp(name, "hsn_win_cell_update") == 0) {
        const int N = a->i[1], d = a->i[2], K = a->i[3];
        if (N < 1 || d < 1 || K < 1) return hsnw_fail(HSNW_E_ARG, "cell_update: sizes must be positive");
        *block = 256;
        bytes = sizeof(float) * (static_cast<size_t>(N) + 2 * static_cast<size_t>(K) * d + 2 * K);
    } else if (strcmp(name, "hsn_win_recurrence") == 0) {
        const int K = a->i[2], d = a->i[3], N = a->i[4];
        if (N < 1 || d < 1 || K < 1) return hsnw_fail(HSNW_E_ARG, "recurrence: sizes must be positive");
        const int kd = K * d;
        *block = kd >= 1024 ? 1024 : round_up32(kd < 64 ? 64 : kd);
        bytes = sizeof(float) * (static_cast<size_t>(N) + 1) * d;
    } else if (strcmp(name, "hsn_win_recurrence_dense") == 0) {
        const int N = a->i[2], d = a->i[3];
        if (N < 1 || d < 1) return hsnw_fail(HSNW_E_ARG, "recurrence_dense: sizes must be positive");
        *block = 256;
        bytes = sizeof(float) * (static_cast<size_t>(N) + 1) * d;
    } else if (strcmp(name, "hsn_win_back_head") == 0 || strcmp(name, "hsn_win_back_mid") == 0 ||
               strcmp(name, "hsn_win_back_tail") == 0) {
        // one warp per slot; the sizes sit at different slots of the three descriptors
        const bool head = name[13] == 'h', tail = name[13] == 't';
        const int K = a->i[2], d = a->i[3], N = head || tail ? a->i[4] : 1;
        const int F = head ? a->i[7] : tail ? a->i[5] : a->i[6];
        if (K < 1 || d < 1 || N < 1 || a->i[1] < 1) return hsnw_fail(HSNW_E_ARG, "back: sizes must be positive");
        if (F < 0 || F >= K) return hsnw_fail(HSNW_E_ARG, "back: the fixed slots must leave a routed slot");
        *block = tail ? 256 : (K >= 32 ? 1024 : (K < 2 ? 64 : 32 * K));
        bytes = head ? sizeof(float) * d : tail ? sizeof(float) * (2 * static_cast<size_t>(K) * d + N) : 0;
    } else {
        return hsnw_fail(HSNW_E_NAME, "launch_shape: no kernel of that name");
    }
    if (bytes > cap) return hsnw_fail(HSNW_E_UNSUPPORTED, "the row's working set exceeds a block's shared memory");
    *shared = static_cast<int>(bytes);
    return HSNW_OK;
}

// ------------------------------------------------------------------------------------------------
// Launch timing (measurement runs only; one profile at a time, from one host thread).
// ------------------------------------------------------------------------------------------------
bool g_hsnw_profile_on = false;
namespace {
struct ProfileMark { cudaEvent_t event; int kind; };
std::vector<ProfileMark> profile_marks;
cudaStream_t profile_stream = nullptr;
const char* const kind_names[HSNW_K_KINDS] = {"init", "pre", "front", "row", "unit", "update", "head", "mid", "tail_head", "rows_fwd", "rows_bwd", "prologue", "decode", "units_fwd", "units_bwd", "scorer_fwd", "scorer_bwd", "tail_fwd", "tail_bwd", "gate_fwd", "gate_bwd", "msg_fwd", "msg_bwd"};
}  // namespace

void hsnw_profile_mark_slow(int kind, cudaStream_t stream) {
    ProfileMark mark{nullptr, kind};
    if (cudaEventCreate(&mark.event) != cudaSuccess) return;
    cudaEventRecord(mark.event, stream);
    profile_stream = stream;
    profile_marks.push_back(mark);
}

extern "C" int hsnw_profile_begin(void) {
    if (g_hsnw_profile_on) return hsnw_fail(HSNW_E_STATE, "profile_begin: a profile is already running");
    profile_marks.clear();
    g_hsnw_profile_on = true;
    return HSNW_OK;
}

extern "C" int hsnw_profile_kinds(void) { return HSNW_K_KINDS; }
extern "C" const char* hsnw_profile_kind_name(int kind) {
    return kind >= 0 && kind < HSNW_K_KINDS ? kind_names[kind] : "";
}

extern "C" int hsnw_profile_end(double* ms_by_kind, int64_t* launches_by_kind, int kinds) {
    if (!g_hsnw_profile_on) return hsnw_fail(HSNW_E_STATE, "profile_end: no profile is running");
    g_hsnw_profile_on = false;
    if (!ms_by_kind || !launches_by_kind || kinds < HSNW_K_KINDS)
        return hsnw_fail(HSNW_E_ARG, "profile_end: needs room for hsnw_profile_kinds() entries");
    for (int k = 0; k < kinds; ++k) {
        ms_by_kind[k] = 0.0;
        launches_by_kind[k] = 0;
    }
    int rc = HSNW_OK;
    if (!profile_marks.empty()) {
        cudaEvent_t last;
        if (cudaEventCreate(&last) != cudaSuccess || cudaEventRecord(last, profile_stream) != cudaSuccess
            || cudaEventSynchronize(last) != cudaSuccess) {
            rc = hsnw_fail(HSNW_E_CUDA, "profile_end: could not record the closing event");
        } else {
            for (size_t i = 0; i < profile_marks.size(); ++i) {
                float ms = 0.0f;
                const cudaEvent_t next = i + 1 < profile_marks.size() ? profile_marks[i + 1].event : last;
                if (cudaEventElapsedTime(&ms, profile_marks[i].event, next) == cudaSuccess) {
                    ms_by_kind[profile_marks[i].kind] += ms;
                    launches_by_kind[profile_marks[i].kind] += 1;
                }
            }
        }
        cudaEventDestroy(last);
    }
    for (ProfileMark& mark : profile_marks) cudaEventDestroy(mark.event);
    profile_marks.clear();
    return rc;
}
