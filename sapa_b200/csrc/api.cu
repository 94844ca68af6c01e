// api.cu — error and dispatch plumbing of the C ABI: a thread-local message buffer (never exit()/abort()) and a
// process-wide record of the kernels the last entry-point call launched.
#include "common.cuh"

#include <cstring>
#include <mutex>

namespace sapa {

static thread_local char g_error[512] = "";
// Kernels launched by the most recent entry-point call of the PROCESS (not of the thread: PyTorch runs the backward of
// an autograd Function on its own worker thread, and the caller must still be able to ask what ran).
static std::mutex g_kernels_lock;
static char g_kernels[512] = "";
static thread_local char g_kernels_copy[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void trace_reset() {
    std::lock_guard<std::mutex> guard(g_kernels_lock);
    g_kernels[0] = '\0';
}

void trace_kernel(const char *name) {
    std::lock_guard<std::mutex> guard(g_kernels_lock);
    const size_t used = strlen(g_kernels), add = strlen(name);
    if (used + add + 2 > sizeof(g_kernels)) return;
    if (used != 0) g_kernels[used] = ',';
    memcpy(g_kernels + used + (used != 0), name, add + 1);
}

int check_launch(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) {
        trace_kernel(what);
        return SAPA_OK;
    }
    set_error("%s: launch failed: %s", what, cudaGetErrorString(err));
    return SAPA_ERR_LAUNCH;
}

}  // namespace sapa

extern "C" {

const char *sapa_last_error(void) { return sapa::g_error; }

const char *sapa_last_kernels(void) {
    std::lock_guard<std::mutex> guard(sapa::g_kernels_lock);
    memcpy(sapa::g_kernels_copy, sapa::g_kernels, sizeof(sapa::g_kernels));
    return sapa::g_kernels_copy;
}

int sapa_abi_version(void) { return 3; }

}  // extern "C"
