// api.cu — error plumbing of the C ABI: a thread-local message buffer, never exit()/abort().
#include "common.cuh"

#include <cstring>

namespace sapa {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int check_launch(const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return SAPA_OK;
    set_error("%s: launch failed: %s", what, cudaGetErrorString(err));
    return SAPA_ERR_LAUNCH;
}

}  // namespace sapa

extern "C" {

const char *sapa_last_error(void) { return sapa::g_error; }

int sapa_abi_version(void) { return 1; }

}  // extern "C"
