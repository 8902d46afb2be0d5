// Error plumbing shared by every C-ABI entry point: a thread-local message buffer
// read through natsl_last_error(), and a launch check that maps CUDA errors to a
// negative status instead of aborting.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"
#include "../../include/natsl_b200.h"

namespace natsl {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
        return NATSL_ERR_CUDA;
    }
    return NATSL_OK;
}

}  // namespace natsl

extern "C" const char* natsl_last_error(void) { return natsl::g_err; }

extern "C" int natsl_abi_version(void) { return NATSL_B200_ABI_VERSION; }
