// Error reporting shared by all launchers.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

extern "C" const char* ce_last_error() { return g_error; }

int ce_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int ce_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ce_fail(CE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return CE_OK;
}

// Lets the Python side confirm which library it loaded and for which architecture it was built.
extern "C" int ce_build_arch() {
#ifdef CE_BUILD_ARCH
    return CE_BUILD_ARCH;
#else
    return 0;
#endif
}
