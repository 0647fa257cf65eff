// Error reporting shared by all launchers.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

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

// Programmatic dependent launch is on unless switched off (ce_set_pdl(0), or CE_PDL=0 in the environment).
static int g_pdl = -1;
bool ce_pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("CE_PDL");
        g_pdl = (e && e[0] == '0') ? 0 : 1;
    }
    return g_pdl != 0;
}
extern "C" void ce_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// Multiprocessors of the current device (asked once).
int ce_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}
