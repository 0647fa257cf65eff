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

// Launch counts by kernel name.  The launchers call ce_note() with a string literal; the table is
// small and searched linearly (a few dozen names), under a lock because launchers may be called from
// several host threads.
#include <mutex>
#include <string.h>
namespace {
struct Noted { const char* name; long long count; };
Noted g_noted[96];
int g_n_noted = 0;
std::mutex g_note_lock;
thread_local const char* g_last_noted = "";
}

void ce_note(const char* name) {
    g_last_noted = name;
    std::lock_guard<std::mutex> hold(g_note_lock);
    for (int i = 0; i < g_n_noted; ++i)
        if (g_noted[i].name == name || strcmp(g_noted[i].name, name) == 0) { ++g_noted[i].count; return; }
    if (g_n_noted < 96) g_noted[g_n_noted++] = Noted{name, 1};
}

// "name=count" lines of every kernel launched so far into buf (at most cap bytes, always terminated);
// returns the number of bytes the full list needs.
extern "C" int ce_kernel_counts(char* buf, int cap) {
    std::lock_guard<std::mutex> hold(g_note_lock);
    int need = 0;
    if (cap > 0) buf[0] = 0;
    for (int i = 0; i < g_n_noted; ++i) {
        char line[160];
        int n = snprintf(line, sizeof(line), "%s=%lld\n", g_noted[i].name, g_noted[i].count);
        if (need + n < cap) memcpy(buf + need, line, n + 1);
        need += n;
    }
    return need + 1;
}

extern "C" void ce_kernel_counts_reset() {
    std::lock_guard<std::mutex> hold(g_note_lock);
    g_n_noted = 0;
}

// The name the calling thread's last launch was counted under ("" before any).
extern "C" const char* ce_last_kernel() { return g_last_noted; }

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
