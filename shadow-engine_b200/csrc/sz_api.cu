// Library-wide pieces of the C ABI: version, per-thread error text.
#include "sz_common.cuh"

#include <string.h>

static thread_local char g_err[512] = "";

void sz_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sz_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char* sz_version(void) { return "shadowzero_b200 0.1 (sm_100a)"; }
extern "C" const char* sz_last_error(void) { return g_err; }
