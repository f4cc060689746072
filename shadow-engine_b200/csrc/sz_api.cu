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

// ---- per-kernel timing --------------------------------------------------------------------------------------------------------
// The role of the reference's SHADOWZERO_KTIME switch (crates/shadowzero-cuda/src/kernels.rs:527-536,604): while a trace is open,
// every kernel the library launches on this thread is followed by a cudaEventRecord of the next event of the caller's list, so
// event i+1 minus event i is kernel i's time on the stream.  Recording an event between two kernels keeps them from overlapping,
// so a traced pass is for attribution, not for the headline number.
static thread_local cudaEvent_t* g_tr_events = nullptr;
static thread_local int g_tr_cap = 0, g_tr_n = 0;
static thread_local const char* g_tr_names[1024];

void sz_trace_mark(const char* name, cudaStream_t stream) {
    if (!g_tr_events || g_tr_n >= g_tr_cap || g_tr_n >= 1024) return;
    g_tr_names[g_tr_n] = name;
    cudaEventRecord(g_tr_events[g_tr_n], stream);
    g_tr_n++;
}

bool sz_trace_active() { return g_tr_events != nullptr; }

extern "C" int sz_trace_begin(uint64_t* events, int capacity, uint64_t stream) {
    if (!events || capacity < 2) return sz_fail(SZ_E_ARG, "sz_trace_begin: needs a list of at least two events");
    g_tr_events = (cudaEvent_t*)events;
    g_tr_cap = capacity;
    g_tr_n = 0;
    sz_trace_mark("begin", (cudaStream_t)stream);
    return SZ_OK;
}

extern "C" int sz_trace_end(void) {
    const int n = g_tr_n;
    g_tr_events = nullptr;
    g_tr_cap = 0;
    return n;
}

extern "C" const char* sz_trace_name(int i) { return (i >= 0 && i < g_tr_n) ? g_tr_names[i] : ""; }
