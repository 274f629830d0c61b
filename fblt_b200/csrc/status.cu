// Status strings, thread-local error text and the launch counter.
#include "common.cuh"

#include <atomic>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

namespace fblt {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

// FBLT_REPORT_LAUNCHES=1: one line on stderr when the process ends, so that a host program that
// only links the library (no call to fblt_launch_count of its own) can show that its attention
// ran on these kernels.
struct ExitReport {
    ~ExitReport() {
        const char *e = getenv("FBLT_REPORT_LAUNCHES");
        if (e && e[0] == '1')
            fprintf(stderr, "[fblt] %llu kernel launches\n", (unsigned long long)g_launches.load(std::memory_order_relaxed));
    }
};
static ExitReport g_exit_report;

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(FBLT_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return FBLT_OK;
}

} // namespace fblt

extern "C" const char *fblt_last_error(void) { return fblt::g_err; }

extern "C" const char *fblt_status_string(int status) {
    switch (status) {
    case FBLT_OK: return "ok";
    case FBLT_ERR_ARG: return "invalid argument";
    case FBLT_ERR_UNSUPPORTED: return "unsupported shape for the requested kernel";
    case FBLT_ERR_WORKSPACE: return "workspace missing or too small";
    case FBLT_ERR_CUDA: return "CUDA runtime error";
    case FBLT_ERR_CAPACITY: return "capacity exceeded";
    case FBLT_ERR_LIMIT: return "size beyond a fixed maximum";
    case FBLT_ERR_PEER: return "another rank announced a failure";
    case FBLT_ERR_TIMEOUT: return "a host-side deadline passed";
    default: return "unknown status";
    }
}

extern "C" const char *fblt_version(void) { return "fblt_attn sm_100a 1"; }

extern "C" uint64_t fblt_launch_count(void) { return fblt::g_launches.load(std::memory_order_relaxed); }
