// Error reporting of the kernel library: the last failure's message, per host thread.
#include <stdarg.h>

#include "api.h"
#include "common.cuh"
#include "launch.cuh"

int g_rdl_programmatic_launch = 1;

extern "C" void rdl_set_programmatic_launch(int on) { g_rdl_programmatic_launch = on ? 1 : 0; }

// rdl_set_wait_test: which kernel (by fault code) runs with a short wait limit, the limit, the extra bytes
int g_rdl_wait_test_code = 0;
long long g_rdl_wait_test_cycles = 0;
int g_rdl_wait_test_extra = 0;

extern "C" void rdl_set_wait_test(int code, long long cycles, int extra_tx_bytes) {
    g_rdl_wait_test_code = code;
    g_rdl_wait_test_cycles = code ? cycles : 0;
    g_rdl_wait_test_extra = code ? extra_tx_bytes : 0;
}

int rdl_sm_count() {
    static int count[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (count[dev] == 0) {
        int n = 0;
        count[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 1;
    }
    return count[dev];
}

static thread_local char g_error[512] = "";

void rdl_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

extern "C" const char* rdl_last_error(void) { return g_error; }

// Bumped whenever a signature in api.h changes, so that a stale build is noticed on load.
extern "C" int rdl_abi_version(void) { return RDL_ABI_VERSION; }
