// Error text of the last refused call (per host thread) and a version probe.
#include "common.cuh"
#include <stdarg.h>

static thread_local char g_err[512] = "";

void rb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

extern "C" const char* rb_last_error() { return g_err; }

extern "C" int rb_abi_version() { return 1; }

int g_rb_pdl = 1;
// Programmatic dependent launch on (1) or off (0) for the kernels that support it; returns the old value.
extern "C" int rb_set_pdl(int on) { int old = g_rb_pdl; g_rb_pdl = on ? 1 : 0; return old; }

// Compute capability of the current device as major*10+minor, or a negative cudaError_t.
extern "C" int rb_device_cc() {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -(int)e;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return -(int)e;
    e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) return -(int)e;
    return major * 10 + minor;
}
