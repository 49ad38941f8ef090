// Error text of the last failed entry point, and small queries about the device.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[1024] = "";

int gb_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

GB_API const char* gb_last_error() { return g_error; }

// Compute capability of the current device as major*10+minor; the package refuses
// anything but 100 (sm_100a code has no other target).
GB_API int gb_device_arch() {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    return major * 10 + minor;
}

GB_API int gb_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

// Programmatic dependent launch for the kernels that support it (on by default).
static int g_pdl = 1;
bool gb_pdl_enabled() { return g_pdl != 0; }
GB_API int gb_set_pdl(int on) {
    g_pdl = on;
    return 0;
}
