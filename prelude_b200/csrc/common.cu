// Error message storage and library identification.
#include "common.cuh"

#include <stdarg.h>
#include <stdlib.h>

static thread_local char g_pb_error[1024] = "";

int pb_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_pb_error, sizeof(g_pb_error), fmt, ap);
    va_end(ap);
    return 1;
}

bool pb_pdl_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* off = getenv("PRELUDE_NO_PDL");
        state = (off && off[0] && off[0] != '0') ? 0 : 1;
    }
    return state == 1;
}

// Message of the last failed call on this thread.
PB_API const char* pb_last_error() { return g_pb_error; }

// Interface version: the Python side refuses a library built from other sources.
PB_API int pb_abi_version() { return 16; }

// Compute capability the library was compiled for (major*10 + minor).
PB_API int pb_built_for_sm() { return 100; }

// Device check: 0 when the current device can run this library.
PB_API int pb_check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return pb_fail("cudaGetDevice: %s", cudaGetErrorString(e));
    int major = 0, minor = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (major != 10)
        return pb_fail("this library holds sm_100a code only; device %d is sm_%d%d", dev, major, minor);
    return 0;
}
