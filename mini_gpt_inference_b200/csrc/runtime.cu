// Error message store and device queries of the kernel library.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

int mg_set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

MG_API const char* mg_last_error() { return g_error; }

// Compute capability of `device` as major * 10 + minor, or a negative error code.
MG_API int mg_device_arch(int device) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess)
        return mg_set_error(MG_ERR_CUDA, "cannot query device %d", device);
    return major * 10 + minor;
}

MG_API int mg_set_device(int device) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return mg_set_error(MG_ERR_CUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    return MG_OK;
}

static int g_dependent_launch = 0;

int mg_dependent_launch_enabled() { return g_dependent_launch; }

// Turn programmatic dependent launch on (1) or off (0) for the kernels that support it.
MG_API int mg_set_dependent_launch(int on) {
    g_dependent_launch = on ? 1 : 0;
    return MG_OK;
}

// Whether the kernels of this build check the indices they read from device memory (-DMG_GUARDS).
MG_API int mg_guards_enabled() {
#ifdef MG_GUARDS
    return 1;
#else
    return 0;
#endif
}
