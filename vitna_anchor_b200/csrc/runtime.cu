// Small services of the kernel library: error text and a device check.
#include "common.cuh"

VK_API const char* vk_error_string(int status) {
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    switch (status) {
        case VK_OK: return "ok";
        case VK_BAD_SHAPE: return "a size this kernel does not take";
        case VK_BAD_ALIGNMENT: return "a pointer or stride is not aligned as the kernel needs";
        case VK_TOO_LARGE: return "a size beyond the kernel's stated maximum";
        default: return "unknown status";
    }
}

// The compute capability of the current device as major * 10 + minor, or the negated cudaError_t.
VK_API int vk_device_arch() {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) return -(int)e;
    return major * 10 + minor;
}
