// Small services of the kernel library: error text and a device check.
#include "tcgen05_common.cuh"

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

// ---------------------------------------------------------------------------------------------------------------
// Bounded waits: the limit in force, and a one-shot fault for tests of the give-up path.

namespace vk {

static unsigned long long g_wait_cycles = TC_WAIT_CYCLES;
static int g_skip_family = 0, g_skip_stage = -1;

WaitCtl wait_ctl(int* error, int family) {
    WaitCtl wc;
    wc.error = error;
    wc.cycles = g_wait_cycles;
    wc.skip_stage = -1;
    if (g_skip_family == family) {      // taken by this launch alone
        wc.skip_stage = g_skip_stage;
        g_skip_family = 0;
        g_skip_stage = -1;
    }
    return wc;
}

}  // namespace vk

// The limit of one wait on an mbarrier in clock cycles of the device, for every launch from now on (0: the default,
// about a second).  Returns the limit that was in force.
VK_API unsigned long long vk_set_wait_limit_cycles(unsigned long long cycles) {
    const unsigned long long before = vk::g_wait_cycles;
    vk::g_wait_cycles = cycles ? cycles : vk::TC_WAIT_CYCLES;
    return before;
}

// The same limit given in milliseconds at the device's highest clock (a slower clock makes the wait longer, never
// shorter).  ms <= 0: the default.  Returns 0, or the cudaError_t of the attribute query.
VK_API int vk_set_wait_limit_ms(double ms) {
    if (ms <= 0.0) { vk::g_wait_cycles = vk::TC_WAIT_CYCLES; return 0; }
    int dev = 0, khz = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    if (e != cudaSuccess) return (int)e;
    const double cycles = ms * (double)khz;
    vk::g_wait_cycles = cycles < 1000.0 ? 1000ull : (unsigned long long)cycles;
    return 0;
}

// For tests: the next launch of a kernel family (1 the tcgen05 product, 2 its wide variant, 3 the tcgen05 prompt
// attention) leaves stage `stage` of every block unarmed and unfilled, so that the waits on it run out, the kernel
// sets the error word and returns by itself.  No address is out of range and nothing traps.
VK_API void vk_test_skip_stage(int family, int stage) {
    vk::g_skip_family = family;
    vk::g_skip_stage = stage;
}
