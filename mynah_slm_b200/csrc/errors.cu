// Error reporting of the exported entry points: the message of the last
// failure of the calling thread, returned as text. The library never prints
// (the reference's rule for its public API, mynah-slm include/mynah_slm.h:4-8).
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

int mynah_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return -1;
}

int mynah_check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return mynah_fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

MYNAH_API const char* mynah_last_error(void) { return g_error; }

// Compute capability of the current device as major*10+minor, or a negative
// code; the Python side refuses anything but 100 before the first launch.
MYNAH_API int mynah_device_arch(void) {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return mynah_fail("no CUDA device is current");
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    return major * 10 + minor;
}

int mynah_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) return 1;
        cached[dev] = n;
    }
    return cached[dev];
}

// Programmatic dependent launch of the decode-path kernels. Off by default: on this part the decode step
// measured slower with it (dependents that become resident early take slots from the running kernel).
static int g_pdl = 0;
int mynah_pdl_enabled() { return g_pdl; }
MYNAH_API int mynah_set_pdl(int on) {
    g_pdl = on ? 1 : 0;
    return 0;
}

// A bounded wait that runs out, for tests of the host's handling of status bit 16: one thread waits for a word of
// global memory that nothing sets, for at most `limit_ns` of wall clock (a few tens of microseconds), then sets
// MYNAH_ST_TIMEOUT in `status` and returns. The same shape as the bounded waits of the tensor-core kernels
// (a limit, a status bit, nothing left in flight), without any of their machinery.
#include "layout.cuh"

__global__ void wait_probe_kernel(const volatile int* flag, int* status, unsigned long long limit_ns) {
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned it = 0; it < (1u << 24); it++) {              // a bound on iterations as well as on time
        if (*flag != 0) return;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > limit_ns) break;
    }
    atomicOr(status, MYNAH_ST_TIMEOUT);
}

MYNAH_API int mynah_wait_probe(const int* flag, int* status, unsigned long long limit_ns, cudaStream_t stream) {
    MYNAH_REQUIRE(flag != nullptr && status != nullptr && limit_ns <= 1000000ull, "wait_probe: a flag, a status word and a limit of at most 1 ms");
    wait_probe_kernel<<<1, 1, 0, stream>>>(flag, status, limit_ns);
    return mynah_check_launch("wait_probe");
}
