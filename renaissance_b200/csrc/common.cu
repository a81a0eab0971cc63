// Error text, version and device queries of the trb200 library.
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace trb {

char* last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

static std::atomic<unsigned long long> g_launches{0};

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

unsigned long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace trb

extern "C" const char* trb200_last_error(void) { return trb::last_error_buffer(); }

extern "C" int trb200_version(void) { return 100; }

namespace trb { unsigned long long launch_count(); }
extern "C" uint64_t trb200_kernel_launch_count(void) { return trb::launch_count(); }

extern "C" int trb200_device_arch(void) {
    int dev = 0, major = 0, minor = 0;
    TRB_CUDA_TRY(cudaGetDevice(&dev));
    TRB_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    TRB_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    return major * 10 + minor;
}
