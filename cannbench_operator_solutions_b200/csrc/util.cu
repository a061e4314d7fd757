// Library identification, status strings and small host utilities.
#include <atomic>

#include "common.cuh"

namespace w8a8 {

int sm_count()
{
    // one cached value per device ordinal; races only ever write the same value
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return 148;
    }
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            n = 148;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

static std::atomic<int64_t> g_kernel_launches{0};

void note_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }

}  // namespace w8a8

extern "C" int64_t w8a8_kernel_launch_count(void)
{
    return w8a8::g_kernel_launches.load(std::memory_order_relaxed);
}

extern "C" int w8a8_version(void) { return 100; }

extern "C" const char* w8a8_status_string(int status)
{
    switch (status) {
    case W8A8_OK:
        return "ok";
    case W8A8_ERR_INVALID:
        return "invalid argument (shape, dtype, flag or null pointer)";
    case W8A8_ERR_ALIGN:
        return "pointer or pitch alignment requirement not met";
    case W8A8_ERR_GROUP_LIST:
        return "group_list must be a non-decreasing cumulative list ending at M";
    case W8A8_ERR_WORKSPACE:
        return "workspace missing or too small";
    case W8A8_ERR_CUDA:
        return "CUDA runtime or driver call failed";
    case W8A8_ERR_UNSUPPORTED:
        return "configuration not supported by this build";
    case W8A8_ERR_LIMIT:
        return "problem exceeds a fixed capacity limit of this entry point (see its declaration in w8a8ffn.h)";
    default:
        return "unknown status";
    }
}
