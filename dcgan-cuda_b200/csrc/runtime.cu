// Library-wide state: last-error text, launch counter, device properties.
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace dcg {

namespace {
thread_local char g_last_error[512] = "";
std::atomic<uint64_t> g_launches{0};
}  // namespace

char* last_error_buffer() { return g_last_error; }

int fail(int status, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return status;
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launches_total() { return g_launches.load(std::memory_order_relaxed); }

int sm_count()
{
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace dcg

extern "C" const char* dcg_last_error(void) { return dcg::last_error_buffer(); }

extern "C" const char* dcg_build_info(void)
{
    return "dcgan_b200 0.1 (sm_100a; tcgen05 TF32 implicit-GEMM conv, fp32 CUDA-core reference path)";
}

extern "C" uint64_t dcg_launches_total(void) { return dcg::launches_total(); }
