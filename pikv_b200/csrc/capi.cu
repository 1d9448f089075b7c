// Library-wide state of the C ABI: version, per-thread error text, launch counter.
#include "common.cuh"

#include <atomic>
#include <mutex>

namespace pikv {

static thread_local char g_err[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return PIKV_ECUDA;
    }
    return PIKV_OK;
}

}  // namespace pikv

extern "C" {

int pikv_abi_version(void) { return PIKV_ABI_VERSION; }
const char* pikv_last_error(void) { return pikv::g_err; }
uint64_t pikv_launch_count(void) { return pikv::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
