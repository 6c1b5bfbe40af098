// Status reporting, launch accounting and small device queries shared by the
// kernel families of libb2k.so.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "b2k_internal.cuh"

namespace b2k {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return B2K_OK;
    snprintf(g_error, sizeof g_error, "%s: %s (%s)", what, cudaGetErrorString(e),
             cudaGetErrorName(e));
    return static_cast<int>(e);
}

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int current_device() {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

int sm_count() {
    static std::atomic<int> cached[kMaxDevices];
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int env_read(const char *name) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : INT_MIN;
}

// NVTX 3 is header-only: the tools' injection library is looked up on the first call,
// and without a tool attached the calls return at once.
bool nvtx_enabled() {
    static const bool on = env_read("B2K_NVTX") > 0;
    return on;
}
void nvtx_push(const char *name) { nvtxRangePushA(name); }
void nvtx_pop() { nvtxRangePop(); }

}  // namespace b2k

extern "C" {

int b2k_version(void) { return 100; }

const char *b2k_last_error(void) { return b2k::g_error; }

int64_t b2k_launch_count(void) { return b2k::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
