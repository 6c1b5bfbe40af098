// Status reporting, launch accounting and small device queries shared by the
// kernel families of libb2k.so.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

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

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int env_int(const char *name, int fallback) {
    // The environment is read once per name; callers may pass different
    // fallbacks for the same name, so only the parsed variable is cached.
    static std::mutex mu;
    static std::unordered_map<std::string, std::pair<bool, int>> seen;
    std::lock_guard<std::mutex> lock(mu);
    auto it = seen.find(name);
    if (it == seen.end()) {
        const char *v = getenv(name);
        const bool set = v && *v;
        it = seen.emplace(name, std::make_pair(set, set ? atoi(v) : 0)).first;
    }
    return it->second.first ? it->second.second : fallback;
}

}  // namespace b2k

extern "C" {

int b2k_version(void) { return 100; }

const char *b2k_last_error(void) { return b2k::g_error; }

int64_t b2k_launch_count(void) { return b2k::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
