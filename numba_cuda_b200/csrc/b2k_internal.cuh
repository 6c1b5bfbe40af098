// Shared host/device helpers for libb2k.so (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <climits>
#include <mutex>

#include "../../include/b2k.h"

namespace b2k {

// Records a thread-local message and returns `code` (see b2k_last_error()).
int fail(int code, const char *fmt, ...);
// Converts a cudaError_t of a launch/API call into the ABI's positive status.
int check_cuda(cudaError_t e, const char *what);
// Counts kernels launched by this library (reported by b2k_launch_count()).
void note_launch(int n = 1);
// Streaming multiprocessors of the current device (cached per device).
int sm_count();
// Integer knob from the environment (development aid): INT_MIN when unset.
int env_read(const char *name);
// Ordinal of the current device, or -1.
int current_device();
// An NVTX range around one C-ABI call, so that a timeline or an ncu capture can be
// filtered by entry point.  Off unless B2K_NVTX=1 is in the environment (one cached
// flag test per call otherwise).
bool nvtx_enabled();
void nvtx_push(const char *name);
void nvtx_pop();
struct Range {
    const bool on;
    explicit Range(const char *name) : on(nvtx_enabled()) {
        if (on) nvtx_push(name);
    }
    ~Range() {
        if (on) nvtx_pop();
    }
    Range(const Range &) = delete;
    Range &operator=(const Range &) = delete;
};
#define B2K_RANGE(name) b2k::Range b2k_range__(name)

// Set-up that has to happen once on EVERY device a process uses (function
// attributes such as the dynamic shared-memory limit belong to a device, not to
// the process).  `run` remembers per device ordinal what `f` returned.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
    std::atomic<int> done[kMaxDevices];
    cudaError_t status[kMaxDevices];
    std::mutex mu;
    template <typename F>
    cudaError_t run(F &&f) {
        const int dev = current_device();
        if (dev < 0 || dev >= kMaxDevices) return f();
        if (done[dev].load(std::memory_order_acquire)) return status[dev];
        std::lock_guard<std::mutex> lock(mu);
        if (!done[dev].load(std::memory_order_relaxed)) {
            status[dev] = f();
            done[dev].store(1, std::memory_order_release);
        }
        return status[dev];
    }
};

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

template <typename T>
inline bool aligned_to(const void *p, size_t a) {
    return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

// TMA tile transposes (b2k_transpose_tma.cu).  Both return B2K_OK when they
// launched, a positive cudaError_t when the launch failed, and B2K_ERR_UNSUPPORTED
// when the arrays do not meet the tensor-map rules (the caller then takes a
// general kernel).
int transpose_tma(const void *in, void *out, int64_t rows, int64_t cols, int64_t in_stride0, int64_t in_stride1,
                  int64_t out_stride0, int64_t out_stride1, int64_t itemsize, cudaStream_t stream);
int transpose_tma_batched(const void *in, void *out, int64_t rows, int64_t cols, int64_t in_pitch,
                          int64_t out_pitch, int nbatch, const int64_t *batch_len, const int64_t *in_batch_step,
                          const int64_t *out_batch_step, int64_t itemsize, cudaStream_t stream);

}  // namespace b2k

// A knob read from the environment ONCE per call site (a function-local static),
// so that launch paths pay one load for it.
#define B2K_ENV_INT(name, fallback)                                        \
    ([&]() -> int {                                                        \
        static const int v__ = b2k::env_read(name);                        \
        return v__ == INT_MIN ? static_cast<int>(fallback) : v__;          \
    }())

#define B2K_RETURN_IF_LAUNCH_FAILED(what)                      \
    do {                                                       \
        cudaError_t e__ = cudaGetLastError();                  \
        if (e__ != cudaSuccess) return b2k::check_cuda(e__, what); \
    } while (0)
