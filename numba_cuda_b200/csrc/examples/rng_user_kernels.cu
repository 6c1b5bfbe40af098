// Example user kernels written against include/b2k_xoroshiro128p.cuh.  They play
// the role of the @cuda.jit kernels a numba-cuda user writes around the
// xoroshiro128p_* device functions; the test-suite builds them into
// libb2k_examples.so and checks that they consume the same stream as the
// reference functions would.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/b2k_xoroshiro128p.cuh"

// The 3-D strided fill of the reference's documentation example
// (numba/cuda/tests/doc_examples/test_random.py:22-36).
__global__ void random_3d(float *arr, int64_t n0, int64_t n1, int64_t n2, xoroshiro128p_state *rng_states) {
    const int startx = blockIdx.x * blockDim.x + threadIdx.x;
    const int starty = blockIdx.y * blockDim.y + threadIdx.y;
    const int startz = blockIdx.z * blockDim.z + threadIdx.z;
    const int stridex = gridDim.x * blockDim.x, stridey = gridDim.y * blockDim.y, stridez = gridDim.z * blockDim.z;
    const int64_t tid = (static_cast<int64_t>(startz) * stridey * stridex) + (static_cast<int64_t>(starty) * stridex) + startx;
    for (int64_t i = startz; i < n0; i += stridez)
        for (int64_t j = starty; j < n1; j += stridey)
            for (int64_t k = startx; k < n2; k += stridex)
                arr[(i * n1 + j) * n2 + k] = xoroshiro128p_uniform_float32(rng_states, tid);
}

// out[tid*count + i] = normal(states, tid): the shape of the reference's test
// kernels (tests/cudapy/test_random.py:43-53), register-resident style.
__global__ void normals_per_thread(xoroshiro128p_state *states, int64_t n, double *out, int count) {
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (tid >= n) return;
    xoroshiro128p_generator g(states, tid);
    for (int i = 0; i < count; ++i) out[tid * count + i] = g.normal_float64();
    g.store(states, tid);
}

extern "C" __attribute__((visibility("default"))) int b2k_example_random_3d(
    float *arr, int64_t n0, int64_t n1, int64_t n2, void *states, int gx, int gy, int gz, int bx, int by, int bz,
    void *stream) {
    random_3d<<<dim3(gx, gy, gz), dim3(bx, by, bz), 0, static_cast<cudaStream_t>(stream)>>>(
        arr, n0, n1, n2, static_cast<xoroshiro128p_state *>(states));
    return static_cast<int>(cudaGetLastError());
}

extern "C" __attribute__((visibility("default"))) int b2k_example_normals_per_thread(
    void *states, int64_t n, double *out, int count, void *stream) {
    normals_per_thread<<<static_cast<unsigned>((n + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<xoroshiro128p_state *>(states), n, out, count);
    return static_cast<int>(cudaGetLastError());
}
