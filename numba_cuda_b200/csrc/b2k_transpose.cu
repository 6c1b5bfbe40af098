// 2-D transpose of device arrays: out[j, i] = in[i, j].
//
// The reference compiles a fresh 32x33 shared-tile kernel on every call and
// moves one element per thread (numba/cuda/kernels/transpose.py:42-63).  This
// file holds the layout-general kernels (any byte strides on either side, any
// item size); the TMA tile kernel for contiguous power-of-two items lives in
// b2k_transpose_tma.cu and is tried first.
#include "b2k_internal.cuh"

namespace {

constexpr int kTile = 32;
constexpr int kBlockRows = 8;

// Power-of-two items: padded shared tile, both global sides walk their own
// fastest-varying direction.
template <typename T>
__global__ void __launch_bounds__(kTile *kBlockRows)
transpose_tile_kernel(const char *__restrict__ in, char *__restrict__ out, int64_t rows, int64_t cols,
                      int64_t is0, int64_t is1, int64_t os0, int64_t os1, int64_t tiles_x) {
    __shared__ T tile[kTile][kTile + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t tile_id = blockIdx.x;
    const int64_t col0 = (tile_id % tiles_x) * kTile;
    const int64_t row0 = (tile_id / tiles_x) * kTile;
#pragma unroll
    for (int k = 0; k < kTile; k += kBlockRows) {
        const int64_t r = row0 + ty + k, c = col0 + tx;
        if (r < rows && c < cols) tile[ty + k][tx] = *reinterpret_cast<const T *>(in + r * is0 + c * is1);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTile; k += kBlockRows) {
        const int64_t orow = col0 + ty + k, ocol = row0 + tx;  // output coordinates
        if (orow < cols && ocol < rows) *reinterpret_cast<T *>(out + orow * os0 + ocol * os1) = tile[tx][ty + k];
    }
}

// Any item size (records, odd sizes): one item per thread, W-byte pieces.
template <typename W>
__global__ void __launch_bounds__(256)
transpose_items_kernel(const char *__restrict__ in, char *__restrict__ out, int64_t rows, int64_t cols,
                       int64_t is0, int64_t is1, int64_t os0, int64_t os1, int64_t itemsize) {
    const int64_t total = rows * cols;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t pieces = itemsize / static_cast<int64_t>(sizeof(W));
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t i = idx % rows;  // input row = output column (fastest on the output side)
        const int64_t j = idx / rows;
        const W *src = reinterpret_cast<const W *>(in + i * is0 + j * is1);
        W *dst = reinterpret_cast<W *>(out + j * os0 + i * os1);
        for (int64_t p = 0; p < pieces; ++p) dst[p] = src[p];
    }
}

bool all_multiple_of(int64_t a, std::initializer_list<int64_t> values) {
    for (int64_t v : values)
        if (v % a != 0) return false;
    return true;
}

template <typename T>
int launch_tile(const void *in, void *out, int64_t rows, int64_t cols, int64_t is0, int64_t is1,
                int64_t os0, int64_t os1, cudaStream_t stream) {
    const int64_t tiles_x = (cols + kTile - 1) / kTile;
    const int64_t tiles_y = (rows + kTile - 1) / kTile;
    const int64_t tiles = tiles_x * tiles_y;
    if (tiles > 0x7FFFFFFFll) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_transpose2d: too many tiles");
    transpose_tile_kernel<T><<<static_cast<unsigned>(tiles), dim3(kTile, kBlockRows), 0, stream>>>(
        static_cast<const char *>(in), static_cast<char *>(out), rows, cols, is0, is1, os0, os1, tiles_x);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_transpose2d launch");
    return B2K_OK;
}

template <typename W>
int launch_items(const void *in, void *out, int64_t rows, int64_t cols, int64_t is0, int64_t is1,
                 int64_t os0, int64_t os1, int64_t itemsize, cudaStream_t stream) {
    const int64_t total = rows * cols;
    int64_t grid = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(b2k::sm_count()) * 16;
    if (grid > cap) grid = cap;
    transpose_items_kernel<W><<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<const char *>(in), static_cast<char *>(out), rows, cols, is0, is1, os0, os1, itemsize);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_transpose2d launch");
    return B2K_OK;
}

}  // namespace

extern "C" int b2k_transpose2d(const void *in_dev, void *out_dev, int64_t rows, int64_t cols,
                               int64_t in_stride0, int64_t in_stride1, int64_t out_stride0,
                               int64_t out_stride1, int64_t itemsize, void *stream) {
    B2K_RANGE("b2k_transpose2d");
    if (rows < 0 || cols < 0 || itemsize <= 0)
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_transpose2d: bad shape or item size");
    if (rows == 0 || cols == 0) return B2K_OK;
    if (!in_dev || !out_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_transpose2d: null pointer");
    cudaStream_t s = b2k::as_stream(stream);

    if (B2K_ENV_INT("B2K_TRANSPOSE_NO_TMA", 0) == 0) {
        const int rc = b2k::transpose_tma(in_dev, out_dev, rows, cols, in_stride0, in_stride1,
                                          out_stride0, out_stride1, itemsize, s);
        if (rc != B2K_ERR_UNSUPPORTED) return rc;
    }

    // Items of up to 4 bytes: the 64x64 tiles of the strided-assignment kernels measured
    // 15-25 % faster than the 32x32 tiles below (out[j, i] = in[i, j] is an assignment
    // whose source strides are swapped).
    if ((itemsize == 1 || itemsize == 2 || itemsize == 4) && B2K_ENV_INT("B2K_TRANSPOSE_VIA_ASSIGN", 1) != 0) {
        const int64_t shape[2] = {cols, rows};
        const int64_t dst_steps[2] = {out_stride0, out_stride1};
        const int64_t src_steps[2] = {in_stride1, in_stride0};
        return b2k_assign(out_dev, in_dev, 2, shape, dst_steps, src_steps, itemsize, stream);
    }

    const int64_t base_in = static_cast<int64_t>(reinterpret_cast<uintptr_t>(in_dev));
    const int64_t base_out = static_cast<int64_t>(reinterpret_cast<uintptr_t>(out_dev));
    auto fits = [&](int64_t a) {
        return all_multiple_of(a, {base_in, base_out, in_stride0, in_stride1, out_stride0, out_stride1});
    };
    switch (itemsize) {
    case 1: return launch_tile<uint8_t>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, s);
    case 2: if (fits(2)) return launch_tile<uint16_t>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, s); break;
    case 4: if (fits(4)) return launch_tile<uint32_t>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, s); break;
    case 8: if (fits(8)) return launch_tile<uint2>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, s); break;
    case 16: if (fits(16)) return launch_tile<uint4>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, s); break;
    default: break;
    }
    if (itemsize % 4 == 0 && fits(4))
        return launch_items<uint32_t>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, itemsize, s);
    return launch_items<uint8_t>(in_dev, out_dev, rows, cols, in_stride0, in_stride1, out_stride0, out_stride1, itemsize, s);
}
