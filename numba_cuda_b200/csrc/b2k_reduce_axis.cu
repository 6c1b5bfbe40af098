// Reduction of a matrix along one axis with a table op: out[j] = fold_i x[i, j]
// (axis 0) or out[i] = fold_j x[i, j] (axis 1), `init` folded into every output.
// The reference reduces 1-D arrays only (numba/cuda/kernels/reduction.py:217-218
// raises for anything else); this is the axis-wise step after it, with the same
// ops, dtypes and wrap-around rules as b2k_reduce.
//
// Rows are contiguous (column stride = item size) and `pitch` bytes apart.  Threads
// move packs of V items: 16 bytes when the base, the pitch and the row length are
// multiples of 16, else 8 or 4 bytes on the same condition, else single items.
//
//  * axis 0, reduce_cols_kernel: a thread owns one pack of columns and walks down
//    the rows; a CTA is `lx` column packs wide (32 for wide matrices, fewer for
//    narrow ones) and 256/lx row lanes tall, four row loads in flight per thread.
//    Row lanes combine through shared memory.  Rows are split into `chunks`
//    (gridDim.y) to fill the GPU: every CTA publishes its partial row, takes a
//    ticket per column tile (atomicInc that wraps to zero), and the CTA that draws
//    the last ticket folds the partial rows (row lanes stride over the chunks, then
//    the same tree).
//  * axis 1, reduce_rows_kernel: a group of G lanes (1..32, or the whole CTA) owns
//    one row, lanes striding over its packs with four loads in flight, then a
//    shuffle butterfly inside the group.  G grows with the row length, so short
//    rows are read coalesced by neighbouring lanes and long rows by whole CTAs.
//  * axis 1 with few, very long rows, reduce_rows_split_kernel: every row is cut
//    into `segments` CTAs with the same ticket scheme.
//
// The order of every fold depends only on the shape and the grid, so float
// results are reproducible.  HBM roofline: sizeof(T) bytes read per item.
#include <cstring>
#include <type_traits>

#include "b2k_internal.cuh"
#include "b2k_reduce_ops.cuh"

namespace {

using namespace b2k_reduce_ops;

constexpr int kThreads = 256;
constexpr int kUnroll = 4;
constexpr int kMaxChunks = 1024;
// Scratch layout: a fixed region of tickets first (always back at zero when a kernel
// ends), partials behind it.  The region is the same for every shape, so a buffer
// that served one shape can serve any other without being cleared again.
constexpr int64_t kMaxTickets = 4096;
constexpr int64_t kTicketRegion = kMaxTickets * 4;

// V items; packs of whole 32-bit words can also be addressed as words, which is how
// the loads fill them and how 8- and 16-bit items are folded (a plain array of small
// items would live in one register per item).
template <typename T, int V, bool WORDS = (V * sizeof(T)) % 4 == 0>
struct Pack {
    T e[V];
};
template <typename T, int V>
struct Pack<T, V, true> {
    union {
        T e[V];
        uint32_t w[V * sizeof(T) / 4];
    };
};

template <typename T, int V>
__device__ __forceinline__ Pack<T, V> load_pack(const unsigned char *p) {
    constexpr int BYTES = V * sizeof(T);
    Pack<T, V> r;
    if constexpr (BYTES % 4 != 0) {
        static_assert(V == 1, "a pack is one item or 4, 8 or 16 bytes");
        r.e[0] = *reinterpret_cast<const T *>(p);
    } else if constexpr (BYTES == 16) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3])
                     : "l"(p));
    } else if constexpr (BYTES == 8) {
        asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];" : "=r"(r.w[0]), "=r"(r.w[1]) : "l"(p));
    } else {
        static_assert(BYTES == 4, "a pack is one item or 4, 8 or 16 bytes");
        asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(r.w[0]) : "l"(p));
    }
    return r;
}

template <typename T, typename Op, int V>
__device__ __forceinline__ void fold_into(Pack<T, V> &acc, const Pack<T, V> &v) {
    if constexpr (WordWise<T, Op>::value && (V * sizeof(T)) % 4 == 0) {
#pragma unroll
        for (int k = 0; k < static_cast<int>(V * sizeof(T) / 4); ++k) acc.w[k] = apply_word<T, Op>(acc.w[k], v.w[k]);
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) acc.e[k] = Op::template apply<T>(acc.e[k], v.e[k]);
    }
}

template <typename T, typename Op, int V>
__device__ __forceinline__ Pack<T, V> identity_pack() {
    Pack<T, V> r;
#pragma unroll
    for (int k = 0; k < V; ++k) r.e[k] = Op::template identity<T>();
    return r;
}

template <typename T, typename Op, int V>
__device__ __forceinline__ T fold_pack(T acc, const Pack<T, V> &v) {
#pragma unroll
    for (int k = 0; k < V; ++k) acc = Op::template apply<T>(acc, v.e[k]);
    return acc;
}

// ---- axis 0 ----------------------------------------------------------------------
template <typename T, typename Op, int V>
__global__ void __launch_bounds__(kThreads)
reduce_cols_kernel(const unsigned char *__restrict__ x, int64_t rows, int64_t packs, int64_t pitch, int lx_log2,
                   int64_t rows_per_chunk, T init, Pack<T, V> *__restrict__ out, Pack<T, V> *__restrict__ partials,
                   unsigned int *__restrict__ tickets, int64_t slab_bytes) {
    __shared__ Pack<T, V> lanes[kThreads];
    __shared__ bool is_last;
    // blockIdx.z numbers the matrices of a batch: `slab_bytes` apart on the input side,
    // one output row, one block of partial rows and one run of tickets each
    x += static_cast<int64_t>(blockIdx.z) * slab_bytes;
    out += static_cast<int64_t>(blockIdx.z) * packs;
    partials += static_cast<int64_t>(blockIdx.z) * gridDim.y * packs;
    tickets += static_cast<int64_t>(blockIdx.z) * gridDim.x;
    const int lx = 1 << lx_log2;
    const int tx = threadIdx.x & (lx - 1), ty = threadIdx.x >> lx_log2, ny = kThreads >> lx_log2;
    const int64_t pack = static_cast<int64_t>(blockIdx.x) * lx + tx;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
    const int64_t r1 = (r0 + rows_per_chunk < rows) ? r0 + rows_per_chunk : rows;

    Pack<T, V> acc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) acc[u] = identity_pack<T, Op, V>();
    if (pack < packs) {
        const unsigned char *col = x + pack * static_cast<int64_t>(V * sizeof(T));
        int64_t r = r0 + ty;
        for (; r + (kUnroll - 1) * ny < r1; r += kUnroll * ny) {
            Pack<T, V> v[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) v[u] = load_pack<T, V>(col + (r + u * ny) * pitch);
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) fold_into<T, Op, V>(acc[u], v[u]);
        }
        for (; r < r1; r += ny) fold_into<T, Op, V>(acc[0], load_pack<T, V>(col + r * pitch));
    }
#pragma unroll
    for (int u = 1; u < kUnroll; ++u) fold_into<T, Op, V>(acc[0], acc[u]);

    lanes[threadIdx.x] = acc[0];
    __syncthreads();
    for (int s = ny >> 1; s >= 1; s >>= 1) {
        if (ty < s) {
            Pack<T, V> mine = lanes[threadIdx.x];
            fold_into<T, Op, V>(mine, lanes[threadIdx.x + s * lx]);
            lanes[threadIdx.x] = mine;
        }
        __syncthreads();
    }
    const bool owner = ty == 0 && pack < packs;
    const unsigned int chunks = gridDim.y;
    if (chunks == 1) {
        if (owner) {
            Pack<T, V> total = lanes[threadIdx.x];
#pragma unroll
            for (int k = 0; k < V; ++k) total.e[k] = Op::template apply<T>(total.e[k], init);
            out[pack] = total;
        }
        return;
    }
    if (owner) partials[static_cast<int64_t>(blockIdx.y) * packs + pack] = lanes[threadIdx.x];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicInc(&tickets[blockIdx.x], chunks - 1) == chunks - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // the last CTA folds the partial rows: row lanes take chunks ty, ty + ny, ..., then
    // the same shared-memory tree as above
    Pack<T, V> total = identity_pack<T, Op, V>();
    if (pack < packs) {
        for (unsigned int c = ty; c < chunks; c += ny) {
            const Pack<T, V> *src = partials + static_cast<int64_t>(c) * packs + pack;
            Pack<T, V> v;
#pragma unroll
            for (int k = 0; k < V; ++k) v.e[k] = __ldcg(&src->e[k]);
            fold_into<T, Op, V>(total, v);
        }
    }
    lanes[threadIdx.x] = total;
    __syncthreads();
    for (int s = ny >> 1; s >= 1; s >>= 1) {
        if (ty < s) {
            Pack<T, V> mine = lanes[threadIdx.x];
            fold_into<T, Op, V>(mine, lanes[threadIdx.x + s * lx]);
            lanes[threadIdx.x] = mine;
        }
        __syncthreads();
    }
    if (owner) {
        total = lanes[threadIdx.x];
#pragma unroll
        for (int k = 0; k < V; ++k) total.e[k] = Op::template apply<T>(total.e[k], init);
        out[pack] = total;
    }
}

// A second form of the same kernel, kept beside the first because neither wins everywhere
// (GB/s read, first form / this form with runs / this form with dealt blocks): float32
// 16384^2 6422 / 6104 / 6474, float64 8192x16384 6938 / 5058 / 6428, uint8 32768^2 6714 /
// 6122 / 4776 -- but one column tile (2^22 x 64 float32) 5379 / 6627 / 5549, few rows
// (64 x 2^22) 6751 / 7126 / 6770, rows of 8-byte packs (2^20 x 250 float32) 4496 / 5344 /
// 6627.  The launcher picks by shape.  With INTERLEAVE the rows go to the chunks in blocks
// of ny * kUnroll rows dealt round robin, so the CTAs that run at the same time sweep one
// window of consecutive rows; without it a chunk is one run of rows, as in the first form
// (same loop; the two differ in what the compiler makes of it).
template <typename T, typename Op, int V, bool INTERLEAVE>
__global__ void __launch_bounds__(kThreads)
reduce_cols_dealt_kernel(const unsigned char *__restrict__ x, int64_t rows, int64_t packs, int64_t pitch, int lx_log2,
                   int64_t rows_per_chunk, T init, Pack<T, V> *__restrict__ out, Pack<T, V> *__restrict__ partials,
                   unsigned int *__restrict__ tickets, int64_t slab_bytes) {
    __shared__ Pack<T, V> lanes[kThreads];
    __shared__ bool is_last;
    // blockIdx.z numbers the matrices of a batch: `slab_bytes` apart on the input side,
    // one output row, one block of partial rows and one run of tickets each
    x += static_cast<int64_t>(blockIdx.z) * slab_bytes;
    out += static_cast<int64_t>(blockIdx.z) * packs;
    partials += static_cast<int64_t>(blockIdx.z) * gridDim.y * packs;
    tickets += static_cast<int64_t>(blockIdx.z) * gridDim.x;
    const int lx = 1 << lx_log2;
    const int tx = threadIdx.x & (lx - 1), ty = threadIdx.x >> lx_log2, ny = kThreads >> lx_log2;
    const int64_t pack = static_cast<int64_t>(blockIdx.x) * lx + tx;
    Pack<T, V> acc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) acc[u] = identity_pack<T, Op, V>();
    if (pack < packs) {
        const unsigned char *col = x + pack * static_cast<int64_t>(V * sizeof(T));
        if constexpr (INTERLEAVE) {
            const int64_t block_rows = static_cast<int64_t>(ny) * kUnroll;
            for (int64_t base = static_cast<int64_t>(blockIdx.y) * block_rows; base < rows;
                 base += static_cast<int64_t>(gridDim.y) * block_rows) {
                const int64_t r = base + ty;
                if (base + block_rows <= rows) {
                    Pack<T, V> v[kUnroll];
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) v[u] = load_pack<T, V>(col + (r + u * ny) * pitch);
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) fold_into<T, Op, V>(acc[u], v[u]);
                } else {
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u)
                        if (r + u * ny < rows) fold_into<T, Op, V>(acc[u], load_pack<T, V>(col + (r + u * ny) * pitch));
                }
            }
        } else {
            const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
            const int64_t r1 = (r0 + rows_per_chunk < rows) ? r0 + rows_per_chunk : rows;
            int64_t r = r0 + ty;
            for (; r + (kUnroll - 1) * ny < r1; r += kUnroll * ny) {
                Pack<T, V> v[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) v[u] = load_pack<T, V>(col + (r + u * ny) * pitch);
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) fold_into<T, Op, V>(acc[u], v[u]);
            }
            for (; r < r1; r += ny) fold_into<T, Op, V>(acc[0], load_pack<T, V>(col + r * pitch));
        }
    }
#pragma unroll
    for (int u = 1; u < kUnroll; ++u) fold_into<T, Op, V>(acc[0], acc[u]);

    lanes[threadIdx.x] = acc[0];
    __syncthreads();
    for (int s = ny >> 1; s >= 1; s >>= 1) {
        if (ty < s) {
            Pack<T, V> mine = lanes[threadIdx.x];
            fold_into<T, Op, V>(mine, lanes[threadIdx.x + s * lx]);
            lanes[threadIdx.x] = mine;
        }
        __syncthreads();
    }
    const bool owner = ty == 0 && pack < packs;
    const unsigned int chunks = gridDim.y;
    if (chunks == 1) {
        if (owner) {
            Pack<T, V> total = lanes[threadIdx.x];
#pragma unroll
            for (int k = 0; k < V; ++k) total.e[k] = Op::template apply<T>(total.e[k], init);
            out[pack] = total;
        }
        return;
    }
    if (owner) partials[static_cast<int64_t>(blockIdx.y) * packs + pack] = lanes[threadIdx.x];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicInc(&tickets[blockIdx.x], chunks - 1) == chunks - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // the last CTA folds the partial rows: row lanes take chunks ty, ty + ny, ..., then
    // the same shared-memory tree as above
    Pack<T, V> total = identity_pack<T, Op, V>();
    if (pack < packs) {
        for (unsigned int c = ty; c < chunks; c += ny) {
            const Pack<T, V> *src = partials + static_cast<int64_t>(c) * packs + pack;
            Pack<T, V> v;
#pragma unroll
            for (int k = 0; k < V; ++k) v.e[k] = __ldcg(&src->e[k]);
            fold_into<T, Op, V>(total, v);
        }
    }
    lanes[threadIdx.x] = total;
    __syncthreads();
    for (int s = ny >> 1; s >= 1; s >>= 1) {
        if (ty < s) {
            Pack<T, V> mine = lanes[threadIdx.x];
            fold_into<T, Op, V>(mine, lanes[threadIdx.x + s * lx]);
            lanes[threadIdx.x] = mine;
        }
        __syncthreads();
    }
    if (owner) {
        total = lanes[threadIdx.x];
#pragma unroll
        for (int k = 0; k < V; ++k) total.e[k] = Op::template apply<T>(total.e[k], init);
        out[pack] = total;
    }
}

// ---- axis 1 ----------------------------------------------------------------------
// Fold of packs [first, last) of one row by `width` cooperating lanes.
template <typename T, typename Op, int V>
__device__ __forceinline__ T fold_row_part(const unsigned char *row, int64_t first, int64_t last, int lane,
                                           int width) {
    T acc[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) acc[u] = Op::template identity<T>();
    int64_t k = first + lane;
    for (; k + static_cast<int64_t>(kUnroll - 1) * width < last; k += static_cast<int64_t>(kUnroll) * width) {
        Pack<T, V> v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            v[u] = load_pack<T, V>(row + (k + static_cast<int64_t>(u) * width) * static_cast<int64_t>(V * sizeof(T)));
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) acc[u] = fold_pack<T, Op, V>(acc[u], v[u]);
    }
    for (; k < last; k += width)
        acc[0] = fold_pack<T, Op, V>(acc[0], load_pack<T, V>(row + k * static_cast<int64_t>(V * sizeof(T))));
#pragma unroll
    for (int u = 1; u < kUnroll; ++u) acc[0] = Op::template apply<T>(acc[0], acc[u]);
    return acc[0];
}

// Block-wide fold; the result is valid in thread 0.
template <typename T, typename Op>
__device__ __forceinline__ T block_fold(T v, T *slots) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = Op::template apply<T>(v, shuffle_xor(v, m));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) slots[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = (lane < kThreads / 32) ? slots[lane] : Op::template identity<T>();
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) v = Op::template apply<T>(v, shuffle_xor(v, m));
    }
    __syncthreads();
    return v;
}

template <typename T, typename Op, int V>
__global__ void __launch_bounds__(kThreads)
reduce_rows_kernel(const unsigned char *__restrict__ x, int64_t rows, int64_t packs, int64_t pitch, int group_log2,
                   T init, T *__restrict__ out) {
    __shared__ T slots[kThreads / 32];
    const int width = 1 << group_log2;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads >> group_log2) + (threadIdx.x >> group_log2);
    const int lane = threadIdx.x & (width - 1);
    T acc = Op::template identity<T>();
    if (row < rows) acc = fold_row_part<T, Op, V>(x + row * pitch, 0, packs, lane, width);
    if (width == kThreads) {
        acc = block_fold<T, Op>(acc, slots);
    } else {
        // groups are aligned inside a warp: butterfly over the group's lanes only
        for (int m = (width < 32 ? width : 32) >> 1; m > 0; m >>= 1)
            acc = Op::template apply<T>(acc, shuffle_xor(acc, m));
    }
    if (lane == 0 && row < rows) out[row] = Op::template apply<T>(acc, init);
}

template <typename T, typename Op, int V>
__global__ void __launch_bounds__(kThreads)
reduce_rows_split_kernel(const unsigned char *__restrict__ x, int64_t packs, int64_t pitch, int64_t packs_per_segment,
                         T init, T *__restrict__ out, T *__restrict__ partials, unsigned int *__restrict__ tickets) {
    __shared__ T slots[kThreads / 32];
    __shared__ bool is_last;
    const int64_t row = blockIdx.y;
    const unsigned int segments = gridDim.x;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * packs_per_segment;
    const int64_t last = (first + packs_per_segment < packs) ? first + packs_per_segment : packs;
    T acc = fold_row_part<T, Op, V>(x + row * pitch, first, last, threadIdx.x, kThreads);
    acc = block_fold<T, Op>(acc, slots);
    if (threadIdx.x == 0) {
        partials[row * segments + blockIdx.x] = acc;
        __threadfence();
        is_last = atomicInc(&tickets[row], segments - 1) == segments - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x == 0) {
        T total = Op::template identity<T>();
        for (unsigned int s = 0; s < segments; ++s) total = Op::template apply<T>(total, __ldcg(partials + row * segments + s));
        out[row] = Op::template apply<T>(total, init);
    }
}

// ---- host ------------------------------------------------------------------------
struct Plan {
    int64_t pack_bytes;   // bytes moved per load: 16, 8, 4 or one item
    int64_t packs;        // packs per row
    // axis 0
    int lx_log2;
    int64_t tiles, chunks, rows_per_chunk;
    // axis 1
    int group_log2;
    bool split;
    int64_t segments, packs_per_segment;
    // scratch layout: tickets first, partials after `ticket_bytes`
    int64_t ticket_bytes, scratch_bytes;
};

int log2_ceil(int64_t v) {
    int l = 0;
    while ((int64_t(1) << l) < v) ++l;
    return l;
}

Plan make_plan(int64_t rows, int64_t cols, int64_t item, int axis, int64_t alignment, int64_t batch = 1) {
    Plan p{};
    // widest pack that the layout's alignment and the row length allow
    p.pack_bytes = item;
    for (int64_t bytes = 16; bytes > item && bytes >= 4; bytes /= 2) {
        if (alignment % bytes == 0 && (cols * item) % bytes == 0) {
            p.pack_bytes = bytes;
            break;
        }
    }
    p.packs = cols * item / p.pack_bytes;
    const int64_t sms = b2k::sm_count();
    if (axis == 0) {
        // CTA width in packs: 32 (512-byte row segments, eight row lanes) measured best for
        // tall matrices of 4- and 8-byte items; single bytes gain 17 % from 64 (their packs
        // carry 16 items of work each), and matrices of few rows from a whole CTA's width
        // (one row lane walks all rows: 64 x 2^22 float32 6015 -> 6748 GB/s)
        const int wide = rows <= 256 ? 8 : (item == 1 ? 6 : 5);
        p.lx_log2 = p.packs >= (int64_t(1) << wide) ? wide : log2_ceil(p.packs < 1 ? 1 : p.packs);
        const int64_t lx = int64_t(1) << p.lx_log2, ny = kThreads / lx;
        p.tiles = (p.packs + lx - 1) / lx;
        const int64_t columns_of_ctas = p.tiles * batch;
        int64_t chunks = (sms * 8 + columns_of_ctas - 1) / columns_of_ctas;
        const int64_t most = rows / (ny * kUnroll);  // every chunk gets at least one unrolled pass
        if (chunks > most) chunks = most;
        if (chunks > kMaxChunks) chunks = kMaxChunks;
        if (chunks < 1 || columns_of_ctas > kMaxTickets) chunks = 1;
        p.rows_per_chunk = (rows + chunks - 1) / chunks;
        p.chunks = (rows + p.rows_per_chunk - 1) / (p.rows_per_chunk < 1 ? 1 : p.rows_per_chunk);
        if (p.chunks < 1) p.chunks = 1;
        p.ticket_bytes = p.chunks > 1 ? kTicketRegion : 0;
        p.scratch_bytes = p.ticket_bytes + (p.chunks > 1 ? batch * p.chunks * p.packs * p.pack_bytes : 0);
    } else {
        // lanes per row: about 64 bytes per lane, a whole CTA for long rows
        const int64_t want = (p.packs * p.pack_bytes + 63) / 64;
        p.group_log2 = want >= 64 ? 8 : (want > 32 ? 5 : log2_ceil(want < 1 ? 1 : want));
        p.split = p.group_log2 == 8 && rows < 2 * sms && rows <= kMaxTickets && p.packs >= 16 * kThreads * kUnroll;
        if (p.split) {
            int64_t segments = (4 * sms + rows - 1) / rows;
            const int64_t most = p.packs / (kThreads * kUnroll * 2);
            if (segments > most) segments = most;
            if (segments > 64) segments = 64;  // folded by one thread per row
            if (segments < 2) {
                p.split = false;
            } else {
                p.packs_per_segment = (p.packs + segments - 1) / segments;
                p.segments = (p.packs + p.packs_per_segment - 1) / p.packs_per_segment;
                p.ticket_bytes = kTicketRegion;
                p.scratch_bytes = p.ticket_bytes + rows * p.segments * item;
            }
        }
    }
    return p;
}

template <typename T, typename Op, int V>
int launch_planned(const Plan &p, const void *x, int64_t rows, int64_t pitch, int axis, T init, void *out,
                   void *scratch, cudaStream_t stream, int64_t batch, int64_t slab_bytes) {
    const unsigned char *src = static_cast<const unsigned char *>(x);
    unsigned char *sc = static_cast<unsigned char *>(scratch);
    if (axis == 0) {
        if (p.tiles > 0x7FFFFFFFll) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_reduce_axis: too many columns");
        const dim3 grid(static_cast<unsigned>(p.tiles), static_cast<unsigned>(p.chunks), static_cast<unsigned>(batch));
        // which form: see the note above reduce_cols_dealt_kernel
        const int form = B2K_ENV_INT("B2K_AXIS0_FORM", -1);
        const int pick = form >= 0 ? form : (p.pack_bytes < 16 && p.pack_bytes > static_cast<int64_t>(sizeof(T))) ? 2
                                            : (p.tiles == 1 || rows <= 256) ? 1 : 0;
        auto kernel = pick == 2 ? reduce_cols_dealt_kernel<T, Op, V, true>
                      : pick == 1 ? reduce_cols_dealt_kernel<T, Op, V, false> : reduce_cols_kernel<T, Op, V>;
        kernel<<<grid, kThreads, 0, stream>>>(
            src, rows, p.packs, pitch, p.lx_log2, p.rows_per_chunk, init, static_cast<Pack<T, V> *>(out),
            reinterpret_cast<Pack<T, V> *>(sc + p.ticket_bytes), reinterpret_cast<unsigned int *>(sc), slab_bytes);
    } else if (p.split) {
        const dim3 grid(static_cast<unsigned>(p.segments), static_cast<unsigned>(rows));
        reduce_rows_split_kernel<T, Op, V><<<grid, kThreads, 0, stream>>>(
            src, p.packs, pitch, p.packs_per_segment, init, static_cast<T *>(out),
            reinterpret_cast<T *>(sc + p.ticket_bytes), reinterpret_cast<unsigned int *>(sc));
    } else {
        const int64_t per_cta = kThreads >> p.group_log2;
        const int64_t grid = (rows + per_cta - 1) / per_cta;
        if (grid > 0x7FFFFFFFll) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_reduce_axis: too many rows");
        reduce_rows_kernel<T, Op, V><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            src, rows, p.packs, pitch, p.group_log2, init, static_cast<T *>(out));
    }
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_reduce_axis launch");
    return B2K_OK;
}

template <typename T, typename Op>
int launch_typed(const Plan &p, const void *x, int64_t rows, int64_t pitch, int axis, const void *init_host,
                 void *out, void *scratch, cudaStream_t stream, int64_t batch, int64_t slab_bytes) {
    T init;
    memcpy(&init, init_host, sizeof(T));
    constexpr int SIZE = sizeof(T);
    if constexpr (SIZE < 16) {
        if (p.pack_bytes == 16) return launch_planned<T, Op, 16 / SIZE>(p, x, rows, pitch, axis, init, out, scratch, stream, batch, slab_bytes);
    }
    if constexpr (SIZE < 8) {
        if (p.pack_bytes == 8) return launch_planned<T, Op, (8 / SIZE > 0 ? 8 / SIZE : 1)>(p, x, rows, pitch, axis, init, out, scratch, stream, batch, slab_bytes);
    }
    if constexpr (SIZE < 4) {
        if (p.pack_bytes == 4) return launch_planned<T, Op, (4 / SIZE > 0 ? 4 / SIZE : 1)>(p, x, rows, pitch, axis, init, out, scratch, stream, batch, slab_bytes);
    }
    return launch_planned<T, Op, 1>(p, x, rows, pitch, axis, init, out, scratch, stream, batch, slab_bytes);
}

// Integer +, *, &, |, ^ wrap identically for both signs, so signed types run those
// ops in the unsigned type of their width; only max and min need the sign.
template <typename S, typename U>
int dispatch_integer(int op, bool is_signed, const Plan &p, const void *x, int64_t rows, int64_t pitch, int axis,
                     const void *init_host, void *out, void *scratch, cudaStream_t stream, int64_t batch,
                     int64_t slab_bytes) {
    switch (op) {
    case B2K_ADD: return launch_typed<U, OpAdd>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_MUL: return launch_typed<U, OpMul>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_AND: return launch_typed<U, OpAnd>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_OR: return launch_typed<U, OpOr>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_XOR: return launch_typed<U, OpXor>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_MAX:
        return is_signed ? launch_typed<S, OpMax>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes)
                         : launch_typed<U, OpMax>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_MIN:
        return is_signed ? launch_typed<S, OpMin>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes)
                         : launch_typed<U, OpMin>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    default: return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_axis: unknown op %d", op);
    }
}

template <typename F>
int dispatch_float(int op, const Plan &p, const void *x, int64_t rows, int64_t pitch, int axis,
                   const void *init_host, void *out, void *scratch, cudaStream_t stream, int64_t batch,
                     int64_t slab_bytes) {
    switch (op) {
    case B2K_ADD: return launch_typed<F, OpAdd>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_MUL: return launch_typed<F, OpMul>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_MAX: return launch_typed<F, OpMax>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    case B2K_MIN: return launch_typed<F, OpMin>(p, x, rows, pitch, axis, init_host, out, scratch, stream, batch, slab_bytes);
    default: return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_axis: bitwise op on a floating-point type");
    }
}

int64_t item_size(int dtype) {
    switch (dtype) {
    case B2K_I8: case B2K_U8: return 1;
    case B2K_I16: case B2K_U16: return 2;
    case B2K_I32: case B2K_U32: case B2K_F32: return 4;
    case B2K_I64: case B2K_U64: case B2K_F64: return 8;
    default: return 0;
    }
}

// Largest power of two (up to 16) that divides the input base, the pitch and the
// output base.
int64_t layout_alignment(const void *x, int64_t pitch, const void *out) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | static_cast<uintptr_t>(pitch) |
                           reinterpret_cast<uintptr_t>(out) | 16u;
    return static_cast<int64_t>(bits & (~bits + 1));
}

}  // namespace

extern "C" {

int64_t b2k_reduce_axis_scratch_bytes(int64_t rows, int64_t cols, int dtype, int axis) {
    const int64_t item = item_size(dtype);
    if (rows <= 0 || cols <= 0 || item == 0 || (axis != 0 && axis != 1)) return 0;
    // the largest over the pack widths, so that one buffer serves any alignment
    int64_t most = 0;
    for (int64_t alignment = 16; alignment >= 1; alignment /= 2) {
        const Plan p = make_plan(rows, cols, item, axis, alignment);
        if (p.scratch_bytes > most) most = p.scratch_bytes;
    }
    return most;
}

static int reduce_axis_impl(const char *who, int op, int dtype, const void *x_dev, int64_t batch, int64_t rows,
                            int64_t cols, int64_t pitch_bytes, int64_t slab_bytes, int axis, const void *init_host,
                            void *out_dev, void *scratch_dev, int64_t scratch_bytes, void *stream) {
    const int64_t item = item_size(dtype);
    if (item == 0) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: unknown dtype %d", who, dtype);
    if (axis != 0 && axis != 1) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: axis must be 0 or 1", who);
    if (rows < 0 || cols < 0 || batch < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: negative shape", who);
    if (batch > 65535) return b2k::fail(B2K_ERR_TOO_LARGE, "%s: at most 65535 matrices per call", who);
    if (!init_host) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: null init", who);
    const int64_t outputs = (axis == 0 ? cols : rows) * batch;
    if (outputs == 0) return B2K_OK;
    if (!out_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: null output", who);
    if (reinterpret_cast<uintptr_t>(out_dev) % item)
        return b2k::fail(B2K_ERR_ALIGNMENT, "%s: output not aligned to its item size", who);
    const int64_t reduced = axis == 0 ? rows : cols;
    if (reduced > 0) {
        if (!x_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: null input", who);
        if (reinterpret_cast<uintptr_t>(x_dev) % item || pitch_bytes % item || slab_bytes % item)
            return b2k::fail(B2K_ERR_ALIGNMENT, "%s: input, pitch or matrix stride not aligned to the item size", who);
        if (pitch_bytes < cols * item) return b2k::fail(B2K_ERR_INVALID_ARG, "%s: pitch shorter than a row", who);
    }
    // an empty reduced axis leaves `init` in every output: same kernels, zero rows / packs
    const int64_t alignment = layout_alignment(x_dev, pitch_bytes | (batch > 1 ? slab_bytes : 0), out_dev);
    const Plan p = make_plan(rows, cols, item, axis, alignment, batch);
    if (p.scratch_bytes > 0) {
        if (!scratch_dev || scratch_bytes < p.scratch_bytes || reinterpret_cast<uintptr_t>(scratch_dev) % 256)
            return b2k::fail(B2K_ERR_SCRATCH, "%s: scratch of %lld bytes (256-byte aligned, zeroed once) needed", who,
                             static_cast<long long>(p.scratch_bytes));
    }
    cudaStream_t s = b2k::as_stream(stream);
    const int64_t pitch = pitch_bytes;
    switch (dtype) {
    case B2K_I8: return dispatch_integer<int8_t, uint8_t>(op, true, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_U8: return dispatch_integer<int8_t, uint8_t>(op, false, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_I16: return dispatch_integer<int16_t, uint16_t>(op, true, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_U16: return dispatch_integer<int16_t, uint16_t>(op, false, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_I32: return dispatch_integer<int32_t, uint32_t>(op, true, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_U32: return dispatch_integer<int32_t, uint32_t>(op, false, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_I64: return dispatch_integer<int64_t, uint64_t>(op, true, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_U64: return dispatch_integer<int64_t, uint64_t>(op, false, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    case B2K_F32: return dispatch_float<float>(op, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    default: return dispatch_float<double>(op, p, x_dev, rows, pitch, axis, init_host, out_dev, scratch_dev, s, batch, slab_bytes);
    }
}

int b2k_reduce_axis(int op, int dtype, const void *x_dev, int64_t rows, int64_t cols, int64_t pitch_bytes, int axis,
                    const void *init_host, void *out_dev, void *scratch_dev, int64_t scratch_bytes, void *stream) {
    B2K_RANGE("b2k_reduce_axis");
    return reduce_axis_impl("b2k_reduce_axis", op, dtype, x_dev, 1, rows, cols, pitch_bytes, 0, axis, init_host,
                            out_dev, scratch_dev, scratch_bytes, stream);
}

int64_t b2k_reduce_cols_batched_scratch_bytes(int64_t batch, int64_t rows, int64_t cols, int dtype) {
    const int64_t item = item_size(dtype);
    if (batch <= 0 || rows <= 0 || cols <= 0 || item == 0) return 0;
    int64_t most = 0;
    for (int64_t alignment = 16; alignment >= 1; alignment /= 2) {
        const Plan p = make_plan(rows, cols, item, 0, alignment, batch);
        if (p.scratch_bytes > most) most = p.scratch_bytes;
    }
    return most;
}

int b2k_reduce_cols_batched(int op, int dtype, const void *x_dev, int64_t batch, int64_t rows, int64_t cols,
                            int64_t pitch_bytes, int64_t matrix_stride_bytes, const void *init_host, void *out_dev,
                            void *scratch_dev, int64_t scratch_bytes, void *stream) {
    B2K_RANGE("b2k_reduce_cols_batched");
    if (batch > 1 && matrix_stride_bytes < 0)
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_cols_batched: negative matrix stride");
    return reduce_axis_impl("b2k_reduce_cols_batched", op, dtype, x_dev, batch, rows, cols, pitch_bytes,
                            matrix_stride_bytes, 0, init_host, out_dev, scratch_dev, scratch_bytes, stream);
}

}  // extern "C"
