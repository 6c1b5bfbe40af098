// N-D strided assignment with broadcasting: dst[idx] = src[idx'] for every index of
// a common shape, where both sides are described by byte strides and a source
// stride of 0 repeats the source along that axis.  This is the device side of
// DeviceNDArray.__setitem__ (numba/cuda/cudadrv/devicearray.py:535-576, 735-791)
// and of N-D axis permutations.
//
// The host first rewrites the problem: axes of length 1 disappear, the item is
// split off as an innermost axis of bytes, axes are ordered by falling destination
// stride (assignment has no order of its own, so the axis that is densest in the
// destination becomes the fastest one), neighbouring axes that are contiguous on
// both sides are merged, and the innermost axis is regrouped into the widest unit
// (16, 8, 4, 2 or 1 bytes) that every pointer and stride allows.  Kernels:
//
//  * direct: one thread per unit, four units in flight per thread, consecutive
//    threads on consecutive units of the fastest destination axis.  Reads are
//    coalesced too whenever the source is dense along the same axis (slices,
//    row / scalar broadcasts, plain copies);
//  * fill: the source repeats along the fastest destination axis (scalar and
//    per-row fills): the unit is replicated into 16-byte stores;
//  * repeat: the source repeats along a slower axis (one row assigned to every
//    row): each thread reads its unit once and stores it to 16 rows;
//  * runs: dense runs whose two sides are aligned differently (a slice shifted by
//    one item, rows of an odd pitch) move as aligned 16-byte destination chunks
//    fed from the two covering source words, shifted in registers;
//  * tiled: when the source is dense along a DIFFERENT axis q than the destination
//    (axis permutations), tiles over (destination axis p, source axis q) go
//    through shared memory so that both sides see coalesced accesses;
//  * byte tiles: the same for single bytes, with 32-bit global accesses on rows of
//    any alignment (covering words, funnel shifts, 4 x 4 byte blocks in registers);
//  * the TMA tile transpose of b2k_transpose_tma.cu, as a stack of 2-D problems,
//    when such a permutation also meets the tensor-map alignment rules.
//
// b2k_fill is the same machinery for one source item handed over by value.
#include <algorithm>
#include <cstring>

#include "b2k_internal.cuh"

namespace {

constexpr int kMaxAxes = 8;

struct Axes {
    int n;                        // axes in use, the last one is the fastest
    int64_t len[kMaxAxes];        // in units
    int64_t dst_step[kMaxAxes];   // bytes
    int64_t src_step[kMaxAxes];   // bytes, 0 = broadcast
    // b2k_fill: the one source item travels in the kernel parameters; kernels that
    // are handed a null source read from here instead
    alignas(16) unsigned char value[16];
};

template <typename Index>
__device__ __forceinline__ void locate(const Axes &ax, Index linear, int64_t &doff, int64_t &soff) {
    doff = 0;
    soff = 0;
#pragma unroll
    for (int k = kMaxAxes - 1; k >= 0; --k) {
        if (k < ax.n) {
            const Index len = static_cast<Index>(ax.len[k]);
            const Index q = linear / len;
            const Index i = linear - q * len;
            linear = q;
            doff += static_cast<int64_t>(i) * ax.dst_step[k];
            soff += static_cast<int64_t>(i) * ax.src_step[k];
        }
    }
}

constexpr int kDirectThreads = 256;
constexpr int kDirectUnroll = 4;

template <typename U, typename Index>
__global__ void __launch_bounds__(kDirectThreads)
assign_direct_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                     const __grid_constant__ Axes ax, uint64_t total) {
    if (src == nullptr) src = ax.value;
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * (kDirectThreads * kDirectUnroll) + threadIdx.x;
    U value[kDirectUnroll];
    int64_t doff[kDirectUnroll];
#pragma unroll
    for (int j = 0; j < kDirectUnroll; ++j) {
        const uint64_t g = base + static_cast<uint64_t>(j) * kDirectThreads;
        if (g < total) {
            int64_t soff;
            locate<Index>(ax, static_cast<Index>(g), doff[j], soff);
            value[j] = *reinterpret_cast<const U *>(src + soff);
        }
    }
#pragma unroll
    for (int j = 0; j < kDirectUnroll; ++j) {
        const uint64_t g = base + static_cast<uint64_t>(j) * kDirectThreads;
        if (g < total) *reinterpret_cast<U *>(dst + doff[j]) = value[j];
    }
}

// The source repeats along the fastest destination axis (row fills, scalar fills):
// a thread reads one source unit S and stores it replicated into a 16-byte unit.
template <typename S, typename Index>
__global__ void __launch_bounds__(kDirectThreads)
assign_fill_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                   const __grid_constant__ Axes ax, uint64_t total) {
    if (src == nullptr) src = ax.value;
    constexpr int REP = 16 / sizeof(S);
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * (kDirectThreads * kDirectUnroll) + threadIdx.x;
#pragma unroll
    for (int j = 0; j < kDirectUnroll; ++j) {
        const uint64_t g = base + static_cast<uint64_t>(j) * kDirectThreads;
        if (g < total) {
            int64_t doff, soff;
            locate<Index>(ax, static_cast<Index>(g), doff, soff);
            union {
                uint4 wide;
                S part[REP];
            } v;
            const S one = *reinterpret_cast<const S *>(src + soff);
#pragma unroll
            for (int k = 0; k < REP; ++k) v.part[k] = one;
            *reinterpret_cast<uint4 *>(dst + doff) = v.wide;
        }
    }
}

// The source repeats along an axis that is not the fastest one (a row assigned to
// every row of a matrix): a thread reads its unit once and stores it to `per_thread`
// consecutive positions of the repeated axis.  `ax` holds the other axes, with the
// repeated axis replaced by its chunks (axis 0, the slowest).
constexpr int kRepeatRows = 16;

template <typename U, typename Index>
__global__ void __launch_bounds__(kDirectThreads)
assign_repeat_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                     const __grid_constant__ Axes ax, uint64_t total, uint64_t units_per_chunk, int64_t repeat_step,
                     int64_t repeat_len) {
    if (src == nullptr) src = ax.value;
    const uint64_t g = static_cast<uint64_t>(blockIdx.x) * kDirectThreads + threadIdx.x;
    if (g >= total) return;
    int64_t doff, soff;
    locate<Index>(ax, static_cast<Index>(g), doff, soff);
    const int64_t chunk = static_cast<int64_t>(static_cast<Index>(g) / static_cast<Index>(units_per_chunk));
    int64_t count = repeat_len - chunk * kRepeatRows;
    if (count > kRepeatRows) count = kRepeatRows;
    const U value = *reinterpret_cast<const U *>(src + soff);
    unsigned char *to = dst + doff;
    if (count == kRepeatRows) {
#pragma unroll
        for (int r = 0; r < kRepeatRows; ++r) *reinterpret_cast<U *>(to + r * repeat_step) = value;
    } else {
        for (int64_t r = 0; r < count; ++r) *reinterpret_cast<U *>(to + r * repeat_step) = value;
    }
}

// Tiles over (axis p = ax.n-1, the fastest in the destination; axis q, the densest
// in the source): TQ units along q by TP units along p.  Blocks enumerate (other
// axes..., q tiles, p tiles).  Throughput follows the bytes a thread has in flight
// between the two barriers, so 1- and 2-byte units get 128x64 tiles (32 loads per
// thread).
constexpr int kTiledThreads = 256;

template <typename U>
struct TileShape {
    static constexpr int TQ = sizeof(U) <= 2 ? 128 : (sizeof(U) == 4 ? 64 : 32);
    static constexpr int TP = sizeof(U) <= 4 ? 64 : 32;
    // row pitch in units: one bank (4 bytes) more than the row for units up to 4
    // bytes, one unit more for wider ones, so column reads spread over the banks
    static constexpr int PITCH = TQ + (sizeof(U) <= 4 ? 4 / sizeof(U) : 1);
};

template <typename U, typename Index>
__global__ void __launch_bounds__(kTiledThreads)
assign_tiled_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                    const __grid_constant__ Axes ax, int q, int64_t tiles_p, int64_t tiles_q) {
    constexpr int TQ = TileShape<U>::TQ, TP = TileShape<U>::TP, PITCH = TileShape<U>::PITCH;
    __shared__ U cell[TP * PITCH];
    const int p = ax.n - 1;
    // block -> (rest, tq, tp)
    uint64_t b = blockIdx.x;
    const int64_t tp = static_cast<int64_t>(b % static_cast<uint64_t>(tiles_p));
    b /= static_cast<uint64_t>(tiles_p);
    const int64_t tq = static_cast<int64_t>(b % static_cast<uint64_t>(tiles_q));
    Index rest = static_cast<Index>(b / static_cast<uint64_t>(tiles_q));
    int64_t dbase = 0, sbase = 0;
#pragma unroll
    for (int k = kMaxAxes - 1; k >= 0; --k) {
        if (k < ax.n && k != p && k != q) {
            const Index len = static_cast<Index>(ax.len[k]);
            const Index quo = rest / len;
            const Index i = rest - quo * len;
            rest = quo;
            dbase += static_cast<int64_t>(i) * ax.dst_step[k];
            sbase += static_cast<int64_t>(i) * ax.src_step[k];
        }
    }
    const int64_t p0 = tp * TP, q0 = tq * TQ;
    const int64_t np = ax.len[p] - p0, nq = ax.len[q] - q0;  // extent left along each tile axis
    // load: lanes along q (dense in the source), rows along p
    {
        constexpr int ROWS = kTiledThreads / TQ, PASSES = TP / ROWS;
        const int tx = threadIdx.x % TQ, ty = threadIdx.x / TQ;
        const unsigned char *from = src + sbase + p0 * ax.src_step[p] + (q0 + tx) * ax.src_step[q];
        const int64_t row_step = ax.src_step[p];
        U held[PASSES];
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const int row = ty + j * ROWS;
            if (tx < nq && row < np) held[j] = *reinterpret_cast<const U *>(from + row * row_step);
        }
        // all loads are issued before the first shared-memory store waits for one
        asm volatile("" ::: "memory");
#pragma unroll
        for (int j = 0; j < PASSES; ++j) cell[(ty + j * ROWS) * PITCH + tx] = held[j];
    }
    __syncthreads();
    // store: lanes along p (dense in the destination), rows along q
    {
        constexpr int ROWS = kTiledThreads / TP, PASSES = TQ / ROWS;
        const int tx = threadIdx.x % TP, ty = threadIdx.x / TP;
        unsigned char *to = dst + dbase + (p0 + tx) * ax.dst_step[p] + q0 * ax.dst_step[q];
        const int64_t row_step = ax.dst_step[q];
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const int row = ty + j * ROWS;
            if (tx < np && row < nq) *reinterpret_cast<U *>(to + row * row_step) = cell[tx * PITCH + row];
        }
    }
}

// Square tiles of TILE x TILE units for units of 4 bytes and more (the rectangular
// form above, instantiated at 64x64, compiled to a slower kernel for them).
template <typename U, typename Index, int TILE>
__global__ void __launch_bounds__(kTiledThreads)
assign_tiled_square_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                    const __grid_constant__ Axes ax, int q, int64_t tiles_p, int64_t tiles_q) {
    // a row pitch of TILE + 1 units keeps the column reads of 4-byte units conflict-free
    __shared__ U cell[TILE][TILE + 1];
    constexpr int ROWS = kTiledThreads / TILE;  // tile rows covered per pass
    constexpr int PASSES = TILE / ROWS;
    const int p = ax.n - 1;
    // block -> (rest, tq, tp)
    uint64_t b = blockIdx.x;
    const int64_t tp = static_cast<int64_t>(b % static_cast<uint64_t>(tiles_p));
    b /= static_cast<uint64_t>(tiles_p);
    const int64_t tq = static_cast<int64_t>(b % static_cast<uint64_t>(tiles_q));
    Index rest = static_cast<Index>(b / static_cast<uint64_t>(tiles_q));
    int64_t dbase = 0, sbase = 0;
#pragma unroll
    for (int k = kMaxAxes - 1; k >= 0; --k) {
        if (k < ax.n && k != p && k != q) {
            const Index len = static_cast<Index>(ax.len[k]);
            const Index quo = rest / len;
            const Index i = rest - quo * len;
            rest = quo;
            dbase += static_cast<int64_t>(i) * ax.dst_step[k];
            sbase += static_cast<int64_t>(i) * ax.src_step[k];
        }
    }
    const int64_t p0 = tp * TILE, q0 = tq * TILE;
    const int64_t np = ax.len[p] - p0, nq = ax.len[q] - q0;  // extent left along each tile axis
    const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    // load: lanes along q (dense in the source), rows along p
    {
        const unsigned char *from = src + sbase + p0 * ax.src_step[p] + (q0 + tx) * ax.src_step[q];
        const int64_t row_step = ax.src_step[p];
        U held[PASSES];
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const int row = ty + j * ROWS;
            if (tx < nq && row < np) held[j] = *reinterpret_cast<const U *>(from + row * row_step);
        }
#pragma unroll
        for (int j = 0; j < PASSES; ++j) cell[ty + j * ROWS][tx] = held[j];
    }
    __syncthreads();
    // store: lanes along p (dense in the destination), rows along q
    {
        unsigned char *to = dst + dbase + (p0 + tx) * ax.dst_step[p] + q0 * ax.dst_step[q];
        const int64_t row_step = ax.dst_step[q];
#pragma unroll
        for (int j = 0; j < PASSES; ++j) {
            const int row = ty + j * ROWS;
            if (tx < np && row < nq) *reinterpret_cast<U *>(to + row * row_step) = cell[tx][row];
        }
    }
}

// Single bytes, source dense along q and destination dense along p, any pitches:
// the tiled kernel above would move one byte per lane.  Here a CTA moves a tile of
// 128 x 128 bytes with 32-bit global accesses on both sides although no row is
// aligned:
//   1. every source row segment is read as the ALIGNED words that cover it (33 at
//      most, coalesced; 17 loads in flight per lane) into R, with the row's byte
//      offset s = address mod 4 noted beside it;
//   2. threads transpose 4 x 4 byte blocks: four unaligned 4-byte groups are cut out
//      of R with a funnel shift by the row's offset, permuted in registers and
//      written to T (rows = q, bytes = p) as aligned words;
//   3. every destination row segment is written as aligned words cut out of T with a
//      funnel shift by the destination offset; the partial words at the two ends
//      go out as single bytes.
// Words of step 1 that are not wholly inside the source's address extent
// [src_lo, src_hi) are put together from single bytes, so nothing outside the
// array is touched.  Pitches in words (34 for R, 33 for T) make the 32-bit accesses
// of steps 1-3 bank-conflict free (lanes: 8 column blocks x 4 row blocks in step 2).
constexpr int kByteTile = 128;
constexpr int kRawPitch = 34, kTurnedPitch = 33;

__device__ __forceinline__ uint32_t load_covering_word(const unsigned char *word, const unsigned char *lo,
                                                       const unsigned char *hi) {
    if (word >= lo && word + 4 <= hi) return *reinterpret_cast<const uint32_t *>(word);
    uint32_t v = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b)
        if (word + b >= lo && word + b < hi) v |= static_cast<uint32_t>(word[b]) << (8 * b);
    return v;
}

template <typename Index>
__global__ void __launch_bounds__(kTiledThreads)
assign_byte_tiles_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                         const __grid_constant__ Axes ax, int q, int64_t tiles_p, int64_t tiles_q,
                         const unsigned char *src_lo, const unsigned char *src_hi) {
    __shared__ uint32_t raw[kByteTile * kRawPitch];
    __shared__ uint32_t turned[kByteTile * kTurnedPitch];
    __shared__ unsigned char offset_of_row[kByteTile];
    const int p = ax.n - 1;
    uint64_t blk = blockIdx.x;
    const int64_t tp = static_cast<int64_t>(blk % static_cast<uint64_t>(tiles_p));
    blk /= static_cast<uint64_t>(tiles_p);
    const int64_t tq = static_cast<int64_t>(blk % static_cast<uint64_t>(tiles_q));
    Index rest = static_cast<Index>(blk / static_cast<uint64_t>(tiles_q));
    int64_t dbase = 0, sbase = 0;
#pragma unroll
    for (int k = kMaxAxes - 1; k >= 0; --k) {
        if (k < ax.n && k != p && k != q) {
            const Index len = static_cast<Index>(ax.len[k]);
            const Index quo = rest / len;
            const Index i = rest - quo * len;
            rest = quo;
            dbase += static_cast<int64_t>(i) * ax.dst_step[k];
            sbase += static_cast<int64_t>(i) * ax.src_step[k];
        }
    }
    const int64_t p0 = tp * kByteTile, q0 = tq * kByteTile;
    const int np = static_cast<int>(ax.len[p] - p0 < kByteTile ? ax.len[p] - p0 : kByteTile);
    const int nq = static_cast<int>(ax.len[q] - q0 < kByteTile ? ax.len[q] - q0 : kByteTile);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int ROWS_PER_WARP = kByteTile / (kTiledThreads / 32);  // 16

    // 1. source rows -> raw (aligned covering words)
    {
        const unsigned char *tile = src + sbase + p0 * ax.src_step[p] + q0;
        const int64_t row_step = ax.src_step[p];
        uint32_t held[ROWS_PER_WARP + 1];
        // Tiles whose covering words all lie inside the source extent (all but those
        // holding the array's first or last bytes) take plain predicated loads, which
        // the compiler can keep in flight together; the others check every word.
        const unsigned char *end_a = tile, *end_b = tile + (np - 1) * row_step;
        const unsigned char *lowest = end_a < end_b ? end_a : end_b, *highest = end_a < end_b ? end_b : end_a;
        const bool interior = lowest - 3 >= src_lo && highest + nq + 7 <= src_hi;
        if (interior) {
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) {
                const int r = warp * ROWS_PER_WARP + i;
                const unsigned char *first = tile + r * row_step;
                const int s = static_cast<int>(reinterpret_cast<uintptr_t>(first) & 3u);
                held[i] = 0u;
                if (r < np && 4 * lane < s + nq) held[i] = *reinterpret_cast<const uint32_t *>(first - s + 4 * lane);
            }
            const int r = warp * ROWS_PER_WARP + (lane & (ROWS_PER_WARP - 1));
            const unsigned char *first = tile + r * row_step;
            const int s = static_cast<int>(reinterpret_cast<uintptr_t>(first) & 3u);
            held[ROWS_PER_WARP] = 0u;
            if (lane < ROWS_PER_WARP && r < np && 4 * 32 < s + nq)
                held[ROWS_PER_WARP] = *reinterpret_cast<const uint32_t *>(first - s + 4 * 32);
            if (lane < ROWS_PER_WARP) offset_of_row[r] = static_cast<unsigned char>(s);
        } else {
#pragma unroll
            for (int i = 0; i < ROWS_PER_WARP; ++i) {
                const int r = warp * ROWS_PER_WARP + i;
                const unsigned char *first = tile + r * row_step;
                const int s = static_cast<int>(reinterpret_cast<uintptr_t>(first) & 3u);
                const bool needed = r < np && 4 * lane < s + nq;
                held[i] = needed ? load_covering_word(first - s + 4 * lane, src_lo, src_hi) : 0u;
            }
            // the 33rd word of a row exists when the row starts inside a word
            const int r = warp * ROWS_PER_WARP + (lane & (ROWS_PER_WARP - 1));
            const unsigned char *first = tile + r * row_step;
            const int s = static_cast<int>(reinterpret_cast<uintptr_t>(first) & 3u);
            const bool needed = lane < ROWS_PER_WARP && r < np && 4 * 32 < s + nq;
            held[ROWS_PER_WARP] = needed ? load_covering_word(first - s + 4 * 32, src_lo, src_hi) : 0u;
            if (lane < ROWS_PER_WARP) offset_of_row[r] = static_cast<unsigned char>(s);
        }
        asm volatile("" ::: "memory");  // all loads issued before the first store waits
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; ++i) raw[(warp * ROWS_PER_WARP + i) * kRawPitch + lane] = held[i];
        if (lane < ROWS_PER_WARP) raw[(warp * ROWS_PER_WARP + lane) * kRawPitch + 32] = held[ROWS_PER_WARP];
    }
    __syncthreads();

    // 2. 4 x 4 byte blocks: raw (rows p) -> turned (rows q)
    {
        const int col_block_lo = lane & 7, row_block_lo = lane >> 3;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int cb = it * 8 + col_block_lo;    // bytes 4cb .. 4cb+3 of the source rows
            const int rb = warp * 4 + row_block_lo;  // source rows 4rb .. 4rb+3
            uint32_t x[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = 4 * rb + i;
                const int o = offset_of_row[r] + 4 * cb;
                const uint32_t *words = raw + r * kRawPitch + (o >> 2);
                x[i] = __funnelshift_r(words[0], words[1], 8 * (o & 3));
            }
            const uint32_t t0 = __byte_perm(x[0], x[1], 0x5140), t1 = __byte_perm(x[2], x[3], 0x5140);
            const uint32_t t2 = __byte_perm(x[0], x[1], 0x7362), t3 = __byte_perm(x[2], x[3], 0x7362);
            uint32_t *out = turned + (4 * cb) * kTurnedPitch + rb;
            out[0 * kTurnedPitch] = __byte_perm(t0, t1, 0x5410);
            out[1 * kTurnedPitch] = __byte_perm(t0, t1, 0x7632);
            out[2 * kTurnedPitch] = __byte_perm(t2, t3, 0x5410);
            out[3 * kTurnedPitch] = __byte_perm(t2, t3, 0x7632);
        }
    }
    __syncthreads();

    // 3. turned -> destination rows (aligned words, single bytes at the ends)
    {
        unsigned char *tile = dst + dbase + q0 * ax.dst_step[q] + p0;
        const int64_t row_step = ax.dst_step[q];
        const unsigned char *turned_bytes = reinterpret_cast<const unsigned char *>(turned);
        auto put = [&](int j, int k) {
            unsigned char *first = tile + j * row_step;
            const int t = static_cast<int>(reinterpret_cast<uintptr_t>(first) & 3u);
            const int o = 4 * k - t;  // row byte position of the word's first byte
            if (o + 4 <= 0 || o >= np) return;
            if (o >= 0 && o + 4 <= np) {
                const uint32_t *words = turned + j * kTurnedPitch + (o >> 2);
                *reinterpret_cast<uint32_t *>(first + o) = __funnelshift_r(words[0], words[1], 8 * (o & 3));
            } else {
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    if (o + b >= 0 && o + b < np) first[o + b] = turned_bytes[j * (kTurnedPitch * 4) + o + b];
            }
        };
#pragma unroll 4
        for (int i = 0; i < ROWS_PER_WARP; ++i) {
            const int j = warp * ROWS_PER_WARP + i;
            if (j < nq) put(j, lane);
        }
        if (lane < ROWS_PER_WARP && warp * ROWS_PER_WARP + lane < nq) put(warp * ROWS_PER_WARP + lane, 32);
    }
}

// Dense runs whose two sides are not aligned alike (a slice that starts one item in,
// rows of an odd pitch): the unit chosen by the host would shrink to the item or a
// byte.  Here a thread owns one ALIGNED 16-byte chunk of a destination run: it loads
// the two aligned 16-byte source words that cover the chunk's bytes, shifts them by
// the run's misalignment (a word select plus a funnel shift), and stores 16 bytes.
// The partial chunks at the two ends of a run are copied byte by byte, and so is a
// chunk whose covering words would reach outside the source's address extent
// [src_lo, src_hi).  `ax` holds the axes other than the run axis.
constexpr int kRunThreads = 256;
constexpr int kRunUnroll = 2;

template <typename Index>
__global__ void __launch_bounds__(kRunThreads)
assign_runs_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src,
                   const __grid_constant__ Axes ax, uint64_t total, int64_t run_bytes, uint64_t chunks_per_run,
                   const unsigned char *src_lo, const unsigned char *src_hi) {
    const uint64_t base = static_cast<uint64_t>(blockIdx.x) * (kRunThreads * kRunUnroll) + threadIdx.x;
    uint4 lo_word[kRunUnroll], hi_word[kRunUnroll];
    unsigned char *to[kRunUnroll];
    const unsigned char *from[kRunUnroll];
    int64_t pos0[kRunUnroll];
    int mode[kRunUnroll];  // 0: nothing, 1: aligned words in lo/hi, 2: byte by byte
#pragma unroll
    for (int j = 0; j < kRunUnroll; ++j) {
        const uint64_t g = base + static_cast<uint64_t>(j) * kRunThreads;
        mode[j] = 0;
        if (g >= total) continue;
        const Index run = static_cast<Index>(g / chunks_per_run);
        const int64_t chunk = static_cast<int64_t>(g - static_cast<uint64_t>(run) * chunks_per_run);
        int64_t doff, soff;
        locate<Index>(ax, run, doff, soff);
        unsigned char *d = dst + doff;
        const unsigned char *s = src + soff;
        const int64_t p0 = 16 * chunk - static_cast<int64_t>(reinterpret_cast<uintptr_t>(d) & 15u);
        if (p0 >= run_bytes) continue;
        to[j] = d;
        from[j] = s;
        pos0[j] = p0;
        mode[j] = 2;
        if (p0 >= 0 && p0 + 16 <= run_bytes) {
            const unsigned char *first = s + p0;
            const unsigned char *aligned = first - (reinterpret_cast<uintptr_t>(first) & 15u);
            if (aligned >= src_lo && aligned + 32 <= src_hi) {
                lo_word[j] = *reinterpret_cast<const uint4 *>(aligned);
                hi_word[j] = *reinterpret_cast<const uint4 *>(aligned + 16);
                mode[j] = 1;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kRunUnroll; ++j) {
        if (mode[j] == 1) {
            const unsigned int m = static_cast<unsigned int>(reinterpret_cast<uintptr_t>(from[j] + pos0[j]) & 15u);
            const uint32_t w[8] = {lo_word[j].x, lo_word[j].y, lo_word[j].z, lo_word[j].w,
                                   hi_word[j].x, hi_word[j].y, hi_word[j].z, hi_word[j].w};
            uint32_t u[6], t[5];
#pragma unroll
            for (int i = 0; i < 6; ++i) u[i] = (m & 8u) ? w[i + 2] : w[i];
#pragma unroll
            for (int i = 0; i < 5; ++i) t[i] = (m & 4u) ? u[i + 1] : u[i];
            const unsigned int shift = (m & 3u) * 8u;
            uint4 v;
            v.x = __funnelshift_r(t[0], t[1], shift);
            v.y = __funnelshift_r(t[1], t[2], shift);
            v.z = __funnelshift_r(t[2], t[3], shift);
            v.w = __funnelshift_r(t[3], t[4], shift);
            *reinterpret_cast<uint4 *>(to[j] + pos0[j]) = v;
        } else if (mode[j] == 2) {
            for (int b = 0; b < 16; ++b) {
                const int64_t pos = pos0[j] + b;
                if (pos >= 0 && pos < run_bytes) to[j][pos] = from[j][pos];
            }
        }
    }
}

int64_t iabs64(int64_t v) { return v < 0 ? -v : v; }

template <typename U>
int launch_unit(void *dst, const void *src, const Axes &ax, uint64_t total, bool narrow_index, int q,
                cudaStream_t stream) {
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    if (q >= 0) {
        constexpr bool SQUARE = sizeof(U) >= 4;
        constexpr int TP = SQUARE ? (sizeof(U) == 4 ? 64 : 32) : TileShape<U>::TP;
        constexpr int TQ = SQUARE ? TP : TileShape<U>::TQ;
        const int p = ax.n - 1;
        const int64_t tiles_p = (ax.len[p] + TP - 1) / TP;
        const int64_t tiles_q = (ax.len[q] + TQ - 1) / TQ;
        uint64_t rest = 1;
        for (int k = 0; k < ax.n; ++k)
            if (k != p && k != q) rest *= static_cast<uint64_t>(ax.len[k]);
        const uint64_t blocks = rest * static_cast<uint64_t>(tiles_p) * static_cast<uint64_t>(tiles_q);
        if (blocks > 0x7FFFFFFFull) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many tiles");
        const unsigned grid = static_cast<unsigned>(blocks);
        if constexpr (SQUARE) {
            if (narrow_index)
                assign_tiled_square_kernel<U, uint32_t, TP><<<grid, kTiledThreads, 0, stream>>>(d, s, ax, q, tiles_p, tiles_q);
            else
                assign_tiled_square_kernel<U, uint64_t, TP><<<grid, kTiledThreads, 0, stream>>>(d, s, ax, q, tiles_p, tiles_q);
        } else {
            if (narrow_index)
                assign_tiled_kernel<U, uint32_t><<<grid, kTiledThreads, 0, stream>>>(d, s, ax, q, tiles_p, tiles_q);
            else
                assign_tiled_kernel<U, uint64_t><<<grid, kTiledThreads, 0, stream>>>(d, s, ax, q, tiles_p, tiles_q);
        }
    } else {
        const uint64_t per_block = kDirectThreads * kDirectUnroll;
        const uint64_t blocks = (total + per_block - 1) / per_block;
        if (blocks > 0x7FFFFFFFull) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many units");
        if (narrow_index)
            assign_direct_kernel<U, uint32_t><<<static_cast<unsigned>(blocks), kDirectThreads, 0, stream>>>(
                d, s, ax, total);
        else
            assign_direct_kernel<U, uint64_t><<<static_cast<unsigned>(blocks), kDirectThreads, 0, stream>>>(
                d, s, ax, total);
    }
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_assign launch");
    return B2K_OK;
}

int launch_byte_tiles(void *dst, const void *src, const Axes &ax, uint64_t total, int q, cudaStream_t stream) {
    const int p = ax.n - 1;
    const int64_t tiles_p = (ax.len[p] + kByteTile - 1) / kByteTile;
    const int64_t tiles_q = (ax.len[q] + kByteTile - 1) / kByteTile;
    uint64_t rest = 1;
    bool narrow = total <= 0xFFFFFFFFull;
    const unsigned char *lo = static_cast<const unsigned char *>(src), *hi = lo + 1;
    for (int k = 0; k < ax.n; ++k) {
        if (k != p && k != q) rest *= static_cast<uint64_t>(ax.len[k]);
        if (ax.len[k] > 0xFFFFFFFFll) narrow = false;
        const int64_t span = (ax.len[k] - 1) * ax.src_step[k];
        if (span < 0) lo += span; else hi += span;
    }
    const uint64_t blocks = rest * static_cast<uint64_t>(tiles_p) * static_cast<uint64_t>(tiles_q);
    if (blocks > 0x7FFFFFFFull) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many tiles");
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    if (narrow)
        assign_byte_tiles_kernel<uint32_t><<<static_cast<unsigned>(blocks), kTiledThreads, 0, stream>>>(
            d, s, ax, q, tiles_p, tiles_q, lo, hi);
    else
        assign_byte_tiles_kernel<uint64_t><<<static_cast<unsigned>(blocks), kTiledThreads, 0, stream>>>(
            d, s, ax, q, tiles_p, tiles_q, lo, hi);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_assign launch");
    return B2K_OK;
}

int launch_runs(void *dst, const void *src, const Axes &ax, cudaStream_t stream) {
    // the fastest axis (dense on both sides, in bytes after scaling by the unit) is the run
    const int n = ax.n;
    const int64_t run_bytes = ax.len[n - 1] * ax.dst_step[n - 1];
    Axes outer{};
    outer.n = n - 1;
    uint64_t runs = 1;
    bool narrow = true;
    const unsigned char *lo = static_cast<const unsigned char *>(src), *hi = lo + run_bytes;
    for (int k = 0; k + 1 < n; ++k) {
        outer.len[k] = ax.len[k];
        outer.dst_step[k] = ax.dst_step[k];
        outer.src_step[k] = ax.src_step[k];
        runs *= static_cast<uint64_t>(ax.len[k]);
        if (ax.len[k] > 0xFFFFFFFFll) narrow = false;
        const int64_t span = (ax.len[k] - 1) * ax.src_step[k];
        if (span < 0) lo += span; else hi += span;
    }
    if (runs > 0xFFFFFFFFull) narrow = false;
    const uint64_t chunks_per_run = static_cast<uint64_t>((run_bytes + 15) / 16 + 1);
    if (runs > (uint64_t(1) << 62) / chunks_per_run) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many chunks");
    const uint64_t total = runs * chunks_per_run;
    const uint64_t per_block = kRunThreads * kRunUnroll;
    const uint64_t blocks = (total + per_block - 1) / per_block;
    if (blocks > 0x7FFFFFFFull) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many chunks");
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    if (narrow)
        assign_runs_kernel<uint32_t><<<static_cast<unsigned>(blocks), kRunThreads, 0, stream>>>(
            d, s, outer, total, run_bytes, chunks_per_run, lo, hi);
    else
        assign_runs_kernel<uint64_t><<<static_cast<unsigned>(blocks), kRunThreads, 0, stream>>>(
            d, s, outer, total, run_bytes, chunks_per_run, lo, hi);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_assign launch");
    return B2K_OK;
}

template <typename U>
int launch_repeat(void *dst, const void *src, const Axes &ax, int b, cudaStream_t stream) {
    // the other axes keep their order; the chunks of axis b become the slowest axis
    Axes rest{};
    memcpy(rest.value, ax.value, sizeof rest.value);
    const int64_t chunks = (ax.len[b] + kRepeatRows - 1) / kRepeatRows;
    rest.n = ax.n;
    rest.len[0] = chunks;
    rest.dst_step[0] = ax.dst_step[b] * kRepeatRows;
    rest.src_step[0] = 0;
    uint64_t units_per_chunk = 1;
    bool narrow = chunks <= 0xFFFFFFFFll;
    for (int k = 0, j = 1; k < ax.n; ++k) {
        if (k == b) continue;
        rest.len[j] = ax.len[k];
        rest.dst_step[j] = ax.dst_step[k];
        rest.src_step[j] = ax.src_step[k];
        units_per_chunk *= static_cast<uint64_t>(ax.len[k]);
        if (ax.len[k] > 0xFFFFFFFFll) narrow = false;
        ++j;
    }
    const uint64_t total = units_per_chunk * static_cast<uint64_t>(chunks);
    if (total > 0xFFFFFFFFull) narrow = false;
    const uint64_t blocks = (total + kDirectThreads - 1) / kDirectThreads;
    if (blocks > 0x7FFFFFFFull) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many units");
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    if (narrow)
        assign_repeat_kernel<U, uint32_t><<<static_cast<unsigned>(blocks), kDirectThreads, 0, stream>>>(
            d, s, rest, total, units_per_chunk, ax.dst_step[b], ax.len[b]);
    else
        assign_repeat_kernel<U, uint64_t><<<static_cast<unsigned>(blocks), kDirectThreads, 0, stream>>>(
            d, s, rest, total, units_per_chunk, ax.dst_step[b], ax.len[b]);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_assign launch");
    return B2K_OK;
}

template <typename S>
int launch_fill(void *dst, const void *src, const Axes &ax, uint64_t total, bool narrow_index,
                cudaStream_t stream) {
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    const uint64_t per_block = kDirectThreads * kDirectUnroll;
    const uint64_t blocks = (total + per_block - 1) / per_block;
    if (blocks > 0x7FFFFFFFull) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: too many units");
    if (narrow_index)
        assign_fill_kernel<S, uint32_t><<<static_cast<unsigned>(blocks), kDirectThreads, 0, stream>>>(d, s, ax, total);
    else
        assign_fill_kernel<S, uint64_t><<<static_cast<unsigned>(blocks), kDirectThreads, 0, stream>>>(d, s, ax, total);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_assign launch");
    return B2K_OK;
}

}  // namespace

namespace {
int assign_impl(void *dst, const void *src, const void *value_host, int ndim, const int64_t *shape,
                const int64_t *dst_strides, const int64_t *src_strides, int64_t itemsize, void *stream);
}  // namespace

extern "C" int b2k_assign(void *dst, const void *src, int ndim, const int64_t *shape, const int64_t *dst_strides,
                          const int64_t *src_strides, int64_t itemsize, void *stream) {
    B2K_RANGE("b2k_assign");
    if (ndim > 0 && !src_strides) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: null shape or strides");
    return assign_impl(dst, src, nullptr, ndim, shape, dst_strides, src_strides, itemsize, stream);
}

extern "C" int b2k_fill(void *dst, int ndim, const int64_t *shape, const int64_t *dst_strides, const void *value_host,
                        int64_t itemsize, void *stream) {
    B2K_RANGE("b2k_fill");
    if (!value_host) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_fill: null value");
    if (itemsize < 1 || itemsize > 16)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_fill: items of 1..16 bytes (got %lld)", static_cast<long long>(itemsize));
    if (ndim < 0 || ndim > 32) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_fill: ndim %d outside 0..32", ndim);
    const int64_t zeros[32] = {};
    return assign_impl(dst, nullptr, value_host, ndim, shape, dst_strides, zeros, itemsize, stream);
}

namespace {
int assign_impl(void *dst, const void *src, const void *value_host, int ndim, const int64_t *shape,
                const int64_t *dst_strides, const int64_t *src_strides, int64_t itemsize, void *stream) {
    if (ndim < 0 || ndim > 32) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: ndim %d outside 0..32", ndim);
    if (itemsize <= 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: itemsize must be positive");
    if (ndim > 0 && (!shape || !dst_strides || !src_strides))
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: null shape or strides");

    struct Axis {
        int64_t len, ds, ss;
    };
    Axis axes[34];
    int n = 0;
    for (int k = 0; k < ndim; ++k) {
        if (shape[k] < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: negative extent");
        if (shape[k] == 0) return B2K_OK;
        if (shape[k] == 1) continue;
        if (dst_strides[k] == 0)
            return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: destination stride 0 on axis %d of length %lld", k,
                             static_cast<long long>(shape[k]));
        axes[n++] = Axis{shape[k], dst_strides[k], src_strides[k]};
    }
    if (!dst || (!src && !value_host)) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_assign: null pointer");

    // densest destination axis last; equal strides keep their given order
    std::stable_sort(axes, axes + n, [](const Axis &a, const Axis &b) { return iabs64(a.ds) > iabs64(b.ds); });
    // the item itself: one more axis of bytes, dense on both sides
    axes[n++] = Axis{itemsize, 1, 1};
    // merge neighbours that are contiguous on both sides
    int m = 0;
    for (int k = 0; k < n; ++k) {
        if (m > 0 && axes[m - 1].ds == axes[k].len * axes[k].ds && axes[m - 1].ss == axes[k].len * axes[k].ss) {
            axes[m - 1].len *= axes[k].len;
            axes[m - 1].ds = axes[k].ds;
            axes[m - 1].ss = axes[k].ss;
        } else {
            axes[m++] = axes[k];
        }
    }
    n = m;
    // widest unit: divides the dense run, both addresses and every other step
    int64_t unit = 16;
    auto fits = [&](int64_t u) {
        if (axes[n - 1].len % u) return false;
        // (a null source stands for the 16-byte aligned value in the kernel parameters)
        if (reinterpret_cast<uintptr_t>(dst) % u || reinterpret_cast<uintptr_t>(src) % u) return false;
        for (int k = 0; k + 1 < n; ++k)
            if (axes[k].ds % u || axes[k].ss % u) return false;
        return true;
    };
    while (unit > 1 && !fits(unit)) unit /= 2;
    axes[n - 1].len /= unit;
    axes[n - 1].ds = unit;
    axes[n - 1].ss = unit;
    if (axes[n - 1].len == 1 && n > 1) --n;
    if (n > kMaxAxes)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_assign: %d axes remain after merging (at most %d)", n, kMaxAxes);

    Axes ax{};
    ax.n = n;
    if (value_host) memcpy(ax.value, value_host, static_cast<size_t>(itemsize));
    uint64_t total = 1;
    bool narrow = true;
    for (int k = 0; k < n; ++k) {
        ax.len[k] = axes[k].len;
        ax.dst_step[k] = axes[k].ds;
        ax.src_step[k] = axes[k].ss;
        if (axes[k].len > 0xFFFFFFFFll) narrow = false;
        if (total > (uint64_t(1) << 62) / static_cast<uint64_t>(axes[k].len))
            return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_assign: more than 2^62 units");
        total *= static_cast<uint64_t>(axes[k].len);
    }
    if (total > 0xFFFFFFFFull) narrow = false;

    cudaStream_t st = b2k::as_stream(stream);

    // The source repeats along the fastest axis and the destination is dense there:
    // store the repeated unit 16 bytes at a time where the rows allow it.
    if (unit < 16 && ax.src_step[n - 1] == 0 && ax.dst_step[n - 1] == unit) {
        const int64_t rep = 16 / unit;
        bool wide = ax.len[n - 1] % rep == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
        for (int k = 0; k + 1 < n; ++k)
            if (ax.dst_step[k] % 16) wide = false;
        if (wide) {
            Axes fill = ax;
            fill.len[n - 1] /= rep;
            fill.dst_step[n - 1] = 16;
            const uint64_t units = total / static_cast<uint64_t>(rep);
            switch (unit) {
            case 8: return launch_fill<uint2>(dst, src, fill, units, narrow, st);
            case 4: return launch_fill<uint32_t>(dst, src, fill, units, narrow, st);
            case 2: return launch_fill<uint16_t>(dst, src, fill, units, narrow, st);
            default: return launch_fill<uint8_t>(dst, src, fill, units, narrow, st);
            }
        }
    }

    // Both sides dense along the fastest axis, but their alignments kept the unit
    // below 16 bytes: long runs go through aligned 16-byte chunks all the same.
    if (src && unit < 16 && ax.src_step[n - 1] == unit && ax.dst_step[n - 1] == unit &&
        ax.len[n - 1] * unit >= 128 && B2K_ENV_INT("B2K_ASSIGN_RUNS", 1) != 0) {
        bool repeats = false;  // (a repeated source has its own kernel below)
        for (int k = 0; k + 1 < n; ++k)
            if (ax.src_step[k] == 0 && ax.len[k] >= 2 * kRepeatRows) repeats = true;
        if (!repeats) return launch_runs(dst, src, ax, st);
    }

    // The source repeats along a slower axis and both sides are dense along the
    // fastest one: read once, store to many rows.
    if (n >= 2 && ax.src_step[n - 1] == unit && ax.dst_step[n - 1] == unit) {
        int b = -1;
        for (int k = 0; k + 1 < n; ++k)
            if (ax.src_step[k] == 0 && ax.len[k] >= 2 * kRepeatRows && (b < 0 || ax.len[k] > ax.len[b])) b = k;
        if (b >= 0) {
            switch (unit) {
            case 16: return launch_repeat<uint4>(dst, src, ax, b, st);
            case 8: return launch_repeat<uint2>(dst, src, ax, b, st);
            case 4: return launch_repeat<uint32_t>(dst, src, ax, b, st);
            case 2: return launch_repeat<uint16_t>(dst, src, ax, b, st);
            default: return launch_repeat<uint8_t>(dst, src, ax, b, st);
            }
        }
    }

    // Source densest along another axis q than the destination (an axis permutation).
    int q = -1;
    if (n >= 2 && B2K_ENV_INT("B2K_ASSIGN_TILED", 1) != 0) {
        int best = -1;
        for (int k = 0; k < n; ++k) {
            if (ax.src_step[k] == 0) continue;
            if (best < 0 || iabs64(ax.src_step[k]) < iabs64(ax.src_step[best])) best = k;
        }
        // worth it only when the source run along the destination's fastest axis is
        // strided by more than a sector and both tile axes are long enough
        if (best >= 0 && best != n - 1 && iabs64(ax.src_step[n - 1]) >= 32 && ax.len[best] >= 8 &&
            ax.len[n - 1] >= 8)
            q = best;
    }
    // Both sides dense along their own axis, everything 16-byte aligned, at most
    // three further axes: a stack of 2-D transposes for the TMA tile kernel.
    if (q >= 0 && n <= 5 && ax.dst_step[n - 1] == unit && ax.src_step[q] == unit && ax.len[q] >= 32 &&
        ax.len[n - 1] >= 32 && total * static_cast<uint64_t>(unit) >= (1u << 20) &&
        B2K_ENV_INT("B2K_ASSIGN_TMA", 1) != 0) {
        int64_t blen[3], istep[3], ostep[3];
        int nb = 0;
        for (int k = n - 2; k >= 0; --k) {  // fastest batch axis first
            if (k == q) continue;
            blen[nb] = ax.len[k];
            istep[nb] = ax.src_step[k];
            ostep[nb] = ax.dst_step[k];
            ++nb;
        }
        // in = rows (axis p) x cols (axis q, dense); out = cols x rows (axis p dense)
        const int rc = b2k::transpose_tma_batched(src, dst, ax.len[n - 1], ax.len[q], ax.src_step[n - 1],
                                                  ax.dst_step[q], nb, blen, istep, ostep, unit, st);
        if (rc != B2K_ERR_UNSUPPORTED) return rc;
    }

    switch (unit) {
    case 16: return launch_unit<uint4>(dst, src, ax, total, narrow, q, st);
    case 8: return launch_unit<uint2>(dst, src, ax, total, narrow, q, st);
    case 4: return launch_unit<uint32_t>(dst, src, ax, total, narrow, q, st);
    case 2: return launch_unit<uint16_t>(dst, src, ax, total, narrow, q, st);
    default:
        if (q >= 0 && ax.src_step[q] == 1 && ax.dst_step[n - 1] == 1 && ax.len[q] >= 32 && ax.len[n - 1] >= 32 &&
            B2K_ENV_INT("B2K_ASSIGN_BYTE_TILES", 1) != 0)
            return launch_byte_tiles(dst, src, ax, total, q, st);
        return launch_unit<uint8_t>(dst, src, ax, total, narrow, q, st);
    }
}
}  // namespace
