// TMA tile transpose for items of 1, 2, 4, 8 or 16 bytes (sm_100a).
//
// Replaces the one-element-per-thread tile kernel of
// numba/cuda/kernels/transpose.py:42-57 for arrays whose rows are contiguous
// and 16-byte aligned on both sides.
//
// Data path of one input tile of R rows x 128 bytes (128/ES columns):
//
//   global --cp.async.bulk.tensor (tiled, 128-byte swizzle)--> stage A[s]
//   A[s]   --ld.shared.v4 per (row, 16-byte chunk); lanes walk rows, and the
//            swizzle puts chunk q of row r at chunk (q ^ (r & 7)), so a
//            quarter-warp always touches eight different bank groups----------.
//   B[b]   <-st.shared of single items, lanes walk the contiguous direction <-'
//            (1- and 2-byte items: four / two rows are first interleaved in
//             registers with byte permutes so that every store is a 32-bit word)
//   B[b]   --cp.async.bulk.tensor store (tiled, no swizzle)--> global
//
// B holds the transposed tile as (128/ES) output rows of R items, R = 64 (8 KB
// tiles, four load stages).  For single bytes an output row of a tile is 64 bytes,
// half a line: the tile below writes the other half a few tiles later and the two
// meet in L2 (measured faster than 128-row tiles of 16 KB).  Edge tiles
// need no code: out-of-range parts of a load read as zero and out-of-range
// parts of a store are dropped by the tensor-map bounds.
//
// Two persistent CTAs per SM walk the tiles panel by panel (see TileOrder); a
// ring of NSTAGE loads per CTA stays in flight and B is double buffered against
// the asynchronous store.  Two CTAs per SM is a sharp optimum on B200: one cannot
// hide its own transpose step, three or more only add DRAM page conflicts.
//
// HBM roofline: 2*ES bytes per item (one read, one write).
#include <cuda.h>

#include <mutex>

#include "b2k_internal.cuh"

namespace {

constexpr uint32_t kWaitLimit = 1u << 22;  // mbarrier polls before giving up

__device__ unsigned int g_wait_timeouts = 0;  // bumped when a bounded wait runs out

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait: false when the phase did not complete within kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t spin = 0; spin < kWaitLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, const void *src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(smem_addr(src))
                 : "memory");
}
__device__ __forceinline__ void tma_load_5d(void *dst, const CUtensorMap *map, int x, int y, int b0, int b1,
                                            int b2, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], "
        "[%7];" ::"r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(b0), "r"(b1), "r"(b2), "r"(smem_addr(bar))
        : "memory");
}
__device__ __forceinline__ void tma_store_5d(const CUtensorMap *map, int x, int y, int b0, int b1, int b2,
                                             const void *src) {
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];"
                 ::"l"(map), "r"(x), "r"(y), "r"(b0), "r"(b1), "r"(b2), "r"(smem_addr(src))
                 : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int ES> struct Item;
template <> struct Item<1> { using type = uint8_t; };
template <> struct Item<2> { using type = uint16_t; };
template <> struct Item<4> { using type = uint32_t; };
template <> struct Item<8> { using type = uint2; };
template <> struct Item<16> { using type = uint4; };

// Transpose one staged tile: A is R rows x 128 B (swizzled), B is (128/ES) rows
// of R items (linear).
//
// Items of 4 bytes and more: a thread reads one 16-byte chunk of one row and
// scatters its items; lanes walk rows, so reads are conflict-free through the
// swizzle and writes run along B's contiguous direction.
template <int ES, int R, int THREADS>
__device__ __forceinline__ void transpose_tile(const unsigned char *A, unsigned char *B) {
    using T = typename Item<ES>::type;
    constexpr int EPC = 16 / ES;  // items per 16-byte chunk
    constexpr int ITEMS = R * 8;  // (row, chunk) pairs
    static_assert(ITEMS % THREADS == 0, "tile must split evenly over the block");
#pragma unroll
    for (int w = threadIdx.x; w < ITEMS; w += THREADS) {
        const int r = w % R;
        const int q = w / R;
        const uint4 v = *reinterpret_cast<const uint4 *>(A + r * 128 + ((q ^ (r & 7)) << 4));
        union { uint4 raw; T e[EPC]; } u;
        u.raw = v;
        T *dst = reinterpret_cast<T *>(B) + static_cast<size_t>(q * EPC) * R + r;
#pragma unroll
        for (int k = 0; k < EPC; ++k) dst[k * R] = u.e[k];
    }
}

// 2-byte items, R = 64, 256 threads: a thread owns two consecutive rows (2g, 2g+1)
// and one chunk of eight columns, pairs the rows with byte permutes and stores
// eight 32-bit words (column c, rows 2g..2g+1).  Lane mapping inside a warp:
// quarter-warp s, lane j -> row pair g = 8s + j, chunk q0 ^ (j >> 2) with q0 = warp;
// the eight lanes of a quarter-warp then read eight different swizzled chunks and
// the 32 lanes of a store hit 32 different banks (bank = g).
template <>
__device__ __forceinline__ void transpose_tile<2, 64, 256>(const unsigned char *A, unsigned char *B) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = lane & 7;
    const int g = (lane >> 3) * 8 + j;
    const int q = warp ^ (j >> 2);
    const int r0 = 2 * g;
    const uint4 a = *reinterpret_cast<const uint4 *>(A + r0 * 128 + ((q ^ (r0 & 7)) << 4));
    const uint4 b = *reinterpret_cast<const uint4 *>(A + (r0 + 1) * 128 + ((q ^ ((r0 + 1) & 7)) << 4));
    uint32_t *dst = reinterpret_cast<uint32_t *>(B) + (q * 8) * 32 + g;  // B row = 64 items = 32 words
    const uint32_t ra[4] = {a.x, a.y, a.z, a.w}, rb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        dst[(2 * k) * 32] = __byte_perm(ra[k], rb[k], 0x5410);      // column 2k:   low halves
        dst[(2 * k + 1) * 32] = __byte_perm(ra[k], rb[k], 0x7632);  // column 2k+1: high halves
    }
}

// 1-byte items, R = 64, 256 threads: a thread owns four consecutive rows (4g..4g+3)
// and eight columns (half h of chunk q), transposes two 4x4 byte blocks with byte
// permutes and stores eight 32-bit words (column c, rows 4g..4g+3; a B row is 64
// bytes = 16 words).  Thread t: i = t mod 16 gives h = i & 1 and the swizzled chunk
// position i >> 1, so the sixteen lanes of a half-warp read sixteen different 8-byte
// bank pairs whatever their rows; g = (i + t / 16) mod 16 puts every row group twice
// into a warp, and the upper half-warp stores its columns in swapped pairs, so the
// two lanes that share a row group hit different banks (bank = 16 (c & 1) + g).
template <>
__device__ __forceinline__ void transpose_tile<1, 64, 256>(const unsigned char *A, unsigned char *B) {
    const int i = threadIdx.x & 15, upper = (threadIdx.x >> 4) & 1;
    const int g = (i + (threadIdx.x >> 4)) & 15;
    const int h = i & 1;
    const int q = (i >> 1) ^ ((g & 1) << 2);
    const int r0 = 4 * g;
    uint2 row[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
        row[k] = *reinterpret_cast<const uint2 *>(A + (r0 + k) * 128 + ((q ^ ((r0 + k) & 7)) << 4) + h * 8);
    uint32_t o[8];
    {
        const uint32_t t0 = __byte_perm(row[0].x, row[1].x, 0x5140), t1 = __byte_perm(row[2].x, row[3].x, 0x5140);
        const uint32_t t2 = __byte_perm(row[0].x, row[1].x, 0x7362), t3 = __byte_perm(row[2].x, row[3].x, 0x7362);
        o[0] = __byte_perm(t0, t1, 0x5410);
        o[1] = __byte_perm(t0, t1, 0x7632);
        o[2] = __byte_perm(t2, t3, 0x5410);
        o[3] = __byte_perm(t2, t3, 0x7632);
    }
    {
        const uint32_t t0 = __byte_perm(row[0].y, row[1].y, 0x5140), t1 = __byte_perm(row[2].y, row[3].y, 0x5140);
        const uint32_t t2 = __byte_perm(row[0].y, row[1].y, 0x7362), t3 = __byte_perm(row[2].y, row[3].y, 0x7362);
        o[4] = __byte_perm(t0, t1, 0x5410);
        o[5] = __byte_perm(t0, t1, 0x7632);
        o[6] = __byte_perm(t2, t3, 0x5410);
        o[7] = __byte_perm(t2, t3, 0x7632);
    }
    uint32_t *dst = reinterpret_cast<uint32_t *>(B) + (q * 16 + h * 8) * 16 + g;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = upper ? (j ^ 1) : j;
        dst[c * 16] = upper ? o[j ^ 1] : o[j];
    }
}

// Tile order.  Tiles are numbered panel by panel: a panel is `panel_w` tiles wide
// (along input columns) and spans all tile rows; inside a panel the tile column
// varies fastest.  CTAs that run at the same time therefore cover a 2-D patch of
// the matrix, which keeps both the 128-byte-wide reads and the R-item-wide
// writes of neighbouring CTAs next to each other in memory instead of lining
// one of the two sides up at a power-of-two pitch.
struct TileOrder {
    int tiles_x, tiles_y, panel_w;
    // tile numbers fit 31 bits (checked by the launcher): 32-bit divisions only
    __device__ __forceinline__ void coords(unsigned int id, int &tx, int &ty) const {
        const unsigned int per_panel = static_cast<unsigned int>(panel_w) * static_cast<unsigned int>(tiles_y);
        const int panel = static_cast<int>(id / per_panel);
        const int within = static_cast<int>(id - static_cast<unsigned int>(panel) * per_panel);
        const int tx0 = panel * panel_w;
        const int w = min(panel_w, tiles_x - tx0);
        ty = within / w;
        tx = tx0 + within - ty * w;
    }
};

template <int ES, int R, int NSTAGE, int THREADS, int NOUT, bool SPLIT>
__global__ void __launch_bounds__(THREADS)
transpose_tma_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                     const TileOrder order, long long tiles, int refill_thread) {
    constexpr int TILE_BYTES = R * 128;
    constexpr int TCOLS = 128 / ES;
    // tensor-map elements per item along the contiguous direction (32-bit words
    // for items wider than 4 bytes); x coordinates are counted in those elements
    constexpr int WORDS = ES > 4 ? ES / 4 : 1;
    extern __shared__ unsigned char smem_raw[];
    // the 128-byte swizzle pattern is a function of address bits 7..9
    unsigned char *base = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *A = base;
    unsigned char *B = base + NSTAGE * TILE_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(B + NOUT * TILE_BYTES);

    const long long first = blockIdx.x;
    const long long step = gridDim.x;

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < NSTAGE; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        // fill the ring
#pragma unroll
        for (int s = 0; s < NSTAGE; ++s) {
            const long long id = first + s * step;
            if (id < tiles) {
                int tx, ty;
                order.coords(static_cast<unsigned int>(id), tx, ty);
                mbar_expect_tx(&full[s], TILE_BYTES);
                tma_load_2d(A + s * TILE_BYTES, &in_map, tx * (TCOLS * WORDS), ty * R, &full[s]);
            }
        }
    }
    __syncthreads();

    // Thread 0 stores finished tiles and refills the load ring (SPLIT: as two
    // separate blocks, the refill by `refill_thread`, which the launcher sets to 0).
    // Tile coordinates are worked out before the wait for the tile.
    bool ok = true;
    int it = 0;
    for (long long id = first; id < tiles; id += step, ++it) {
        const int s = it % NSTAGE;
        const int b = it % NOUT;
        int tx = 0, ty = 0;
        bool refill = false;
        int ltx = 0, lty = 0;
        if constexpr (SPLIT) {
            if (threadIdx.x == 0) {
                order.coords(static_cast<unsigned int>(id), tx, ty);
                tma_wait_read<NOUT - 1>();  // the store that last read B[b] has drained
            }
            if (threadIdx.x == refill_thread) {
                const long long next = id + NSTAGE * step;
                refill = next < tiles;
                if (refill) order.coords(static_cast<unsigned int>(next), ltx, lty);
            }
        } else {
            if (threadIdx.x == 0) {
                order.coords(static_cast<unsigned int>(id), tx, ty);
                const long long next = id + NSTAGE * step;
                refill = next < tiles;
                if (refill) order.coords(static_cast<unsigned int>(next), ltx, lty);
                tma_wait_read<NOUT - 1>();  // the store that last read B[b] has drained
            }
        }
        ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
        // every thread polls the same barrier, so the vote only guards against skew
        if (!__syncthreads_and(ok)) { ok = false; break; }

        transpose_tile<ES, R, THREADS>(A + s * TILE_BYTES, B + b * TILE_BYTES);
        fence_async_smem();
        __syncthreads();

        if constexpr (SPLIT) {
            if (threadIdx.x == 0) {
                // output coordinates: x runs along input rows, y along input columns
                tma_store_2d(&out_map, ty * (R * WORDS), tx * TCOLS, B + b * TILE_BYTES);
                tma_commit();
            }
            if (threadIdx.x == refill_thread && refill) {
                mbar_expect_tx(&full[s], TILE_BYTES);
                tma_load_2d(A + s * TILE_BYTES, &in_map, ltx * (TCOLS * WORDS), lty * R, &full[s]);
            }
        } else {
            if (threadIdx.x == 0) {
                tma_store_2d(&out_map, ty * (R * WORDS), tx * TCOLS, B + b * TILE_BYTES);
                tma_commit();
                if (refill) {
                    mbar_expect_tx(&full[s], TILE_BYTES);
                    tma_load_2d(A + s * TILE_BYTES, &in_map, ltx * (TCOLS * WORDS), lty * R, &full[s]);
                }
            }
        }
    }
    if (threadIdx.x == 0) {
        if (!ok) atomicAdd(&g_wait_timeouts, 1u);
        tma_wait_all();
    }
}

// The same pipeline over a stack of 2-D problems: up to three further axes (batch
// axes) select the 2-D slice, tile numbers run slice by slice, and the tensor maps
// are five-dimensional with a box depth of 1 along the batch axes.  This serves
// N-D axis permutations whose source and destination are dense along two
// different axes (b2k_assign).
struct BatchSplit {
    unsigned int tiles2d;     // tiles per 2-D slice
    unsigned int len0, len1;  // lengths of the first two batch axes (the third takes the rest)
    // one grid stride (gridDim.x tiles) as slice-local tiles plus batch steps, so
    // that a CTA walks its tiles with additions instead of divisions
    unsigned int adv_tile, adv0, adv1, adv2;
};

struct TileCoord {
    int tx, ty, b0, b1, b2;
};

// Position of a CTA's next tile to load: tile number inside the slice and the
// batch coordinates.
struct TileCursor {
    unsigned int id2, b0, b1, b2;

    __device__ __forceinline__ void seek(const BatchSplit &bs, unsigned int id) {
        const unsigned int b = id / bs.tiles2d;
        id2 = id - b * bs.tiles2d;
        const unsigned int q0 = b / bs.len0;
        b0 = b - q0 * bs.len0;
        const unsigned int q1 = q0 / bs.len1;
        b1 = q0 - q1 * bs.len1;
        b2 = q1;
    }
    __device__ __forceinline__ void advance(const BatchSplit &bs) {
        id2 += bs.adv_tile;
        unsigned int carry = id2 >= bs.tiles2d;
        if (carry) id2 -= bs.tiles2d;
        b0 += bs.adv0 + carry;
        carry = b0 >= bs.len0;
        if (carry) b0 -= bs.len0;
        b1 += bs.adv1 + carry;
        carry = b1 >= bs.len1;
        if (carry) b1 -= bs.len1;
        b2 += bs.adv2 + carry;
    }
    __device__ __forceinline__ TileCoord coord(const TileOrder &order) const {
        TileCoord c;
        order.coords(id2, c.tx, c.ty);
        c.b0 = static_cast<int>(b0);
        c.b1 = static_cast<int>(b1);
        c.b2 = static_cast<int>(b2);
        return c;
    }
};

template <int ES, int R, int NSTAGE, int THREADS, int NOUT>
__global__ void __launch_bounds__(THREADS)
transpose_tma_batched_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                             const TileOrder order, const BatchSplit bs, long long tiles, int refill_thread) {
    constexpr int TILE_BYTES = R * 128;
    constexpr int TCOLS = 128 / ES;
    constexpr int WORDS = ES > 4 ? ES / 4 : 1;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *base = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *A = base;
    unsigned char *B = base + NSTAGE * TILE_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(B + NOUT * TILE_BYTES);
    // where each staged tile goes: written when its load is issued, read when it is stored
    __shared__ TileCoord staged[NSTAGE];

    const long long first = blockIdx.x;
    const long long step = gridDim.x;

    TileCursor cursor{0, 0, 0, 0};
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < NSTAGE; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
        cursor.seek(bs, static_cast<unsigned int>(first));
#pragma unroll
        for (int s = 0; s < NSTAGE; ++s) {
            const long long id = first + s * step;
            if (id < tiles) {
                const TileCoord c = cursor.coord(order);
                staged[s] = c;
                mbar_expect_tx(&full[s], TILE_BYTES);
                tma_load_5d(A + s * TILE_BYTES, &in_map, c.tx * (TCOLS * WORDS), c.ty * R, c.b0, c.b1, c.b2,
                            &full[s]);
                cursor.advance(bs);
            }
        }
    }
    __syncthreads();

    // Thread 0 issues everything (the launcher passes refill_thread = 0; see launch()
    // for why the store and the refill stay two separate blocks).
    bool ok = true;
    int it = 0;
    for (long long id = first; id < tiles; id += step, ++it) {
        const int s = it % NSTAGE;
        const int b = it % NOUT;
        TileCoord cur{0, 0, 0, 0, 0}, nxt{0, 0, 0, 0, 0};
        bool refill = false;
        if (threadIdx.x == 0) {
            cur = staged[s];
            tma_wait_read<NOUT - 1>();  // the store that last read B[b] has drained
        }
        if (threadIdx.x == refill_thread) {
            refill = id + NSTAGE * step < tiles;
            if (refill) nxt = cursor.coord(order);
        }
        ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
        if (!__syncthreads_and(ok)) { ok = false; break; }

        transpose_tile<ES, R, THREADS>(A + s * TILE_BYTES, B + b * TILE_BYTES);
        fence_async_smem();
        __syncthreads();

        if (threadIdx.x == 0) {
            tma_store_5d(&out_map, cur.ty * (R * WORDS), cur.tx * TCOLS, cur.b0, cur.b1, cur.b2, B + b * TILE_BYTES);
            tma_commit();
        }
        if (threadIdx.x == refill_thread && refill) {
            staged[s] = nxt;
            mbar_expect_tx(&full[s], TILE_BYTES);
            tma_load_5d(A + s * TILE_BYTES, &in_map, nxt.tx * (TCOLS * WORDS), nxt.ty * R, nxt.b0, nxt.b1, nxt.b2,
                        &full[s]);
            cursor.advance(bs);
        }
    }
    if (threadIdx.x == 0) {
        if (!ok) atomicAdd(&g_wait_timeouts, 1u);
        tma_wait_all();
    }
}

// ---- host --------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::mutex mu;
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A 2-D map over `rows` lines of `cols` items (ES bytes each, lines `pitch` bytes
// apart) with a box of box_cols x box_rows items.
template <int ES>
bool make_map(CUtensorMap *map, const void *ptr, int64_t rows, int64_t cols, int64_t pitch, int box_cols,
              int box_rows, bool swizzle) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    // map elements: the item itself up to 4 bytes, 32-bit words for wider items
    constexpr int UNIT = ES >= 4 ? 4 : ES;
    constexpr int WORDS = ES / UNIT;
    const CUtensorMapDataType type = UNIT == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                     : UNIT == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols) * WORDS, static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols * WORDS), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    return enc(map, type, 2, const_cast<void *>(ptr), dims, strides, box, elem_strides,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int ES, int R, int NSTAGE, int THREADS = 256, int NOUT = 2>
int launch(const void *in, void *out, int64_t rows, int64_t cols, int64_t in_pitch, int64_t out_pitch,
           cudaStream_t stream) {
    constexpr int TCOLS = 128 / ES;
    constexpr int UNIT = ES >= 4 ? 4 : ES;
    static_assert(R * (ES / UNIT) <= 256, "store box exceeds the tensor-map limit");
    CUtensorMap in_map, out_map;
    if (!make_map<ES>(&in_map, in, rows, cols, in_pitch, TCOLS, R, true) ||
        !make_map<ES>(&out_map, out, cols, rows, out_pitch, R, TCOLS, false))
        return B2K_ERR_UNSUPPORTED;
    const int64_t tiles_x = (cols + TCOLS - 1) / TCOLS;
    const int64_t tiles_y = (rows + R - 1) / R;
    const int64_t tiles = tiles_x * tiles_y;
    if (tiles > 0x7FFFFFFFll) return B2K_ERR_UNSUPPORTED;  // the kernel numbers tiles in 31 bits
    constexpr int SMEM = (NSTAGE + NOUT) * R * 128 + NSTAGE * 8 + 1024;
    // Two code shapes for the issuing thread, chosen by measurement.  With the
    // store and the refill in separate blocks (SPLIT) lines that are not 128-byte
    // aligned run 10-40 % faster, and 4-byte items gain 2-3 % on aligned lines too;
    // the merged shape is 3-7 % ahead for 1- and 2-byte items on 128-byte-aligned
    // lines.  DRAM traffic and the isolated launch time are the same for both, so
    // the difference comes from how the CTAs' requests fall into step over
    // back-to-back tiles.
    const bool aligned = in_pitch % 128 == 0 && out_pitch % 128 == 0;
    const bool auto_split = ES >= 4 || !aligned;
    const int forced = B2K_ENV_INT("B2K_TRANSPOSE_SPLIT", -1);
    const bool split = forced < 0 ? auto_split : forced != 0;
    auto kernel = split ? transpose_tma_kernel<ES, R, NSTAGE, THREADS, NOUT, true>
                        : transpose_tma_kernel<ES, R, NSTAGE, THREADS, NOUT, false>;
    // the shared-memory limit is a per-device attribute of the function
    static b2k::PerDeviceOnce once;
    const cudaError_t attr_status = once.run([] {
        cudaError_t e = cudaFuncSetAttribute(transpose_tma_kernel<ES, R, NSTAGE, THREADS, NOUT, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(transpose_tma_kernel<ES, R, NSTAGE, THREADS, NOUT, false>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        return e;
    });
    if (attr_status != cudaSuccess) return b2k::check_cuda(attr_status, "transpose smem attribute");
    // two resident CTAs per SM measured best (more CTAs only add DRAM page conflicts)
    const int per_sm = B2K_ENV_INT("B2K_TRANSPOSE_CTAS_PER_SM", 2);
    int64_t grid = static_cast<int64_t>(b2k::sm_count()) * (per_sm < 1 ? 1 : per_sm);
    if (grid > tiles) grid = tiles;
    int panel_w = B2K_ENV_INT("B2K_TRANSPOSE_PANEL", 4);
    if (panel_w < 1 || panel_w > tiles_x) panel_w = static_cast<int>(tiles_x);
    const TileOrder order{static_cast<int>(tiles_x), static_cast<int>(tiles_y), panel_w};
    // the refill thread is a run-time argument on purpose: as a constant the compiler
    // would fuse the two blocks of the SPLIT shape back into one
    kernel<<<static_cast<unsigned>(grid), THREADS, SMEM, stream>>>(in_map, out_map, order,
                                                                   static_cast<long long>(tiles),
                                                                   B2K_ENV_INT("B2K_TRANSPOSE_REFILL_THREAD", 0));
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_transpose2d (tma) launch");
    return B2K_OK;
}

// A 5-D map for the batched kernel: axis 0 and 1 as in make_map, then up to three
// batch axes (length 1 where unused) with a box depth of 1.
template <int ES>
bool make_map5(CUtensorMap *map, const void *ptr, int64_t rows, int64_t cols, int64_t pitch, int box_cols,
               int box_rows, bool swizzle, const int64_t *batch_len, const int64_t *batch_step) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    constexpr int UNIT = ES >= 4 ? 4 : ES;
    constexpr int WORDS = ES / UNIT;
    const CUtensorMapDataType type = UNIT == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                     : UNIT == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const cuuint64_t dims[5] = {static_cast<cuuint64_t>(cols) * WORDS, static_cast<cuuint64_t>(rows),
                                static_cast<cuuint64_t>(batch_len[0]), static_cast<cuuint64_t>(batch_len[1]),
                                static_cast<cuuint64_t>(batch_len[2])};
    const cuuint64_t strides[4] = {static_cast<cuuint64_t>(pitch), static_cast<cuuint64_t>(batch_step[0]),
                                   static_cast<cuuint64_t>(batch_step[1]), static_cast<cuuint64_t>(batch_step[2])};
    const cuuint32_t box[5] = {static_cast<cuuint32_t>(box_cols * WORDS), static_cast<cuuint32_t>(box_rows), 1, 1, 1};
    const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
    return enc(map, type, 5, const_cast<void *>(ptr), dims, strides, box, elem_strides,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int ES, int R, int NSTAGE, int THREADS = 256, int NOUT = 2>
int launch_batched(const void *in, void *out, int64_t rows, int64_t cols, int64_t in_pitch, int64_t out_pitch,
                   const int64_t *batch_len, const int64_t *in_batch_step, const int64_t *out_batch_step,
                   cudaStream_t stream) {
    constexpr int TCOLS = 128 / ES;
    CUtensorMap in_map, out_map;
    if (!make_map5<ES>(&in_map, in, rows, cols, in_pitch, TCOLS, R, true, batch_len, in_batch_step) ||
        !make_map5<ES>(&out_map, out, cols, rows, out_pitch, R, TCOLS, false, batch_len, out_batch_step))
        return B2K_ERR_UNSUPPORTED;
    const int64_t tiles_x = (cols + TCOLS - 1) / TCOLS;
    const int64_t tiles_y = (rows + R - 1) / R;
    const int64_t tiles2d = tiles_x * tiles_y;
    const int64_t slices = batch_len[0] * batch_len[1] * batch_len[2];
    if (tiles2d > 0x7FFFFFFFll || slices > 0x7FFFFFFFll || tiles2d * slices > 0x7FFFFFFFll)
        return B2K_ERR_UNSUPPORTED;  // the kernel numbers tiles in 31 bits
    const int64_t tiles = tiles2d * slices;
    constexpr int SMEM = (NSTAGE + NOUT) * R * 128 + NSTAGE * 8 + 1024;
    auto kernel = transpose_tma_batched_kernel<ES, R, NSTAGE, THREADS, NOUT>;
    static b2k::PerDeviceOnce once;
    const cudaError_t attr_status = once.run([&] {
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    });
    if (attr_status != cudaSuccess) return b2k::check_cuda(attr_status, "transpose smem attribute");
    const int per_sm = B2K_ENV_INT("B2K_TRANSPOSE_CTAS_PER_SM", 2);
    int64_t grid = static_cast<int64_t>(b2k::sm_count()) * (per_sm < 1 ? 1 : per_sm);
    if (grid > tiles) grid = tiles;
    int panel_w = B2K_ENV_INT("B2K_TRANSPOSE_PANEL", 4);
    if (panel_w < 1 || panel_w > tiles_x) panel_w = static_cast<int>(tiles_x);
    const TileOrder order{static_cast<int>(tiles_x), static_cast<int>(tiles_y), panel_w};
    const int64_t adv_slices = grid / tiles2d;
    const BatchSplit bs{static_cast<unsigned int>(tiles2d),
                        static_cast<unsigned int>(batch_len[0]),
                        static_cast<unsigned int>(batch_len[1]),
                        static_cast<unsigned int>(grid % tiles2d),
                        static_cast<unsigned int>(adv_slices % batch_len[0]),
                        static_cast<unsigned int>(adv_slices / batch_len[0] % batch_len[1]),
                        static_cast<unsigned int>(adv_slices / batch_len[0] / batch_len[1])};
    // (the refill thread, always 0 here, is a kernel argument for the same reason as in launch())
    kernel<<<static_cast<unsigned>(grid), THREADS, SMEM, stream>>>(in_map, out_map, order, bs,
                                                                   static_cast<long long>(tiles), 0);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("batched transpose (tma) launch");
    return B2K_OK;
}

}  // namespace

namespace b2k {

int transpose_tma(const void *in, void *out, int64_t rows, int64_t cols, int64_t in_stride0, int64_t in_stride1,
                  int64_t out_stride0, int64_t out_stride1, int64_t itemsize, cudaStream_t stream) {
    if (itemsize != 1 && itemsize != 2 && itemsize != 4 && itemsize != 8 && itemsize != 16)
        return B2K_ERR_UNSUPPORTED;
    // tensor-map rules: contiguous lines, 16-byte aligned bases and pitches
    if (in_stride1 != itemsize || out_stride1 != itemsize) return B2K_ERR_UNSUPPORTED;
    if (!aligned_to<void>(in, 16) || !aligned_to<void>(out, 16)) return B2K_ERR_UNSUPPORTED;
    if (in_stride0 % 16 != 0 || out_stride0 % 16 != 0) return B2K_ERR_UNSUPPORTED;
    if (in_stride0 < cols * itemsize || out_stride0 < rows * itemsize) return B2K_ERR_UNSUPPORTED;
    if (in_stride0 >= (int64_t(1) << 40) || out_stride0 >= (int64_t(1) << 40)) return B2K_ERR_UNSUPPORTED;
    if (rows * (itemsize >= 4 ? itemsize / 4 : 1) >= (int64_t(1) << 31) ||
        cols * (itemsize >= 4 ? itemsize / 4 : 1) >= (int64_t(1) << 31))
        return B2K_ERR_UNSUPPORTED;
    // small arrays: the general tile kernel has less fixed cost
    if (rows * cols * itemsize < B2K_ENV_INT("B2K_TRANSPOSE_TMA_MIN_BYTES", 1 << 16)) return B2K_ERR_UNSUPPORTED;
    // Single bytes on lines that are multiples of 64 bytes run 10-18 % faster through
    // the stacked kernel with an empty stack (its issuing thread reads the coordinates
    // of the tile to store from shared memory instead of recomputing them, which
    // counts when the tile itself takes few instructions); measured slower for wider
    // items and for other pitches.
    if (itemsize == 1 && in_stride0 % 64 == 0 && out_stride0 % 64 == 0)
        return transpose_tma_batched(in, out, rows, cols, in_stride0, out_stride0, 0, nullptr, nullptr, nullptr,
                                     itemsize, stream);
    switch (itemsize) {
    case 1: return launch<1, 64, 4>(in, out, rows, cols, in_stride0, out_stride0, stream);
    case 2: return launch<2, 64, 4>(in, out, rows, cols, in_stride0, out_stride0, stream);
    case 4: return launch<4, 64, 4>(in, out, rows, cols, in_stride0, out_stride0, stream);
    case 8: return launch<8, 64, 4>(in, out, rows, cols, in_stride0, out_stride0, stream);
    default: return launch<16, 64, 4>(in, out, rows, cols, in_stride0, out_stride0, stream);
    }
}


// out[b..., j, i] = in[b..., i, j] for up to three batch axes with their own byte
// steps on each side; rows of both sides contiguous.  B2K_ERR_UNSUPPORTED when the
// tensor-map rules (16-byte alignment of bases, pitches and steps) do not hold.
int transpose_tma_batched(const void *in, void *out, int64_t rows, int64_t cols, int64_t in_pitch,
                          int64_t out_pitch, int nbatch, const int64_t *batch_len, const int64_t *in_batch_step,
                          const int64_t *out_batch_step, int64_t itemsize, cudaStream_t stream) {
    if (itemsize != 1 && itemsize != 2 && itemsize != 4 && itemsize != 8 && itemsize != 16)
        return B2K_ERR_UNSUPPORTED;
    if (nbatch < 0 || nbatch > 3) return B2K_ERR_UNSUPPORTED;
    if (!aligned_to<void>(in, 16) || !aligned_to<void>(out, 16)) return B2K_ERR_UNSUPPORTED;
    const int64_t limit = int64_t(1) << 40;
    if (in_pitch % 16 != 0 || out_pitch % 16 != 0 || in_pitch <= 0 || out_pitch <= 0 || in_pitch >= limit ||
        out_pitch >= limit)
        return B2K_ERR_UNSUPPORTED;
    if (in_pitch < cols * itemsize || out_pitch < rows * itemsize) return B2K_ERR_UNSUPPORTED;
    const int64_t words = itemsize >= 4 ? itemsize / 4 : 1;
    if (rows * words >= (int64_t(1) << 31) || cols * words >= (int64_t(1) << 31)) return B2K_ERR_UNSUPPORTED;
    int64_t len[3] = {1, 1, 1}, istep[3] = {in_pitch, in_pitch, in_pitch}, ostep[3] = {out_pitch, out_pitch, out_pitch};
    for (int k = 0; k < nbatch; ++k) {
        if (batch_len[k] < 1 || batch_len[k] >= (int64_t(1) << 31)) return B2K_ERR_UNSUPPORTED;
        if (in_batch_step[k] <= 0 || out_batch_step[k] <= 0 || in_batch_step[k] % 16 != 0 ||
            out_batch_step[k] % 16 != 0 || in_batch_step[k] >= limit || out_batch_step[k] >= limit)
            return B2K_ERR_UNSUPPORTED;
        len[k] = batch_len[k];
        istep[k] = in_batch_step[k];
        ostep[k] = out_batch_step[k];
    }
    switch (itemsize) {
    case 1: return launch_batched<1, 64, 4>(in, out, rows, cols, in_pitch, out_pitch, len, istep, ostep, stream);
    case 2: return launch_batched<2, 64, 4>(in, out, rows, cols, in_pitch, out_pitch, len, istep, ostep, stream);
    case 4: return launch_batched<4, 64, 4>(in, out, rows, cols, in_pitch, out_pitch, len, istep, ostep, stream);
    case 8: return launch_batched<8, 64, 4>(in, out, rows, cols, in_pitch, out_pitch, len, istep, ostep, stream);
    default: return launch_batched<16, 64, 4>(in, out, rows, cols, in_pitch, out_pitch, len, istep, ostep, stream);
    }
}

}  // namespace b2k

// Number of bounded waits that ran out in TMA transpose kernels on the current
// device since the library was loaded (0 in a healthy run).  Synchronises.
extern "C" B2K_API int b2k_transpose_wait_timeouts(unsigned int *count_out) {
    if (!count_out) return b2k::fail(B2K_ERR_INVALID_ARG, "null output");
    return b2k::check_cuda(cudaMemcpyFromSymbol(count_out, g_wait_timeouts, sizeof(unsigned int)),
                           "b2k_transpose_wait_timeouts");
}
