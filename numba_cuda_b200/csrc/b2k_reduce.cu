// Single-launch full reduction of a 1-D array with a table op.
//
// Replaces the reference's three-launch schedule (numba/cuda/kernels/
// reduction.py:233-258: full blocks -> tail block -> fold of <=65 partials, with
// only 64x128 threads and scalar loads) by one persistent-grid kernel:
//
//   * every CTA step folds one contiguous chunk of 32-byte vectors (256-bit
//     loads), UNROLL independent loads in flight per thread, one accumulator
//     per slot; CTAs stride over chunks;
//   * lanes combine with a shuffle butterfly, warps through shared memory;
//   * each block publishes its partial, then takes a ticket (atomicInc that
//     wraps to zero by itself); the block that draws the last ticket folds all
//     partials in index order, folds `init` in and writes the result.
//
// The fold order depends only on (n, grid size), so floating-point results are
// reproducible run to run.  HBM roofline: sizeof(T) bytes read per element.
#include <cstring>
#include <mutex>
#include <type_traits>

#include "b2k_internal.cuh"
#include "b2k_reduce_ops.cuh"

namespace {

using namespace b2k_reduce_ops;

constexpr int kThreads = 512;
constexpr int kUnroll = 4;
constexpr int kMaxGrid = 4096;
constexpr int kTicketBytes = 256;  // control words, padded so partials stay 256-B aligned
// Scratch layout.  Bytes 0..255: ticket of set 0 at byte 0 and of set 1 at byte 4; at
// bytes 64 and 72 the 64-bit "read" markers of the two sets (cross-GPU calls only).
// Then kMaxGrid 8-byte partial slots of set 0, then those of set 1.  Plain reductions
// use set 0 alone and need only the first half of the buffer.
constexpr int kSetBytes = 8 * kMaxGrid;
constexpr int kScratchPlain = kTicketBytes + kSetBytes;
constexpr int kScratchFull = kTicketBytes + 2 * kSetBytes;

// Block-wide fold; the result is valid in thread 0.  `slots` holds one T per warp.
template <typename T, typename Op, int THREADS>
__device__ __forceinline__ T block_fold(T v, T *slots) {
    constexpr int WARPS = THREADS / 32;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = Op::template apply<T>(v, shuffle_xor(v, m));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) slots[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = (lane < WARPS) ? slots[lane] : Op::template identity<T>();
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) v = Op::template apply<T>(v, shuffle_xor(v, m));
    }
    __syncthreads();
    return v;
}

// Every CTA step folds one contiguous chunk of THREADS*UNROLL 32-byte vectors
// (sm_100 has 256-bit global loads), so the CTAs in flight sweep one contiguous
// window of the array.
struct alignas(32) Bits256 { uint4 lo, hi; };

__device__ __forceinline__ Bits256 load_stream32(const Bits256 *p) {
    Bits256 r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.lo.x), "=r"(r.lo.y), "=r"(r.lo.z), "=r"(r.lo.w), "=r"(r.hi.x), "=r"(r.hi.y),
                   "=r"(r.hi.z), "=r"(r.hi.w)
                 : "l"(p));
    return r;
}

// ---- cross-GPU combine inside the kernel ------------------------------------------
// When the array is sharded over several GPUs of one NVLink domain, the block that
// finishes a GPU's local fold also does the exchange: it stores its value into a
// mailbox in every peer's memory (plain peer stores over NVLink), waits until every
// peer's value for this call has arrived in its own mailbox, and folds the values in
// rank order.  No second launch and no library collective.
//
// A value travels as 64-bit words that each carry 32 bits of payload under a 32-bit tag
// of the call's epoch (epoch mod (2^32 - 1), plus one: never zero, and different for
// epochs two apart): {tag, value bits 31..0} and, for 8-byte items, {tag, value bits
// 63..32}.  A 64-bit store is single-copy atomic, so a word that
// shows this call's epoch also shows its payload: no separate flag, and no release
// fence between a value and its flag (a fence at system scope has to wait for the
// remote write to be acknowledged -- a full NVLink round trip before the flag could
// even leave).  The cost of the exchange is one one-way trip of one or two stores.
// Mailboxes are double-buffered by epoch parity, so nothing is ever reset; a peer can
// be at most one call ahead (it cannot finish call k+1 before this rank has published
// k+1).  The wait is bounded: when it runs out the block records an error status,
// writes the identity-folded result and returns.
//
// Pipelining across calls.  Ticket and partial slots exist twice and a cross-GPU call
// uses the set of its epoch's parity.  The block that folds a set's partials then
// publishes "set read by call e" in that set's marker, and a CTA of call e+2 checks the
// marker (a bounded wait that is normally satisfied at once) before it writes its
// partial.  With B2K_REDUCE_INPUT_READY this is the only thing an ordinary CTA waits
// for: it does not wait for the preceding kernel at all, so its SM slot is free again as
// soon as its own loads are done, and only the ONE block that runs the exchange waits
// for the preceding call to complete (mailboxes and result stay in stream order).  A
// rank that is late therefore stalls one block per call in flight on its peers, not
// their loads: every GPU streams at its own pace and the ranks meet in the tails.
constexpr int kMaxPeers = 16;
constexpr int kMailboxWords = 2 * kMaxPeers * 2;  // [parity][writer]{low word, high word}

// Folds the eight words of a 32-byte vector into a word of running results.
template <typename T, typename Op>
__device__ __forceinline__ uint32_t fold_words(uint32_t acc, const Bits256 &raw) {
    acc = apply_word<T, Op>(acc, apply_word<T, Op>(raw.lo.x, raw.lo.y));
    acc = apply_word<T, Op>(acc, apply_word<T, Op>(raw.lo.z, raw.lo.w));
    acc = apply_word<T, Op>(acc, apply_word<T, Op>(raw.hi.x, raw.hi.y));
    acc = apply_word<T, Op>(acc, apply_word<T, Op>(raw.hi.z, raw.hi.w));
    return acc;
}

struct PeerLink {
    unsigned long long *mailbox[kMaxPeers];  // mailbox of every rank (own one included)
    int world;
    int rank;
    unsigned long long epoch;               // same on every rank for one call: 1, 2, 3, ...
    unsigned long long tag;                 // ((epoch mod (2^32 - 1)) + 1) << 32
    unsigned long long *marker;             // "read by call e" word of this call's scratch set
    unsigned long long timeout_ns;
    // [0] = 1 when a wait ran out; [1], [2] = %globaltimer (ns) when this GPU's local fold
    // was complete and when every peer's value had been seen
    unsigned long long *status;
};

__device__ __forceinline__ void store_relaxed_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long load_relaxed_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_release_gpu(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long load_acquire_gpu(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Runs in the last block of a GPU.  `local` is valid in thread 0.  Returns the fold
// over all ranks (valid in thread 0).  Thread p talks to rank p.
template <typename T, typename Op, int THREADS>
__device__ __forceinline__ T exchange_with_peers(T local, const PeerLink &link) {
    constexpr int WORDS = sizeof(T) > 4 ? 2 : 1;
    __shared__ unsigned long long mine_bits;
    __shared__ unsigned long long peer_bits[kMaxPeers];
    __shared__ int all_arrived;
    if (threadIdx.x == 0) {
        unsigned long long b = 0;
        memcpy(&b, &local, sizeof(T));
        mine_bits = b;
        all_arrived = 1;
        link.status[1] = global_timer_ns();
    }
    __syncthreads();
    const int slot_base = static_cast<int>(link.epoch & 1ull) * kMaxPeers;
    const unsigned long long tag = link.tag;
    if (threadIdx.x < link.world) {
        const int p = threadIdx.x;
        // publish to rank p (this rank's own mailbox included: one code path)
        unsigned long long *theirs = link.mailbox[p] + 2 * (slot_base + link.rank);
        store_relaxed_sys(theirs, tag | (mine_bits & 0xFFFFFFFFull));
        if (WORDS == 2) store_relaxed_sys(theirs + 1, tag | (mine_bits >> 32));
        // collect from rank p: spin for the first microseconds (the values of ranks
        // that run in step arrive within one NVLink trip), then back off
        const unsigned long long *here = link.mailbox[link.rank] + 2 * (slot_base + p);
        unsigned long long w0 = 0, w1 = tag;
        unsigned long long t0 = 0;
        bool arrived = false;
        for (unsigned int spin = 0;; ++spin) {
            w0 = load_relaxed_sys(here);
            if (WORDS == 2) w1 = load_relaxed_sys(here + 1);
            if ((w0 >> 32) == (tag >> 32) && (w1 >> 32) == (tag >> 32)) { arrived = true; break; }
            if (spin == 64) t0 = global_timer_ns();
            if (spin > 64) {
                if (global_timer_ns() - t0 > link.timeout_ns) break;
                __nanosleep(spin < 4096 ? 20 : 200);
            }
        }
        if (arrived) peer_bits[p] = (w0 & 0xFFFFFFFFull) | (WORDS == 2 ? (w1 << 32) : 0ull);
        else atomicExch(&all_arrived, 0);
    }
    __syncthreads();
    T result = Op::template identity<T>();
    if (threadIdx.x == 0) {
        link.status[2] = global_timer_ns();
        if (all_arrived) {
            for (int p = 0; p < link.world; ++p) {
                T v;
                memcpy(&v, &peer_bits[p], sizeof(T));
                result = Op::template apply<T>(result, v);
            }
        } else {
            link.status[0] = 1;
        }
    }
    return result;
}

template <typename T, typename Op, int THREADS, int UNROLL, bool PEER>
__global__ void __launch_bounds__(THREADS)
reduce_kernel(const T *__restrict__ x, int64_t n, T init, T *__restrict__ out,
              T *partials, unsigned int *ticket, const int input_ready, const PeerLink link) {
    constexpr int VEC = 32 / sizeof(T);
    __shared__ T slots[THREADS / 32];
    __shared__ bool is_last;

    // Programmatic dependent launch: the next kernel on the stream may be scheduled
    // as soon as every CTA of this one has started, and then waits below for this
    // kernel to complete, with its memory visible, before it touches anything this
    // kernel may still write.  When the caller has promised that the input was
    // complete before the preceding kernel began (input_ready), that wait moves
    // behind the load loop: the reads of reduction k+1 then overlap the last block
    // (and the cross-GPU exchange) of reduction k, and only the scratch, the mailboxes
    // and the result are touched in stream order.  In a cross-GPU call the scratch is
    // double-buffered and guarded by its own marker, so there only the block that runs
    // the exchange waits for the predecessor (see the notes on pipelining above).  Both
    // instructions do nothing in a launch without the programmatic attribute.
    asm volatile("griddepcontrol.launch_dependents;");
    if (!input_ready) asm volatile("griddepcontrol.wait;" ::: "memory");
    // cross-GPU calls: the marker that frees this call's scratch set is normally in place
    // long before the kernel starts; looking at it now keeps that round trip to L2 off the
    // end of the CTA's life
    unsigned long long marker_seen = 0;
    if constexpr (PEER) {
        if (threadIdx.x == 0) marker_seen = load_acquire_gpu(link.marker);
    }

    const uintptr_t addr = reinterpret_cast<uintptr_t>(x);
    int64_t head = static_cast<int64_t>(((32u - (addr & 31u)) & 31u) / sizeof(T));
    if (head > n) head = n;
    const Bits256 *xv = reinterpret_cast<const Bits256 *>(x + head);
    const int64_t nvec = (n - head) / VEC;
    const int64_t tail_begin = head + nvec * VEC;
    constexpr int64_t CHUNK = static_cast<int64_t>(THREADS) * UNROLL;
    const int64_t nchunks = nvec / CHUNK;

    T acc[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) acc[u] = Op::template identity<T>();

    if constexpr (WordWise<T, Op>::value) {
        // 8- and 16-bit integers: every slot keeps a word of four / two running results
        // and folds the vectors a word at a time; the items meet after the loops
        uint32_t packed[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) packed[u] = identity_word<T, Op>();
        for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
            const Bits256 *p = xv + c * CHUNK + threadIdx.x;
            Bits256 raw[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) raw[u] = load_stream32(p + u * THREADS);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) packed[u] = fold_words<T, Op>(packed[u], raw[u]);
        }
        for (int64_t v = nchunks * CHUNK + static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; v < nvec;
             v += static_cast<int64_t>(gridDim.x) * THREADS)
            packed[0] = fold_words<T, Op>(packed[0], load_stream32(xv + v));
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) acc[u] = fold_word<T, Op>(acc[u], packed[u]);
    } else {
        for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
            const Bits256 *p = xv + c * CHUNK + threadIdx.x;
            Bits256 raw[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) raw[u] = load_stream32(p + u * THREADS);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                acc[u] = fold_vector<T, Op>(acc[u], raw[u].lo);
                acc[u] = fold_vector<T, Op>(acc[u], raw[u].hi);
            }
        }
        // vectors past the last whole chunk, spread over the grid
        for (int64_t v = nchunks * CHUNK + static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; v < nvec;
             v += static_cast<int64_t>(gridDim.x) * THREADS) {
            const Bits256 raw = load_stream32(xv + v);
            acc[0] = fold_vector<T, Op>(acc[0], raw.lo);
            acc[0] = fold_vector<T, Op>(acc[0], raw.hi);
        }
    }
    if (input_ready && !PEER) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (blockIdx.x == 0) {  // fewer than 32 scalars on each side
        if (threadIdx.x < head) acc[0] = Op::template apply<T>(acc[0], x[threadIdx.x]);
        const int64_t t = tail_begin + threadIdx.x;
        if (t < n) acc[0] = Op::template apply<T>(acc[0], x[t]);
    }
#pragma unroll
    for (int u = 1; u < UNROLL; ++u) acc[0] = Op::template apply<T>(acc[0], acc[u]);

    T total = block_fold<T, Op, THREADS>(acc[0], slots);
    if (threadIdx.x == 0) {
        if constexpr (PEER) {
            // this set's partials were last used by the call two epochs back: they may be
            // overwritten once that call's folding block has read them
            const unsigned long long want = link.epoch > 2 ? link.epoch - 2 : 0;
            unsigned long long t0 = 0;
            for (unsigned int spin = 0; marker_seen < want; ++spin) {
                marker_seen = load_acquire_gpu(link.marker);
                if (marker_seen >= want) break;
                if (spin == 64) t0 = global_timer_ns();
                if (spin > 64) {
                    if (global_timer_ns() - t0 > link.timeout_ns) { link.status[0] = 2; break; }
                    __nanosleep(100);
                }
            }
        }
        partials[blockIdx.x] = total;
        // the ticket: an increment that wraps to zero with the last CTA.  It releases the
        // partial just written and acquires the partials of the CTAs that came before.
        unsigned int t;
        asm volatile("atom.acq_rel.gpu.global.inc.u32 %0, [%1], %2;"
                     : "=r"(t) : "l"(ticket), "r"(gridDim.x - 1) : "memory");
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();   // carries thread 0's acquire to the whole block
    if (!is_last) return;
    T mine = Op::template identity<T>();
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += THREADS)
        mine = Op::template apply<T>(mine, __ldcg(partials + i));
    total = block_fold<T, Op, THREADS>(mine, slots);
    if constexpr (PEER) {
        if (threadIdx.x == 0) store_release_gpu(link.marker, link.epoch);   // the set is free for call epoch + 2
        // from here on everything is in stream order: mailboxes, status, result
        if (input_ready) asm volatile("griddepcontrol.wait;" ::: "memory");
        total = exchange_with_peers<T, Op, THREADS>(total, link);
    }
    if (threadIdx.x == 0) out[0] = Op::template apply<T>(total, init);
}

template <typename T, typename Op>
int launch(const void *x, int64_t n, const void *init_host, void *out, void *scratch,
           cudaStream_t stream, const PeerLink *link, unsigned flags) {
    T init;
    memcpy(&init, init_host, sizeof(T));
    // two persistent CTAs per SM measured best on B200; short inputs get one CTA per chunk
    // (spreading an 8 MiB input over twice as many, smaller CTAs measured the same: that
    // case is bound by the fixed latencies of launch, ticket and last-block fold)
    const int per_sm = B2K_ENV_INT("B2K_REDUCE_CTAS_PER_SM", 2);
    int64_t max_grid = static_cast<int64_t>(b2k::sm_count()) * per_sm;
    if (max_grid > kMaxGrid) max_grid = kMaxGrid;
    const int64_t chunk_bytes = static_cast<int64_t>(kThreads) * kUnroll * 32;
    int64_t grid = (n * static_cast<int64_t>(sizeof(T)) + chunk_bytes - 1) / chunk_bytes;
    if (grid < 1) grid = 1;
    if (grid > max_grid) grid = max_grid;
    const int set = link ? static_cast<int>(link->epoch & 1ull) : 0;
    auto *ticket = static_cast<unsigned int *>(scratch) + set;
    auto *partials = reinterpret_cast<T *>(static_cast<char *>(scratch) + kTicketBytes + set * kSetBytes);
    PeerLink with_marker{};
    if (link) {
        with_marker = *link;
        with_marker.marker = reinterpret_cast<unsigned long long *>(static_cast<char *>(scratch) + 64) + set;
        link = &with_marker;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const bool pdl = B2K_ENV_INT("B2K_REDUCE_PDL", 1) != 0;
    cfg.numAttrs = pdl ? 1 : 0;
    const int input_ready = (pdl && (flags & B2K_REDUCE_INPUT_READY)) ? 1 : 0;
    // Pipelined launches leave one CTA slot of the GPU free: the last block of the
    // previous reduction is still folding its partials (and, across GPUs, waiting for
    // its peers) while this kernel's CTAs start.  With every slot claimed, one CTA of
    // this kernel would start only when that block is gone and, its chunks being fixed,
    // finish that much later than the rest.
    if (input_ready && grid == max_grid && grid > 1 && B2K_ENV_INT("B2K_REDUCE_SPARE_SLOT", 1) != 0) {
        grid -= 1;
        cfg.gridDim = dim3(static_cast<unsigned>(grid));
    }
    cudaError_t err;
    if (link) {
        err = cudaLaunchKernelEx(&cfg, reduce_kernel<T, Op, kThreads, kUnroll, true>, static_cast<const T *>(x), n,
                                 init, static_cast<T *>(out), partials, ticket, input_ready, *link);
    } else {
        err = cudaLaunchKernelEx(&cfg, reduce_kernel<T, Op, kThreads, kUnroll, false>, static_cast<const T *>(x), n,
                                 init, static_cast<T *>(out), partials, ticket, input_ready, PeerLink{});
    }
    if (err != cudaSuccess) return b2k::check_cuda(err, "b2k_reduce launch");
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_reduce launch");
    return B2K_OK;
}

template <typename T>
int dispatch_op(int op, const void *x, int64_t n, const void *init_host, void *out,
                void *scratch, cudaStream_t stream, const PeerLink *link, unsigned flags) {
    switch (op) {
    case B2K_ADD: return launch<T, OpAdd>(x, n, init_host, out, scratch, stream, link, flags);
    case B2K_MUL: return launch<T, OpMul>(x, n, init_host, out, scratch, stream, link, flags);
    case B2K_MAX: return launch<T, OpMax>(x, n, init_host, out, scratch, stream, link, flags);
    case B2K_MIN: return launch<T, OpMin>(x, n, init_host, out, scratch, stream, link, flags);
    default: break;
    }
    if constexpr (!(std::is_same<T, float>::value || std::is_same<T, double>::value)) {
        switch (op) {
        case B2K_AND: return launch<T, OpAnd>(x, n, init_host, out, scratch, stream, link, flags);
        case B2K_OR: return launch<T, OpOr>(x, n, init_host, out, scratch, stream, link, flags);
        case B2K_XOR: return launch<T, OpXor>(x, n, init_host, out, scratch, stream, link, flags);
        default: break;
        }
    }
    return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce: op %d is not defined for dtype", op);
}

size_t dtype_size(int dtype) {
    switch (dtype) {
    case B2K_I8: case B2K_U8: return 1;
    case B2K_I16: case B2K_U16: return 2;
    case B2K_I32: case B2K_U32: case B2K_F32: return 4;
    case B2K_I64: case B2K_U64: case B2K_F64: return 8;
    default: return 0;
    }
}

}  // namespace

extern "C" {

int64_t b2k_reduce_scratch_bytes(void) { return kScratchFull; }

static int reduce_impl(int op, int dtype, const void *x_dev, int64_t n, const void *init_host, void *out_dev,
                       void *scratch_dev, int64_t scratch_bytes, void *stream, const PeerLink *link,
                       unsigned flags) {
    const size_t size = dtype_size(dtype);
    if (size == 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce: unknown dtype %d", dtype);
    if (op < B2K_ADD || op > B2K_XOR) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce: unknown op %d", op);
    if (n < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce: negative length %lld", (long long)n);
    if (!init_host || !out_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce: null init or out");
    if (n > 0 && !x_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce: null input with n > 0");
    // cross-GPU calls use both halves of the buffer, plain ones the first half only
    const int64_t scratch_needed = link ? kScratchFull : kScratchPlain;
    if (!scratch_dev || scratch_bytes < scratch_needed)
        return b2k::fail(B2K_ERR_SCRATCH, "b2k_reduce: scratch of %lld bytes required", (long long)scratch_needed);
    if (!b2k::aligned_to<void>(x_dev, size) || !b2k::aligned_to<void>(out_dev, size))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_reduce: pointers must be aligned to the element size");
    if (!b2k::aligned_to<void>(scratch_dev, 256))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_reduce: scratch must be 256-byte aligned");
    cudaStream_t s = b2k::as_stream(stream);
    switch (dtype) {
    case B2K_I8: return dispatch_op<int8_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_I16: return dispatch_op<int16_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_I32: return dispatch_op<int32_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_I64: return dispatch_op<int64_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_U8: return dispatch_op<uint8_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_U16: return dispatch_op<uint16_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_U32: return dispatch_op<uint32_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_U64: return dispatch_op<uint64_t>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    case B2K_F32: return dispatch_op<float>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    default: return dispatch_op<double>(op, x_dev, n, init_host, out_dev, scratch_dev, s, link, flags);
    }
}


int b2k_reduce(int op, int dtype, const void *x_dev, int64_t n, const void *init_host,
               void *out_dev, void *scratch_dev, int64_t scratch_bytes, void *stream) {
    B2K_RANGE("b2k_reduce");
    return reduce_impl(op, dtype, x_dev, n, init_host, out_dev, scratch_dev, scratch_bytes, stream, nullptr, 0u);
}

int b2k_reduce_ex(int op, int dtype, const void *x_dev, int64_t n, const void *init_host, void *out_dev,
                  void *scratch_dev, int64_t scratch_bytes, unsigned flags, void *stream) {
    B2K_RANGE("b2k_reduce_ex");
    if (flags & ~static_cast<unsigned>(B2K_REDUCE_INPUT_READY))
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_ex: unknown flag bits 0x%x", flags);
    return reduce_impl(op, dtype, x_dev, n, init_host, out_dev, scratch_dev, scratch_bytes, stream, nullptr, flags);
}

// ---- mailboxes for the in-kernel cross-GPU combine -----------------------------------
int64_t b2k_peer_mailbox_bytes(void) { return kMailboxWords * 8; }
int b2k_peer_max_world(void) { return kMaxPeers; }
int64_t b2k_peer_handle_bytes(void) { return static_cast<int64_t>(sizeof(cudaIpcMemHandle_t)); }

int b2k_peer_mailbox_create(void **mailbox_dev) {
    if (!mailbox_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_peer_mailbox_create: null output");
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, kMailboxWords * 8);
    if (e != cudaSuccess) return b2k::check_cuda(e, "b2k_peer_mailbox_create: cudaMalloc");
    e = cudaMemset(p, 0, kMailboxWords * 8);
    if (e != cudaSuccess) { cudaFree(p); return b2k::check_cuda(e, "b2k_peer_mailbox_create: cudaMemset"); }
    *mailbox_dev = p;
    return B2K_OK;
}
int b2k_peer_mailbox_destroy(void *mailbox_dev) {
    return b2k::check_cuda(cudaFree(mailbox_dev), "b2k_peer_mailbox_destroy");
}
int b2k_peer_mailbox_export(void *mailbox_dev, void *handle_out) {
    if (!mailbox_dev || !handle_out) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_peer_mailbox_export: null pointer");
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, mailbox_dev);
    if (e != cudaSuccess) return b2k::check_cuda(e, "b2k_peer_mailbox_export: cudaIpcGetMemHandle");
    memcpy(handle_out, &h, sizeof h);
    return B2K_OK;
}
int b2k_peer_mailbox_open(const void *handle, void **peer_mailbox_dev) {
    if (!handle || !peer_mailbox_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_peer_mailbox_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return b2k::check_cuda(e, "b2k_peer_mailbox_open: cudaIpcOpenMemHandle");
    *peer_mailbox_dev = p;
    return B2K_OK;
}
int b2k_peer_mailbox_close(void *peer_mailbox_dev) {
    return b2k::check_cuda(cudaIpcCloseMemHandle(peer_mailbox_dev), "b2k_peer_mailbox_close");
}

int b2k_reduce_peer(int op, int dtype, const void *x_dev, int64_t n, const void *init_host, void *out_dev,
                    void *scratch_dev, int64_t scratch_bytes, void *const *mailboxes, int world, int rank,
                    uint64_t epoch, uint64_t timeout_ns, void *status_dev, unsigned flags, void *stream) {
    B2K_RANGE("b2k_reduce_peer");
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_peer: world %d / rank %d out of range (at most %d ranks)",
                         world, rank, kMaxPeers);
    if (!mailboxes || !status_dev || epoch == 0)
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_peer: null mailboxes/status or epoch 0");
    if (!b2k::aligned_to<void>(status_dev, 8))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_reduce_peer: status must be 8-byte aligned");
    if (flags & ~static_cast<unsigned>(B2K_REDUCE_INPUT_READY))
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_peer: unknown flag bits 0x%x", flags);
    PeerLink link{};
    for (int p = 0; p < world; ++p) {
        if (!mailboxes[p] || !b2k::aligned_to<void>(mailboxes[p], 16))
            return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_peer: mailbox of rank %d missing or unaligned", p);
        link.mailbox[p] = static_cast<unsigned long long *>(mailboxes[p]);
    }
    link.world = world;
    link.rank = rank;
    link.epoch = epoch;
    link.tag = ((epoch % 0xFFFFFFFFull) + 1ull) << 32;
    link.timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
    link.status = static_cast<unsigned long long *>(status_dev);
    return reduce_impl(op, dtype, x_dev, n, init_host, out_dev, scratch_dev, scratch_bytes, stream, &link, flags);
}

}  // extern "C"

// ---- entry point that allocates nothing ------------------------------------------
//
// Some hosts may not allocate device memory at the point where they need a
// reduction: a numba-cuda process whose device memory is owned by an external
// memory-manager plugin (every byte has to come from that pool, and the pool may
// already be fully handed out), a C caller that holds nothing but its input and
// output buffers, or a latency-critical loop that cannot take the device-wide
// synchronisation an allocation or a free can imply.  For them the ticket and
// the block partials live in the fixed array below instead of caller scratch.
//
// In host code the array's name stands for the symbol, not for an address the
// GPU understands; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) unsigned char g_reduce_static_scratch[kScratchPlain];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void *g_static_address[kMaxDevices];  // device address of the array, per device ordinal

int static_scratch_of_current_device(void **address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return b2k::check_cuda(e, "b2k_reduce_noalloc: cudaGetDevice");
    if (device < 0 || device >= kMaxDevices)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_noalloc: device ordinal %d not supported", device);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_address[device] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_reduce_static_scratch);
        if (e != cudaSuccess) return b2k::check_cuda(e, "b2k_reduce_noalloc: cudaGetSymbolAddress");
        if (p == nullptr) return b2k::fail(B2K_ERR_SCRATCH, "b2k_reduce_noalloc: no device address for the scratch array");
        g_static_address[device] = p;
    }
    *address = g_static_address[device];
    return B2K_OK;
}

}  // namespace

extern "C" {

int64_t b2k_reduce_noalloc_max_elements(void) { return int64_t(1) << 32; }

int b2k_reduce_noalloc(int op, int dtype, const void *x_dev, int64_t n, const void *init_host,
                       void *out_dev, void *stream) {
    if (n > b2k_reduce_noalloc_max_elements())
        return b2k::fail(B2K_ERR_TOO_LARGE,
                         "b2k_reduce_noalloc: %lld elements exceed the limit of %lld for the built-in scratch; "
                         "use b2k_reduce with caller-provided scratch",
                         (long long)n, (long long)b2k_reduce_noalloc_max_elements());
    if (n < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_noalloc: negative length %lld", (long long)n);
    void *scratch = nullptr;
    const int rc = static_scratch_of_current_device(&scratch);
    if (rc != B2K_OK) return rc;
    // The array keeps whatever the previous call left.  Only the ticket word has
    // to start at zero (the kernel returns it to zero when it completes, but a
    // launch that failed half-way would not); partial slots are written before
    // they are read.
    const cudaError_t e = cudaMemsetAsync(scratch, 0, kTicketBytes, b2k::as_stream(stream));
    if (e != cudaSuccess) return b2k::check_cuda(e, "b2k_reduce_noalloc: clearing the ticket");
    return b2k_reduce(op, dtype, x_dev, n, init_host, out_dev, scratch, kScratchPlain, stream);
}

}  // extern "C"
