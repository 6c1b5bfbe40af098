/*
 * b2k.h -- C ABI of libb2k.so: sm_100a kernels behind numba-cuda's built-in
 * library kernels (cuda.reduce, device-array transpose, xoroshiro128p RNG,
 * bf16 / fp8 conversion).
 *
 * The reference has no FFI for this path: its library kernels are Python that is
 * JIT-compiled on first use.  Each entry point below names the reference code
 * whose device work it replaces (paths relative to the numba-cuda project root).
 *
 * Conventions
 *   - plain pointers and sizes only; `stream` is a cudaStream_t passed as void*
 *     (NULL = the legacy default stream);
 *   - every pointer named *_dev is device memory of the CURRENT device;
 *   - every call returns an int status: 0 = ok, negative = argument error found
 *     on the host before any launch (B2K_ERR_*), positive = a cudaError_t;
 *   - calls are asynchronous on `stream` and never synchronise;
 *   - scratch is passed in by the caller (sizes from the *_scratch_bytes
 *     functions); the library allocates device memory in one place only:
 *     b2k_peer_mailbox_create (512 bytes per communicator, synchronous);
 *   - b2k_last_error() gives a thread-local message for the last failure.
 */
#ifndef B2K_H_
#define B2K_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B2K_API __attribute__((visibility("default")))
#else
#define B2K_API
#endif

#define B2K_OK 0
#define B2K_ERR_INVALID_ARG (-1)   /* null pointer, negative size, bad enum        */
#define B2K_ERR_UNSUPPORTED (-2)   /* op/dtype pair or cast pair not implemented   */
#define B2K_ERR_ALIGNMENT (-3)     /* pointer not aligned to the element size      */
#define B2K_ERR_SCRATCH (-4)       /* scratch buffer missing or too small          */
#define B2K_ERR_TOO_LARGE (-5)     /* size beyond a stated maximum                 */

/* element types (reduce) */
enum b2k_dtype {
    B2K_I8 = 0, B2K_I16 = 1, B2K_I32 = 2, B2K_I64 = 3,
    B2K_U8 = 4, B2K_U16 = 5, B2K_U32 = 6, B2K_U64 = 7,
    B2K_F32 = 8, B2K_F64 = 9
};

/* binary ops (reduce): the table a user's Python functor is classified into */
enum b2k_op {
    B2K_ADD = 0, B2K_MUL = 1, B2K_MAX = 2, B2K_MIN = 3,
    B2K_AND = 4, B2K_OR = 5, B2K_XOR = 6
};

/* storage formats (cast) */
enum b2k_format {
    B2K_FMT_F32 = 0, B2K_FMT_BF16 = 1, B2K_FMT_E4M3 = 2, B2K_FMT_E5M2 = 3,
    B2K_FMT_F64 = 4, B2K_FMT_F16 = 5, B2K_FMT_E8M0 = 6,  /* b2k_cast_ex only */
    /* integer sides of b2k_cast_ex; BOOL is one byte holding 0 or 1 */
    B2K_FMT_I8 = 7, B2K_FMT_I16 = 8, B2K_FMT_I32 = 9, B2K_FMT_I64 = 10,
    B2K_FMT_U8 = 11, B2K_FMT_U16 = 12, B2K_FMT_U32 = 13, B2K_FMT_U64 = 14,
    B2K_FMT_BOOL = 15
};

/* rounding modes (b2k_cast_ex), numbered like cudaRoundMode */
enum b2k_rounding {
    B2K_ROUND_NEAREST = 0, B2K_ROUND_ZERO = 1, B2K_ROUND_POS_INF = 2, B2K_ROUND_MIN_INF = 3
};

/* draws (RNG fill) */
enum b2k_draw {
    B2K_UNIFORM_F32 = 0, B2K_UNIFORM_F64 = 1, B2K_NORMAL_F32 = 2, B2K_NORMAL_F64 = 3
};

B2K_API int b2k_version(void);
B2K_API const char *b2k_last_error(void);
/* number of kernels this library has launched in the calling process */
B2K_API int64_t b2k_launch_count(void);

/* ---- reduce -------------------------------------------------------------
 * Replaces the three launches + partials allocation of Reduce.__call__
 * (numba/cuda/kernels/reduction.py:194-265) and the kernel bodies
 * gpu_reduce_block_strided / device_reduce_full_block (:44-166) with ONE launch:
 * out_dev[0] = op(fold(x_dev[0..n)), *init_host).
 *   init_host : host pointer to one element of `dtype` (always folded in, as
 *               reduction.py:163-164 does)
 *   out_dev   : one element of `dtype`
 *   scratch   : b2k_reduce_scratch_bytes() bytes, zero-filled once by the caller
 *               before first use; the kernel leaves it reusable.  Two reductions
 *               that may overlap on the GPU need separate scratch.  (b2k_reduce,
 *               b2k_reduce_ex and b2k_reduce_expr touch only the first half of it.)
 * n == 0 writes *init_host to out_dev. */
B2K_API int64_t b2k_reduce_scratch_bytes(void);
B2K_API int b2k_reduce(int op, int dtype, const void *x_dev, int64_t n, const void *init_host,
               void *out_dev, void *scratch_dev, int64_t scratch_bytes, void *stream);

/* The same with flags.  The kernel is launched with the programmatic-dependent-launch
 * attribute; back-to-back reductions on one stream therefore overlap their launch
 * latencies, and results, scratch and mailboxes are still touched strictly in stream
 * order.
 *   B2K_REDUCE_INPUT_READY : the caller promises that x_dev[0..n) was complete before
 *       the kernel that precedes this call on the stream began (it is not produced or
 *       modified by that kernel -- in particular it does not contain the previous
 *       reduction's out_dev).  The reduction may then read its input while the tail
 *       of the preceding kernel (a reduction's last block, its cross-GPU exchange) is
 *       still running: a stream of independent reductions runs as a pipeline.
 *       Without the flag the kernel touches nothing before its predecessor is done. */
#define B2K_REDUCE_INPUT_READY 1u
B2K_API int b2k_reduce_ex(int op, int dtype, const void *x_dev, int64_t n, const void *init_host,
                          void *out_dev, void *scratch_dev, int64_t scratch_bytes, unsigned flags,
                          void *stream);

/* Reduction of a rows x cols matrix along one axis with a table op:
 *   axis 0: out_dev[j] = op(fold_i x[i, j], *init_host)   (cols outputs)
 *   axis 1: out_dev[i] = op(fold_j x[i, j], *init_host)   (rows outputs)
 * Rows are contiguous and `pitch_bytes` apart.  The reference reduces 1-D arrays
 * only (Reduce.__call__ raises TypeError("only support 1D array") otherwise,
 * numba/cuda/kernels/reduction.py:217-218); this is the axis-wise step after it,
 * with the ops, dtypes and wrap-around rules of b2k_reduce.  One launch.
 *   scratch : b2k_reduce_axis_scratch_bytes(rows, cols, dtype, axis) bytes (0 for
 *             most axis-1 shapes), 256-byte aligned, zero-filled once before first
 *             use; the kernel leaves it reusable for calls of the same or a smaller
 *             requirement.  Calls that may overlap on the GPU need separate scratch.
 * An empty reduced axis writes *init_host to every output. */
B2K_API int64_t b2k_reduce_axis_scratch_bytes(int64_t rows, int64_t cols, int dtype, int axis);
B2K_API int b2k_reduce_axis(int op, int dtype, const void *x_dev, int64_t rows, int64_t cols,
                            int64_t pitch_bytes, int axis, const void *init_host, void *out_dev,
                            void *scratch_dev, int64_t scratch_bytes, void *stream);

/* A batch of `batch` matrices (matrix_stride_bytes apart) reduced along axis 0 in ONE
 * launch: out_dev[b * cols + j] = op(fold_i x[b, i, j], *init_host).  This is the
 * reduction of the middle axis of a C-contiguous (batch, rows, cols) array, the step
 * after the 1-D reduce of numba/cuda/kernels/reduction.py:217-218 like b2k_reduce_axis.
 * batch <= 65535.  Scratch rules as for b2k_reduce_axis, size from
 * b2k_reduce_cols_batched_scratch_bytes. */
B2K_API int64_t b2k_reduce_cols_batched_scratch_bytes(int64_t batch, int64_t rows, int64_t cols, int dtype);
B2K_API int b2k_reduce_cols_batched(int op, int dtype, const void *x_dev, int64_t batch, int64_t rows,
                                    int64_t cols, int64_t pitch_bytes, int64_t matrix_stride_bytes,
                                    const void *init_host, void *out_dev, void *scratch_dev,
                                    int64_t scratch_bytes, void *stream);

/* cuda.reduce with an arbitrary user function.  `expr` is a C++ expression over
 * the operands `a` and `b` (the Python layer obtains it by tracing the user's
 * function); the reduce kernel is compiled around it at run time with NVRTC for
 * sm_100a and cached per (device, dtype, expression).  Replaces the reference's
 * JIT compilation of the functor (numba/cuda/kernels/reduction.py:15-21, :185-192).
 * Integer operands are widened to 64 bits inside the expression (`a` and `b` are
 * unsigned long long for unsigned items, long long for signed ones; B2K_ILIT gives a
 * long long, so the caller casts where numba's rule "signed if either side is" asks
 * for it) and truncated on store; float32 literals-with-integers promote to double.
 * Helpers available to the expression: b2k_floordiv, b2k_mod (Python semantics),
 * b2k_truediv, b2k_abs, B2K_ILIT(integer literal), B2K_INF, B2K_NAN.
 * n must be >= 1 (the caller returns init for an empty array).  init_host may be
 * NULL: the bare fold of the items is written (such a function has no identity
 * element, so partial results of shards are combined without one).  The op must be
 * associative and commutative, as the reference requires. */
B2K_API int b2k_reduce_expr(const char *expr, int dtype, const void *x_dev, int64_t n,
                            const void *init_host, void *out_dev, void *scratch_dev,
                            int64_t scratch_bytes, void *stream);

/* Reduce + cross-GPU combine in ONE kernel per GPU (no counterpart in the
 * reference, which has no distributed layer).  For an array sharded over up to
 * b2k_peer_max_world() GPUs of one NVLink domain: every rank calls
 * b2k_reduce_peer on its shard with the same `epoch` (1, 2, 3, ... without gaps, per
 * communicator and scratch buffer); the block that finishes the
 * local fold stores the rank's value into a mailbox in every peer's memory, waits
 * (at most timeout_ns, 0 = 2 s) for the peers' values of this epoch in its own
 * mailbox, folds them in rank order, folds *init_host in and writes out_dev[0] --
 * the same result on every rank.
 *   mailboxes : host array of `world` device pointers, entry r = rank r's mailbox
 *               as visible from this process (own: from b2k_peer_mailbox_create;
 *               others: b2k_peer_mailbox_open of the handle that rank exported).
 *   status_dev: three 64-bit words in device memory, 8-byte aligned.  [0] is set to
 *               1 when a peer's value did not arrive in time, 2 when a scratch set
 *               was not released in time (in the first case the kernel writes
 *               the fold of nothing but *init_host and returns: no hang; the other
 *               ranks may have completed normally, so after a timeout the ranks hold
 *               DIFFERENT results and have to agree on the host what to do).  [1] and
 *               [2] receive the GPU's nanosecond timer when the local fold was done
 *               and when the last peer value had been seen: their difference is what
 *               the exchange cost this rank, launch skew between the ranks included.
 *   scratch   : b2k_reduce_scratch_bytes() bytes, zero-filled once; it belongs to the
 *               communicator (all its calls, whatever the stream).  It holds two
 *               ticket/partial sets that alternate with the epoch, so two calls may
 *               overlap on the GPU; a third waits (bounded) for the first to let go.
 *   flags     : as for b2k_reduce_ex.  With B2K_REDUCE_INPUT_READY only the block
 *               that runs the exchange waits for the preceding kernel; the others
 *               free their SMs as soon as their loads are done, so a peer that is
 *               late does not stall this GPU's reads of the following calls.
 * The mailbox helpers allocate/map b2k_peer_mailbox_bytes() bytes once per
 * communicator; handles are b2k_peer_handle_bytes() bytes and travel between
 * processes by any host channel. */
B2K_API int64_t b2k_peer_mailbox_bytes(void);
B2K_API int64_t b2k_peer_handle_bytes(void);
B2K_API int b2k_peer_max_world(void);
B2K_API int b2k_peer_mailbox_create(void **mailbox_dev);
B2K_API int b2k_peer_mailbox_destroy(void *mailbox_dev);
B2K_API int b2k_peer_mailbox_export(void *mailbox_dev, void *handle_out);
B2K_API int b2k_peer_mailbox_open(const void *handle, void **peer_mailbox_dev);
B2K_API int b2k_peer_mailbox_close(void *peer_mailbox_dev);
B2K_API int b2k_reduce_peer(int op, int dtype, const void *x_dev, int64_t n, const void *init_host,
                            void *out_dev, void *scratch_dev, int64_t scratch_bytes,
                            void *const *mailboxes, int world, int rank, uint64_t epoch,
                            uint64_t timeout_ns, void *status_dev, unsigned flags, void *stream);

/* The same reduction for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.  Meant for hosts whose device memory belongs to
 * someone else at the time of the call (a numba-cuda process running under an
 * external memory-manager plugin whose pool is already handed out), for plain C
 * callers that hold only an input and an output buffer, and for loops that
 * cannot afford the device-wide synchronisation an allocation or free may cause.
 * The ticket and the block partials live in an array that is compiled into the
 * library (33,024 bytes, held by every GPU that loads the library until the
 * process exits); the call itself performs no cudaMalloc / cudaFree and calls no
 * allocating routine.
 *   - n may be at most b2k_reduce_noalloc_max_elements() (2^32); larger inputs
 *     are refused with B2K_ERR_TOO_LARGE -- use b2k_reduce with your own scratch.
 *   - The first call on each device looks up the array's device address (that
 *     device must be current); make that first call before starting any stream
 *     capture.
 *   - All calls on a device share the one array: two calls that may run on the
 *     GPU at the same time (different streams, different threads) race and give
 *     wrong results.  Calls ordered on one stream are fine; each call clears the
 *     part of the array that must start at zero. */
B2K_API int64_t b2k_reduce_noalloc_max_elements(void);
B2K_API int b2k_reduce_noalloc(int op, int dtype, const void *x_dev, int64_t n, const void *init_host,
                               void *out_dev, void *stream);

/* ---- transpose ----------------------------------------------------------
 * Replaces the per-call JIT-compiled tile kernel of
 * numba/cuda/kernels/transpose.py:42-63: out[j, i] = in[i, j] for items of
 * `itemsize` bytes; strides are in bytes and arbitrary for both arrays. */
B2K_API int b2k_transpose2d(const void *in_dev, void *out_dev, int64_t rows, int64_t cols,
                    int64_t in_stride0, int64_t in_stride1,
                    int64_t out_stride0, int64_t out_stride1,
                    int64_t itemsize, void *stream);

/* Diagnostic: how many bounded waits of the TMA transpose kernels have run out on the
 * current device since the library was loaded (0 in a healthy run; a kernel whose
 * wait runs out counts it, drains its copies and returns instead of hanging).
 * Synchronises the device. */
B2K_API int b2k_transpose_wait_timeouts(unsigned int *count_out);

/* ---- strided assignment --------------------------------------------------
 * Replaces the per-ndim JIT-compiled element kernel behind
 * DeviceNDArray.__setitem__ (numba/cuda/cudadrv/devicearray.py:535-576, launched
 * at :735-791): dst[i0, .., ik] = src[i0', .., ik'] over a common `shape`, where a
 * source stride of 0 repeats the source along that axis (the reference's
 * "rhs.shape[i] > 1" factor).  Strides are in bytes, may be negative, and are
 * arbitrary for both sides, so the same call also materialises axis permutations
 * (N-D transposes) and copies between differently laid out arrays.  The two sides
 * must not overlap.  ndim <= 32; at most 8 axes may remain after the library has
 * merged axes that are contiguous on both sides. */
B2K_API int b2k_assign(void *dst_dev, const void *src_dev, int ndim, const int64_t *shape,
                       const int64_t *dst_strides, const int64_t *src_strides, int64_t itemsize,
                       void *stream);
/* The same with ONE source item of 1..16 bytes read from host memory at call time
 * and carried to the kernel in its parameters (d_arr[key] = scalar): no staging
 * copy, nothing for the caller to keep alive. */
B2K_API int b2k_fill(void *dst_dev, int ndim, const int64_t *shape, const int64_t *dst_strides,
                     const void *value_host, int64_t itemsize, void *stream);

/* ---- xoroshiro128p ------------------------------------------------------
 * b2k_xoroshiro128p_init replaces init_xoroshiro128p_states_cpu + the H2D copy
 * (numba/cuda/random.py:242-282): states[i] = jump^(subsequence_start+i)(seed
 * state), computed on the device in parallel.
 *   tables_dev : b2k_xoroshiro128p_tables_bytes() bytes filled once per device
 *                by b2k_xoroshiro128p_build_tables (seed-independent).          */
B2K_API int64_t b2k_xoroshiro128p_tables_bytes(void);
B2K_API int b2k_xoroshiro128p_build_tables(void *tables_dev, int64_t tables_bytes, void *stream);
B2K_API int b2k_xoroshiro128p_init(void *states_dev, int64_t n, uint64_t seed,
                           uint64_t subsequence_start, const void *tables_dev,
                           int64_t tables_bytes, void *stream);

/* One bulk "user kernel" in the layout of the reference's test kernels
 * (numba/cuda/tests/cudapy/test_random.py:29-53): for every generator t in
 * [0, n): out[t*count + i] = draw(states, t), i in [0, count); states are
 * advanced in place.  Replaces the device functions
 * xoroshiro128p_{uniform,normal}_float{32,64} (random.py:160-238) inlined in a
 * caller's kernel.  Up to two segments are generated back to back per
 * generator (segment 1 may be NULL / count 0), so that e.g. 64 uniform f32
 * followed by 16 normal f64 costs one state round trip. */
B2K_API int b2k_xoroshiro128p_fill(void *states_dev, int64_t n,
                           int draw0, void *out0_dev, int64_t count0,
                           int draw1, void *out1_dev, int64_t count1, void *stream);

/* ---- casts --------------------------------------------------------------
 * Bulk elementwise conversion with the semantics of the conversion intrinsics
 *   f32 -> e4m3/e5m2 : cvt_float_to_fp8(x, saturate, interp)
 *                      (numba/cuda/_internal/cuda_fp8.py:3341-3374;
 *                       include/12/cuda_fp8.hpp:245-288)
 *   e4m3/e5m2 -> f32 : float(fp8_e4m3(code)) (cuda_fp8.py:1610-1631;
 *                       cuda_fp8.hpp:473-545, :319-356)
 *   f32 -> bf16      : float32_to_bfloat16 / __float2bfloat16_rn
 *                      (numba/cuda/bf16.py:204-207; cuda_bf16.hpp:471-503)
 *   bf16 -> f32      : bfloat16_to_float32 (bf16.py:206; cuda_bf16.hpp:582-609)
 * saturate: 1 = SATFINITE, 0 = NOSAT (fp8 destinations only). */
B2K_API int b2k_cast(int src_format, int dst_format, int saturate, const void *in_dev,
             void *out_dev, int64_t n, void *stream);

/* The remaining conversion intrinsics as bulk casts.  Everything b2k_cast does
 * (rounding = B2K_ROUND_NEAREST), plus
 *   f32 -> bf16 toward zero / +inf / -inf : float32_to_bfloat16_rz/_ru/_rd
 *                      (numba/cuda/bf16.py:208-210; cuda_bf16.hpp:505-553)
 *   f64 -> bf16      : float64_to_bfloat16 (bf16.py:205; cuda_bf16.hpp:444-470)
 *   f32 -> e8m0, bf16 -> e8m0 (toward zero or +inf, with or without saturation)
 *                    : cvt_float_to_e8m0 / cvt_bfloat16raw_to_e8m0
 *                      (numba/cuda/_internal/cuda_fp8.py:3449-3654;
 *                       include/12/cuda_fp8.hpp:546-589, :689-740)
 *   e8m0 -> bf16, e8m0 -> f32 : cvt_e8m0_to_bf16raw, float(fp8_e8m0)
 *                      (cuda_fp8.hpp:817-851)
 *   f32 <-> f16      : round to nearest even
 *   f64 -> e4m3/e5m2, bf16 -> e4m3/e5m2 : cvt_double_to_fp8 (one rounding from the
 *                      double), cvt_bfloat16raw_to_fp8 (cuda_fp8.py:3269-3338,
 *                      :3413-3446; cuda_fp8.hpp:119-229, :442-450)
 *   f64 -> e8m0      : cvt_double_to_e8m0 (cuda_fp8.py:3557-3590; cuda_fp8.hpp:772-806)
 * and the conversions with an integer side (formats B2K_FMT_I8 .. B2K_FMT_U64,
 * B2K_FMT_BOOL):
 *   int16/32/64, uint16/32/64 <-> bf16 in all four rounding modes, bf16 -> int8 /
 *   uint8 toward zero : int16_to_bfloat16_rn ... bfloat16_to_uint64_ru,
 *                      bfloat16_to_int8_rz (numba/cuda/bf16.py:213-263;
 *                      cuda_bf16.hpp:641-1500).  To an integer: saturating, NaN
 *                      gives 0 (0x8000000000000000 in 64 bits)
 *   any integer -> e4m3/e5m2 (saturate = 1, nearest) and -> e8m0 (saturate = 1,
 *   B2K_ROUND_POS_INF) : the constructors fp8_e4m3(int) ... fp8_e8m0(uint64)
 *                      (cuda_fp8.py:568-613, :1562-1607, :2580-2601;
 *                       cuda_fp8.hpp:955-1023, :1568-1636, :2160-2215)
 *   e4m3/e5m2/e8m0 -> any integer (B2K_ROUND_ZERO) and -> bool : the conversion
 *                      operators int32(fp8_e4m3) ... (cuda_fp8.py:616-926,
 *                      :1610-1944, :2604-2962; cuda_fp8.hpp:1065-1263, :1678-1876,
 *                      :2305-2494)
 *   e4m3/e5m2 -> f16/bf16/f64, e8m0 -> f16/f64, f16 -> e4m3/e5m2 (either
 *   saturation), f16 -> e8m0 : the value types' floating-point neighbours
 *                      (cuda_fp8.hpp:363-388, :473-523, :1031-1063, :2260-2300)
 * A pair or a mode outside this list returns B2K_ERR_UNSUPPORTED. */
B2K_API int b2k_cast_ex(int src_format, int dst_format, int saturate, int rounding, const void *in_dev,
                        void *out_dev, int64_t n, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B2K_H_ */
