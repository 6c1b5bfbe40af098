// Table ops, type limits and warp helpers shared by the reduce kernels
// (b2k_reduce.cu: whole array; b2k_reduce_axis.cu: along one axis of a matrix).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace b2k_reduce_ops {

// ---- ops -----------------------------------------------------------------
// Integer add/mul run in the unsigned type of the same width: numba evaluates
// the functor in int64 and truncates when storing to the dtype's partials
// array, which is the same as wrap-around at the dtype's width.
template <typename T> struct UnsignedOf { using type = T; };
template <> struct UnsignedOf<int8_t> { using type = uint8_t; };
template <> struct UnsignedOf<int16_t> { using type = uint16_t; };
template <> struct UnsignedOf<int32_t> { using type = uint32_t; };
template <> struct UnsignedOf<int64_t> { using type = uint64_t; };

template <typename T> struct Limits;
#define B2K_LIMITS(T, LO, HI)                                   \
    template <> struct Limits<T> {                              \
        __host__ __device__ static T lowest() { return LO; }    \
        __host__ __device__ static T highest() { return HI; }   \
    };
B2K_LIMITS(int8_t, INT8_MIN, INT8_MAX)
B2K_LIMITS(int16_t, INT16_MIN, INT16_MAX)
B2K_LIMITS(int32_t, INT32_MIN, INT32_MAX)
B2K_LIMITS(int64_t, INT64_MIN, INT64_MAX)
B2K_LIMITS(uint8_t, 0, UINT8_MAX)
B2K_LIMITS(uint16_t, 0, UINT16_MAX)
B2K_LIMITS(uint32_t, 0u, UINT32_MAX)
B2K_LIMITS(uint64_t, 0ull, UINT64_MAX)
B2K_LIMITS(float, -__builtin_huge_valf(), __builtin_huge_valf())
B2K_LIMITS(double, -__builtin_huge_val(), __builtin_huge_val())
#undef B2K_LIMITS

struct OpAdd {
    template <typename T> __device__ static T identity() { return T(0); }
    template <typename T> __device__ static T apply(T a, T b) {
        using U = typename UnsignedOf<T>::type;
        return static_cast<T>(static_cast<U>(a) + static_cast<U>(b));
    }
};
struct OpMul {
    template <typename T> __device__ static T identity() { return T(1); }
    template <typename T> __device__ static T apply(T a, T b) {
        using U = typename UnsignedOf<T>::type;
        return static_cast<T>(static_cast<U>(a) * static_cast<U>(b));
    }
};
struct OpMax {
    template <typename T> __device__ static T identity() { return Limits<T>::lowest(); }
    template <typename T> __device__ static T apply(T a, T b) { return (b > a) ? b : a; }
};
struct OpMin {
    template <typename T> __device__ static T identity() { return Limits<T>::highest(); }
    template <typename T> __device__ static T apply(T a, T b) { return (b < a) ? b : a; }
};
struct OpAnd {
    template <typename T> __device__ static T identity() { return static_cast<T>(~T(0)); }
    template <typename T> __device__ static T apply(T a, T b) { return static_cast<T>(a & b); }
};
struct OpOr {
    template <typename T> __device__ static T identity() { return T(0); }
    template <typename T> __device__ static T apply(T a, T b) { return static_cast<T>(a | b); }
};
struct OpXor {
    template <typename T> __device__ static T identity() { return T(0); }
    template <typename T> __device__ static T apply(T a, T b) { return static_cast<T>(a ^ b); }
};

// ---- helpers -------------------------------------------------------------
template <typename T, typename Op>
__device__ __forceinline__ T fold_vector(T acc, const uint4 &raw) {
    constexpr int N = 16 / sizeof(T);
    union { uint4 v; T e[N]; } u;
    u.v = raw;
#pragma unroll
    for (int i = 0; i < N; ++i) acc = Op::template apply<T>(acc, u.e[i]);
    return acc;
}

template <typename T>
__device__ __forceinline__ T shuffle_xor(T v, int mask) {
    if constexpr (sizeof(T) < 4) {
        return static_cast<T>(__shfl_xor_sync(0xffffffffu, static_cast<int>(v), mask));
    } else {
        return __shfl_xor_sync(0xffffffffu, v, mask);
    }
}
__device__ __forceinline__ int64_t shuffle_xor(int64_t v, int mask) {
    return static_cast<int64_t>(__shfl_xor_sync(0xffffffffu, static_cast<long long>(v), mask));
}
__device__ __forceinline__ uint64_t shuffle_xor(uint64_t v, int mask) {
    return static_cast<uint64_t>(
        __shfl_xor_sync(0xffffffffu, static_cast<unsigned long long>(v), mask));
}

// ---- word-wise folds of small integers --------------------------------------
// 8- and 16-bit items, four or two to a 32-bit word: the per-byte / per-halfword
// video instructions fold a whole word at once (add wraps per item, as the scalar op
// does); products have no such form.
template <typename T, typename Op>
struct WordWise {
    static constexpr bool value = std::is_integral<T>::value && sizeof(T) < 4 && !std::is_same<Op, OpMul>::value;
};

template <typename T, typename Op>
__device__ __forceinline__ uint32_t apply_word(uint32_t a, uint32_t b) {
    constexpr bool bytes = sizeof(T) == 1, is_signed = std::is_signed<T>::value;
    if constexpr (std::is_same<Op, OpAdd>::value) {
        // per-item wrap-around add inside a word: add the low bits of every item, then
        // put the top bits back with a carry-less xor
        constexpr uint32_t TOP = bytes ? 0x80808080u : 0x80008000u;
        return ((a & ~TOP) + (b & ~TOP)) ^ ((a ^ b) & TOP);
    }
    else if constexpr (std::is_same<Op, OpAnd>::value) return a & b;
    else if constexpr (std::is_same<Op, OpOr>::value) return a | b;
    else if constexpr (std::is_same<Op, OpXor>::value) return a ^ b;
    else if constexpr (std::is_same<Op, OpMax>::value)
        return bytes ? (is_signed ? __vmaxs4(a, b) : __vmaxu4(a, b)) : (is_signed ? __vmaxs2(a, b) : __vmaxu2(a, b));
    else
        return bytes ? (is_signed ? __vmins4(a, b) : __vminu4(a, b)) : (is_signed ? __vmins2(a, b) : __vminu2(a, b));
}

// The identity of Op replicated into every item of a word, and the fold of a word's
// items into one item.
template <typename T, typename Op>
__device__ __forceinline__ uint32_t identity_word() {
    const uint32_t one = static_cast<uint32_t>(static_cast<typename UnsignedOf<T>::type>(Op::template identity<T>()));
    return sizeof(T) == 1 ? one * 0x01010101u : one * 0x00010001u;
}
template <typename T, typename Op>
__device__ __forceinline__ T fold_word(T acc, uint32_t w) {
#pragma unroll
    for (int k = 0; k < static_cast<int>(4 / sizeof(T)); ++k)
        acc = Op::template apply<T>(acc, static_cast<T>(w >> (8 * sizeof(T) * k)));
    return acc;
}

}  // namespace b2k_reduce_ops
