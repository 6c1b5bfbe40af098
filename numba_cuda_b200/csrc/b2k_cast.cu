// Bulk elementwise conversions f32 <-> bf16 and f32 <-> fp8 (E4M3 / E5M2).
//
// In the reference these conversions are scalar intrinsics reached through a
// non-inlined NVRTC-compiled shim per element (numba/cuda/_internal/
// cuda_fp8.py:166-207, :3341-3374; cuda_bf16.py:2054-2131, :2257-2295) whose
// bodies are the vendored cuda_fp8.hpp / cuda_bf16.hpp.  Here one thread
// converts four elements per step with the packed cvt instructions; the wide
// side moves as one 128-bit access per lane and the narrow side as one 32- or
// 64-bit access per lane, so every warp access is a run of whole 128-byte lines.
// HBM roofline: 4+1 bytes per element for fp8, 4+2 for bf16.
#include <type_traits>

#include "b2k_internal.cuh"

namespace {

constexpr int kThreads = 256;

// ---- scalar conversions ----------------------------------------------------

// Packed saturating convert: the FIRST source operand lands in the HIGH byte.
__device__ __forceinline__ uint32_t pack2_e4m3_sat(float hi, float lo) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack2_e5m2_sat(float hi, float lo) {
    uint16_t r;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// Round-to-nearest-even f32 -> fp8 without saturation: the integer algorithm of
// include/12/cuda_fp8.hpp:119-229 restated on f32 bit patterns (the reference
// widens to double first; widening is exact, so thresholds and dropped bits map
// one to one).  Overflow gives NaN (E4M3) or Inf (E5M2); every NaN gives 0x7F.
template <bool E5M2>
__device__ __forceinline__ uint32_t f32_to_fp8_nosat(float x) {
    constexpr uint32_t kMant = E5M2 ? 2u : 3u;             // stored mantissa bits
    constexpr int kBias = E5M2 ? 15 : 7;
    constexpr uint32_t kHalfMinDenorm = E5M2 ? 0x37000000u : 0x3A800000u;  // 2^-17 / 2^-10
    constexpr uint32_t kMinNorm = E5M2 ? 0x38800000u : 0x3C800000u;        // 2^-14 / 2^-6
    // first magnitude that no longer rounds to the largest finite value
    constexpr uint32_t kOverflowFrom = E5M2 ? 0x47700000u : 0x43E80001u;   // 61440 / >464
    constexpr uint32_t kHalf = 1u << (22u - kMant);

    const uint32_t bits = __float_as_uint(x);
    const uint32_t mag = bits & 0x7FFFFFFFu;
    const uint32_t sign = (bits >> 24) & 0x80u;
    if (mag > 0x7F800000u) return 0x7Fu;                   // NaN: canonical, sign dropped
    if (mag <= kHalfMinDenorm) return sign;
    if (mag >= kOverflowFrom) return sign | (E5M2 ? 0x7Cu : 0x7Fu);
    const int e8 = static_cast<int>(mag >> 23) - 127 + kBias;
    uint32_t mant = (bits >> (23u - kMant)) & ((1u << kMant) - 1u);
    uint32_t code;
    if (mag >= kMinNorm) {
        code = (static_cast<uint32_t>(e8) << kMant) | mant;
        const uint32_t dropped = bits & ((kHalf << 1) - 1u);
        if (dropped > kHalf || (dropped == kHalf && (mant & 1u))) ++code;
    } else {
        const uint32_t shift = static_cast<uint32_t>(1 - e8);
        mant |= 1u << kMant;
        code = mant >> shift;
        const uint32_t dropped = (bits | (1u << 23)) & ((kHalf << (shift + 1u)) - 1u);
        const uint32_t mid = kHalf << shift;
        if (dropped > mid || (dropped == mid && (code & 1u))) ++code;
    }
    return code | sign;
}

__device__ __forceinline__ uint32_t fp8x2_to_f16x2_e4m3(uint32_t two_codes) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(static_cast<uint16_t>(two_codes)));
    return r;
}
__device__ __forceinline__ uint32_t fp8x2_to_f16x2_e5m2(uint32_t two_codes) {
    uint32_t r;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(static_cast<uint16_t>(two_codes)));
    return r;
}
__device__ __forceinline__ float f16bits_to_f32(uint32_t h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(static_cast<uint16_t>(h)));
    return f;
}
__device__ __forceinline__ uint32_t pack2_bf16(float hi, float lo) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float bf16bits_to_f32(uint32_t h) {
    float f;
    asm("cvt.f32.bf16 %0, %1;" : "=f"(f) : "h"(static_cast<uint16_t>(h)));
    return f;
}

// ---- four-element converters ------------------------------------------------
// Each converter names its wide and narrow vector types and converts one item
// of four consecutive elements; `one` converts a single element for ragged ends.

template <bool E5M2, bool SAT>
struct F32ToFp8 {
    using In = float4; using Out = uint32_t; using InS = float; using OutS = uint8_t;
    __device__ static Out four(const In &v) {
        if constexpr (SAT) {
            if constexpr (E5M2) return pack2_e5m2_sat(v.y, v.x) | (pack2_e5m2_sat(v.w, v.z) << 16);
            else return pack2_e4m3_sat(v.y, v.x) | (pack2_e4m3_sat(v.w, v.z) << 16);
        } else {
            return f32_to_fp8_nosat<E5M2>(v.x) | (f32_to_fp8_nosat<E5M2>(v.y) << 8) |
                   (f32_to_fp8_nosat<E5M2>(v.z) << 16) | (f32_to_fp8_nosat<E5M2>(v.w) << 24);
        }
    }
    __device__ static OutS one(InS x) {
        if constexpr (SAT) {
            return static_cast<OutS>(E5M2 ? pack2_e5m2_sat(0.0f, x) : pack2_e4m3_sat(0.0f, x));
        } else {
            return static_cast<OutS>(f32_to_fp8_nosat<E5M2>(x));
        }
    }
};

template <bool E5M2>
struct Fp8ToF32 {
    using In = uint32_t; using Out = float4; using InS = uint8_t; using OutS = float;
    __device__ static Out four(const In &codes) {
        const uint32_t lo = E5M2 ? fp8x2_to_f16x2_e5m2(codes & 0xFFFFu) : fp8x2_to_f16x2_e4m3(codes & 0xFFFFu);
        const uint32_t hi = E5M2 ? fp8x2_to_f16x2_e5m2(codes >> 16) : fp8x2_to_f16x2_e4m3(codes >> 16);
        return make_float4(f16bits_to_f32(lo & 0xFFFFu), f16bits_to_f32(lo >> 16),
                           f16bits_to_f32(hi & 0xFFFFu), f16bits_to_f32(hi >> 16));
    }
    __device__ static OutS one(InS c) {
        const uint32_t h = E5M2 ? fp8x2_to_f16x2_e5m2(c) : fp8x2_to_f16x2_e4m3(c);
        return f16bits_to_f32(h & 0xFFFFu);
    }
};

struct F32ToBf16 {
    using In = float4; using Out = uint2; using InS = float; using OutS = uint16_t;
    __device__ static Out four(const In &v) {
        return make_uint2(pack2_bf16(v.y, v.x), pack2_bf16(v.w, v.z));
    }
    __device__ static OutS one(InS x) { return static_cast<OutS>(pack2_bf16(0.0f, x) & 0xFFFFu); }
};

struct Bf16ToF32 {
    using In = uint2; using Out = float4; using InS = uint16_t; using OutS = float;
    __device__ static Out four(const In &v) {
        return make_float4(bf16bits_to_f32(v.x & 0xFFFFu), bf16bits_to_f32(v.x >> 16),
                           bf16bits_to_f32(v.y & 0xFFFFu), bf16bits_to_f32(v.y >> 16));
    }
    __device__ static OutS one(InS h) { return bf16bits_to_f32(h); }
};

// ---- kernels ------------------------------------------------------------------

template <typename V>
__device__ __forceinline__ V load_stream(const V *p) {
    return __ldcs(p);  // read once: evict-first
}
template <typename V>
__device__ __forceinline__ void store_stream(V *p, const V &v) {
    __stcs(p, v);      // written once, not re-read by this kernel
}

// 128-bit path for arrays that are 16- but not 32-byte aligned: four elements per
// thread step, grid-stride.
template <typename C, int UNROLL>
__global__ void __launch_bounds__(kThreads)
cast_items_kernel(const typename C::In *__restrict__ in, typename C::Out *__restrict__ out,
                  int64_t items, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    int64_t i = tid;
    for (; i + (UNROLL - 1) * stride < items; i += UNROLL * stride) {
        typename C::In raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) raw[u] = load_stream(in + i + u * stride);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) store_stream(out + i + u * stride, C::four(raw[u]));
    }
    for (; i < items; i += stride) store_stream(out + i, C::four(load_stream(in + i)));
    // ragged end: fewer than four elements
    const int64_t t = items * 4 + tid;
    if (t < n) {
        const auto *in_s = reinterpret_cast<const typename C::InS *>(in);
        auto *out_s = reinterpret_cast<typename C::OutS *>(out);
        out_s[t] = C::one(in_s[t]);
    }
}


// ---- 256-bit path -------------------------------------------------------------
// Eight elements per thread step.  The wide side moves as one 256-bit access per
// lane (sm_100 has 256-bit global loads and stores), the narrow side as 64 or 128
// bits.  Every CTA owns one contiguous run of kThreads items, so the CTAs in
// flight cover one contiguous window of each array.
struct alignas(32) Bits256 { uint32_t w[8]; };

template <typename V> struct Mover;
template <> struct Mover<Bits256> {
    __device__ static Bits256 load(const Bits256 *p) {
        Bits256 r;
        asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]),
                       "=r"(r.w[6]), "=r"(r.w[7])
                     : "l"(p));
        return r;
    }
    __device__ static void store(Bits256 *p, const Bits256 &v) {
        asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]),
                     "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
                     : "memory");
    }
};
template <> struct Mover<uint4> {
    __device__ static uint4 load(const uint4 *p) { return __ldcs(p); }
    __device__ static void store(uint4 *p, const uint4 &v) { __stcs(p, v); }
};
template <> struct Mover<uint2> {
    __device__ static uint2 load(const uint2 *p) { return __ldcs(p); }
    __device__ static void store(uint2 *p, const uint2 &v) { __stcs(p, v); }
};

// Eight-element view of a four-element converter C.
template <typename C>
struct Eight {
    static constexpr bool kWidens = sizeof(typename C::Out) > sizeof(typename C::In);
    using Narrow4 = typename std::conditional<kWidens, typename C::In, typename C::Out>::type;
    using Narrow8 = typename std::conditional<sizeof(Narrow4) == 4, uint2, uint4>::type;
    using In = typename std::conditional<kWidens, Narrow8, Bits256>::type;
    using Out = typename std::conditional<kWidens, Bits256, Narrow8>::type;

    __device__ static Out convert(const In &v) {
        union { In raw; typename C::In half[2]; } src;
        union { Out raw; typename C::Out half[2]; } dst;
        src.raw = v;
        dst.half[0] = C::four(src.half[0]);
        dst.half[1] = C::four(src.half[1]);
        return dst.raw;
    }
};

template <typename C>
__global__ void __launch_bounds__(kThreads)
cast_wide_kernel(const typename Eight<C>::In *__restrict__ in, typename Eight<C>::Out *__restrict__ out,
                 int64_t items /* of eight elements */, int64_t n) {
    using E = Eight<C>;
    // one item per thread and one CTA per 256 items measured best: the hardware
    // keeps enough CTAs in flight, and they sweep both arrays front to back
    const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (i < items) Mover<typename E::Out>::store(out + i, E::convert(Mover<typename E::In>::load(in + i)));
    // ragged end: fewer than eight elements, done by the last CTA
    if (blockIdx.x == gridDim.x - 1) {
        const int64_t t = items * 8 + threadIdx.x;
        if (t < n) {
            const auto *in_s = reinterpret_cast<const typename C::InS *>(in);
            auto *out_s = reinterpret_cast<typename C::OutS *>(out);
            out_s[t] = C::one(in_s[t]);
        }
    }
}

// Any alignment: one element per thread step.
template <typename C>
__global__ void __launch_bounds__(kThreads)
cast_scalar_kernel(const typename C::InS *__restrict__ in, typename C::OutS *__restrict__ out, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride)
        out[i] = C::one(in[i]);
}

template <typename C>
int launch(const void *in, void *out, int64_t n, cudaStream_t stream) {
    if (n == 0) return B2K_OK;
    if (!b2k::aligned_to<void>(in, sizeof(typename C::InS)) || !b2k::aligned_to<void>(out, sizeof(typename C::OutS)))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_cast: pointers must be aligned to the element size");
    const int64_t cap = static_cast<int64_t>(b2k::sm_count()) * 8;
    const bool vector_ok = b2k::aligned_to<void>(in, sizeof(typename C::In)) &&
                           b2k::aligned_to<void>(out, sizeof(typename C::Out));
    const bool wide_ok = b2k::aligned_to<void>(in, sizeof(typename Eight<C>::In)) &&
                         b2k::aligned_to<void>(out, sizeof(typename Eight<C>::Out)) &&
                         B2K_ENV_INT("B2K_CAST_WIDE", 1) != 0;
    if (wide_ok) {
        const int64_t items = n / 8;
        int64_t grid = (items + kThreads - 1) / kThreads;
        if (grid < 1) grid = 1;
        if (grid > 0x7FFFFFFFll) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_cast: array too large");
        cast_wide_kernel<C><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const typename Eight<C>::In *>(in), static_cast<typename Eight<C>::Out *>(out), items, n);
    } else if (vector_ok) {
        const int64_t items = n / 4;
        int64_t grid = (items + kThreads * 4 - 1) / (kThreads * 4);
        if (grid < 1) grid = 1;
        if (grid > cap) grid = cap;
        cast_items_kernel<C, 4><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const typename C::In *>(in), static_cast<typename C::Out *>(out), items, n);
    } else {
        int64_t grid = (n + kThreads - 1) / kThreads;
        if (grid > cap) grid = cap;
        cast_scalar_kernel<C><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const typename C::InS *>(in), static_cast<typename C::OutS *>(out), n);
    }
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_cast launch");
    return B2K_OK;
}

// ---- further conversions: directed rounding, f64, E8M0, f16 --------------------
// Element-wise converters (`one`) run through a generic wide kernel: eight
// elements per thread (four when an 8-byte type is involved), each side moving as
// one vector access per lane.

template <int MODE>  // cudaRoundMode order: 0 nearest, 1 zero, 2 +inf, 3 -inf
struct F32ToBf16Mode {
    using InS = float; using OutS = uint16_t;
    __device__ static OutS one(InS x) {
        uint16_t r;
        if constexpr (MODE == 1) asm("cvt.rz.bf16.f32 %0, %1;" : "=h"(r) : "f"(x));
        else if constexpr (MODE == 2) asm("cvt.rp.bf16.f32 %0, %1;" : "=h"(r) : "f"(x));
        else if constexpr (MODE == 3) asm("cvt.rm.bf16.f32 %0, %1;" : "=h"(r) : "f"(x));
        else asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(x));
        return r;
    }
};
struct F64ToBf16 {  // __double2bfloat16 (cuda_bf16.hpp:444-470)
    using InS = double; using OutS = uint16_t;
    __device__ static OutS one(InS x) {
        uint16_t r;
        asm("cvt.rn.bf16.f64 %0, %1;" : "=h"(r) : "d"(x));
        return r;
    }
};
template <bool UP, bool SAT>  // __nv_cvt_float_to_e8m0 (cuda_fp8.hpp:689-740)
struct F32ToE8m0 {
    using InS = float; using OutS = uint8_t;
    __device__ static OutS one(InS x) {
        uint16_t r;
        if constexpr (UP && SAT) asm("cvt.rp.satfinite.ue8m0x2.f32 %0, %2, %1;" : "=h"(r) : "f"(x), "f"(0.0f));
        else if constexpr (UP) asm("cvt.rp.ue8m0x2.f32 %0, %2, %1;" : "=h"(r) : "f"(x), "f"(0.0f));
        else if constexpr (SAT) asm("cvt.rz.satfinite.ue8m0x2.f32 %0, %2, %1;" : "=h"(r) : "f"(x), "f"(0.0f));
        else asm("cvt.rz.ue8m0x2.f32 %0, %2, %1;" : "=h"(r) : "f"(x), "f"(0.0f));
        return static_cast<OutS>(r);
    }
};
template <bool UP, bool SAT>  // __nv_cvt_bfloat16raw_to_e8m0 (cuda_fp8.hpp:546-589)
struct Bf16ToE8m0 {
    using InS = uint16_t; using OutS = uint8_t;
    __device__ static OutS one(InS h) {
        uint16_t r;
        const uint32_t in = h;
        if constexpr (UP && SAT) asm("cvt.rp.satfinite.ue8m0x2.bf16x2 %0, %1;" : "=h"(r) : "r"(in));
        else if constexpr (UP) asm("cvt.rp.ue8m0x2.bf16x2 %0, %1;" : "=h"(r) : "r"(in));
        else if constexpr (SAT) asm("cvt.rz.satfinite.ue8m0x2.bf16x2 %0, %1;" : "=h"(r) : "r"(in));
        else asm("cvt.rz.ue8m0x2.bf16x2 %0, %1;" : "=h"(r) : "r"(in));
        return static_cast<OutS>(r);
    }
};
struct E8m0ToBf16 {  // __nv_cvt_e8m0_to_bf16raw (cuda_fp8.hpp:833-851)
    using InS = uint8_t; using OutS = uint16_t;
    __device__ static OutS one(InS e) {
        uint32_t r;
        asm("cvt.rn.bf16x2.ue8m0x2 %0, %1;" : "=r"(r) : "h"(static_cast<uint16_t>(e)));
        return static_cast<OutS>(r);
    }
};
struct E8m0ToF32 {  // float(fp8_e8m0): E8M0 -> bf16 -> f32
    using InS = uint8_t; using OutS = float;
    __device__ static OutS one(InS e) { return bf16bits_to_f32(E8m0ToBf16::one(e)); }
};
struct F32ToF16 {
    using InS = float; using OutS = uint16_t;
    __device__ static OutS one(InS x) {
        uint16_t r;
        asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(x));
        return r;
    }
};
struct F16ToF32 {
    using InS = uint16_t; using OutS = float;
    __device__ static OutS one(InS h) { return f16bits_to_f32(h); }
};

// f64 -> fp8: __nv_cvt_double_to_fp8 (cuda_fp8.hpp:119-229) rounds the double to the
// fp8 grid once, to nearest even, with integer code (on the device too: there is no
// cvt from f64 to fp8).  The same result comes out of two hardware steps: the double
// is first rounded to float32 "to odd" (truncate, then set the last bit if anything
// was cut off), which keeps a sticky trace of every discarded bit, and the float is
// then rounded to nearest even by the float encoder -- with 24 significant bits
// against at most 4 in the target the second rounding sees exactly what a single
// one would.  Doubles beyond the float range truncate to the largest finite float
// and overflow the fp8 range like the double does; doubles below it leave a
// non-zero denormal that rounds to a signed zero like the double does.  NaNs are
// the one case where the integer code's result depends on the double's own bits
// (sign, and for E5M2 the top two mantissa bits), so they are patched in from there.
__device__ __forceinline__ float f64_to_f32_round_to_odd(double x) {
    float f;
    double back;
    asm("cvt.rz.f32.f64 %0, %1;" : "=f"(f) : "d"(x));
    asm("cvt.f64.f32 %0, %1;" : "=d"(back) : "f"(f));
    const uint32_t u = __float_as_uint(f);
    return __uint_as_float(back != x ? (u | 1u) : u);   // a NaN compares unequal and stays a NaN
}
template <bool E5M2, bool SAT>
struct F64ToFp8 {
    using InS = double; using OutS = uint8_t;
    __device__ static uint32_t nan_code(double x) {
        const uint32_t hi = static_cast<uint32_t>(__double2hiint(x));
        return ((hi >> 24) & 0x80u) | (E5M2 ? (0x7Eu | ((hi >> 18) & 3u)) : 0x7Fu);
    }
    __device__ static OutS one(InS x) {
        const uint32_t code = F32ToFp8<E5M2, SAT>::one(f64_to_f32_round_to_odd(x));
        return static_cast<OutS>(x != x ? nan_code(x) : code);
    }
    // two codes at once, `a` in the low byte: one packed cvt in the saturating mode
    __device__ static uint32_t pair(InS a, InS b) {
        const float fa = f64_to_f32_round_to_odd(a), fb = f64_to_f32_round_to_odd(b);
        uint32_t lo, hi;
        if constexpr (SAT) {
            const uint32_t both = E5M2 ? pack2_e5m2_sat(fb, fa) : pack2_e4m3_sat(fb, fa);
            lo = both & 0xFFu;
            hi = both >> 8;
        } else {
            lo = f32_to_fp8_nosat<E5M2>(fa);
            hi = f32_to_fp8_nosat<E5M2>(fb);
        }
        if (a != a) lo = nan_code(a);
        if (b != b) hi = nan_code(b);
        return lo | (hi << 8);
    }
};
// bf16 -> fp8: __nv_cvt_bfloat16raw_to_fp8 (cuda_fp8.hpp:442-450) = the bits moved into
// the top half of a float, then the float conversion.
template <bool E5M2, bool SAT>
struct Bf16ToFp8 {
    using InS = uint16_t; using OutS = uint8_t;
    __device__ static OutS one(InS h) {
        return F32ToFp8<E5M2, SAT>::one(__uint_as_float(static_cast<uint32_t>(h) << 16));
    }
    // two codes at once, `a` in the low byte: one packed cvt in the saturating mode
    __device__ static uint32_t pair(InS a, InS b) {
        const float fa = __uint_as_float(static_cast<uint32_t>(a) << 16);
        const float fb = __uint_as_float(static_cast<uint32_t>(b) << 16);
        if constexpr (SAT) return E5M2 ? pack2_e5m2_sat(fb, fa) : pack2_e4m3_sat(fb, fa);
        else return f32_to_fp8_nosat<E5M2>(fa) | (f32_to_fp8_nosat<E5M2>(fb) << 8);
    }
};
// f64 -> e8m0: __nv_cvt_double_to_e8m0 (cuda_fp8.hpp:772-806).  The double is rounded
// to float "to odd" (a sticky bit for everything discarded lands in the last place),
// so that the directed rounding of the float conversion sees all of the double.
template <bool UP, bool SAT>
struct F64ToE8m0 {
    using InS = double; using OutS = uint8_t;
    __device__ static OutS one(InS x) {
        float f;
        double d;
        asm("cvt.rn.f32.f64 %0, %1;" : "=f"(f) : "d"(x));
        asm("cvt.f64.f32 %0, %1;" : "=d"(d) : "f"(f));
        uint32_t u = __float_as_uint(f);
        const bool not_nan = (u << 1) <= 0xFF000000u;
        if (x > 0.0 && d > x) --u;
        if (x < 0.0 && d < x) --u;
        if (d != x && not_nan) u |= 1u;
        return F32ToE8m0<UP, SAT>::one(__uint_as_float(u));
    }
};

// ---- integer formats -------------------------------------------------------------
// The fp8 value types are constructed from and converted to every integer type
// (cuda_fp8.hpp:955-1023, :1065-1263 for E5M2; :1568-1636, :1678-1876 for E4M3;
// :2160-2215, :2305-2494 for E8M0), and bf16 converts from and to the 16-, 32-
// and 64-bit integers in all four rounding modes (numba/cuda/bf16.py:213-263 =
// cuda_bf16.hpp:641-1500).  Each is one or two cvt instructions; float-to-integer
// cvt saturates at the ends of the integer range and turns a NaN into 0 (into
// 0x8000000000000000 for a 64-bit result), which is what the headers' host paths
// spell out with comparisons.
template <typename I> struct IntPtx;
#define B2K_INT_PTX(I, REG, SUFFIX, CONS)                                                          \
    template <> struct IntPtx<I> {                                                                 \
        template <int MODE> __device__ static uint16_t to_bf16(I v) {                              \
            uint16_t r;                                                                            \
            const REG x = static_cast<REG>(v);                                                     \
            if constexpr (MODE == 1) asm("cvt.rz.bf16." SUFFIX " %0, %1;" : "=h"(r) : CONS(x));    \
            else if constexpr (MODE == 2) asm("cvt.rp.bf16." SUFFIX " %0, %1;" : "=h"(r) : CONS(x)); \
            else if constexpr (MODE == 3) asm("cvt.rm.bf16." SUFFIX " %0, %1;" : "=h"(r) : CONS(x)); \
            else asm("cvt.rn.bf16." SUFFIX " %0, %1;" : "=h"(r) : CONS(x));                        \
            return r;                                                                              \
        }                                                                                          \
        template <int MODE> __device__ static I from_bf16(uint16_t h) {                            \
            REG r;                                                                                 \
            if constexpr (MODE == 1) asm("cvt.rzi." SUFFIX ".bf16 %0, %1;" : "=" CONS(r) : "h"(h)); \
            else if constexpr (MODE == 2) asm("cvt.rpi." SUFFIX ".bf16 %0, %1;" : "=" CONS(r) : "h"(h)); \
            else if constexpr (MODE == 3) asm("cvt.rmi." SUFFIX ".bf16 %0, %1;" : "=" CONS(r) : "h"(h)); \
            else asm("cvt.rni." SUFFIX ".bf16 %0, %1;" : "=" CONS(r) : "h"(h));                    \
            return static_cast<I>(r);                                                              \
        }                                                                                          \
        __device__ static I from_f16_rz(uint16_t h) {                                              \
            REG r;                                                                                 \
            asm("cvt.rzi." SUFFIX ".f16 %0, %1;" : "=" CONS(r) : "h"(h));                          \
            return static_cast<I>(r);                                                              \
        }                                                                                          \
    };
B2K_INT_PTX(int16_t, short, "s16", "h")
B2K_INT_PTX(uint16_t, unsigned short, "u16", "h")
B2K_INT_PTX(int32_t, int, "s32", "r")
B2K_INT_PTX(uint32_t, unsigned int, "u32", "r")
B2K_INT_PTX(int64_t, long long, "s64", "l")
B2K_INT_PTX(uint64_t, unsigned long long, "u64", "l")
#undef B2K_INT_PTX
// the 8-bit results: convert to 32 bits, then clamp (a NaN has become 0 by then)
template <> struct IntPtx<int8_t> {
    template <int MODE> __device__ static int8_t from_bf16(uint16_t h) {
        const int v = IntPtx<int32_t>::from_bf16<MODE>(h);
        return static_cast<int8_t>(v < -128 ? -128 : v > 127 ? 127 : v);
    }
    __device__ static int8_t from_f16_rz(uint16_t h) {
        const int v = IntPtx<int32_t>::from_f16_rz(h);
        return static_cast<int8_t>(v < -128 ? -128 : v > 127 ? 127 : v);
    }
};
template <> struct IntPtx<uint8_t> {
    template <int MODE> __device__ static uint8_t from_bf16(uint16_t h) {
        const unsigned int v = IntPtx<uint32_t>::from_bf16<MODE>(h);
        return static_cast<uint8_t>(v > 255u ? 255u : v);
    }
    __device__ static uint8_t from_f16_rz(uint16_t h) {
        const unsigned int v = IntPtx<uint32_t>::from_f16_rz(h);
        return static_cast<uint8_t>(v > 255u ? 255u : v);
    }
};

template <typename I, int MODE>
struct IntToBf16 {
    using InS = I; using OutS = uint16_t;
    __device__ static OutS one(InS v) { return IntPtx<I>::template to_bf16<MODE>(v); }
};
template <typename I, int MODE>
struct Bf16ToInt {
    using InS = uint16_t; using OutS = I;
    __device__ static OutS one(InS h) { return IntPtx<I>::template from_bf16<MODE>(h); }
};
// fp8_e4m3(int) / fp8_e5m2(int): the integer rounded to float32, then the saturating
// float conversion
template <typename I, bool E5M2>
struct IntToFp8 {
    using InS = I; using OutS = uint8_t;
    __device__ static OutS one(InS v) { return F32ToFp8<E5M2, true>::one(static_cast<float>(v)); }
};
// fp8_e8m0(int): the smallest power of two that is not below |v| (the constructors
// go through float, double or a bf16 bumped up by one place, all to that effect):
// |v| rounded up to float32, then the float conversion rounding up, saturating
template <typename I>
struct IntToE8m0 {
    using InS = I; using OutS = uint8_t;
    __device__ static OutS one(InS v) {
        unsigned long long mag;
        if constexpr (std::is_signed<I>::value) {
            const long long w = static_cast<long long>(v);
            mag = w < 0 ? 0ull - static_cast<unsigned long long>(w) : static_cast<unsigned long long>(w);
        } else {
            mag = static_cast<unsigned long long>(v);
        }
        return F32ToE8m0<true, true>::one(__ull2float_ru(mag));
    }
};
// int(fp8_e4m3) etc.: the code widened to half (exact), then cvt toward zero
template <typename I, bool E5M2>
struct Fp8ToInt {
    using InS = uint8_t; using OutS = I;
    __device__ static OutS one(InS c) {
        const uint32_t h = E5M2 ? fp8x2_to_f16x2_e5m2(c) : fp8x2_to_f16x2_e4m3(c);
        return IntPtx<I>::from_f16_rz(static_cast<uint16_t>(h));
    }
};
template <typename I>
struct E8m0ToInt {
    using InS = uint8_t; using OutS = I;
    __device__ static OutS one(InS e) { return IntPtx<I>::template from_bf16<1>(E8m0ToBf16::one(e)); }
};
// bool(fp8): anything but a zero of either sign; an E8M0 code is never zero
template <int FORMAT>
struct Fp8ToBool {
    using InS = uint8_t; using OutS = uint8_t;
    __device__ static OutS one(InS c) { return FORMAT == B2K_FMT_E8M0 ? 1u : ((c & 0x7Fu) != 0u ? 1u : 0u); }
};
// the remaining floating-point neighbours of the value types
template <bool E5M2>
struct Fp8ToF16 {  // __nv_cvt_fp8_to_halfraw (cuda_fp8.hpp:473-523)
    using InS = uint8_t; using OutS = uint16_t;
    __device__ static OutS one(InS c) {
        return static_cast<OutS>(E5M2 ? fp8x2_to_f16x2_e5m2(c) : fp8x2_to_f16x2_e4m3(c));
    }
};
template <bool E5M2>
struct Fp8ToBf16 {  // __float2bfloat16_rz(float(fp8)): every fp8 value is a bf16 value
    using InS = uint8_t; using OutS = uint16_t;
    __device__ static OutS one(InS c) { return F32ToBf16Mode<1>::one(Fp8ToF32<E5M2>::one(c)); }
};
template <bool E5M2>
struct Fp8ToF64 {
    using InS = uint8_t; using OutS = double;
    __device__ static OutS one(InS c) { return static_cast<double>(Fp8ToF32<E5M2>::one(c)); }
};
struct E8m0ToF64 {
    using InS = uint8_t; using OutS = double;
    __device__ static OutS one(InS e) {
        double d;   // written as a cvt so that no flush-to-zero mode can touch 2^-127
        asm("cvt.f64.f32 %0, %1;" : "=d"(d) : "f"(E8m0ToF32::one(e)));
        return d;
    }
};
struct E8m0ToF16 {  // __float2half_rn(float(fp8_e8m0)): beyond 2^15 it is infinity, below 2^-25 zero
    using InS = uint8_t; using OutS = uint16_t;
    __device__ static OutS one(InS e) { return F32ToF16::one(E8m0ToF32::one(e)); }
};
template <bool E5M2, bool SAT>
struct F16ToFp8 {  // __nv_cvt_halfraw_to_fp8 (cuda_fp8.hpp:363-388)
    using InS = uint16_t; using OutS = uint8_t;
    __device__ static OutS one(InS h) {
        if constexpr (SAT) {
            uint16_t r;
            if constexpr (E5M2) asm("cvt.rn.satfinite.e5m2x2.f16x2 %0, %1;" : "=h"(r) : "r"(static_cast<uint32_t>(h)));
            else asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(static_cast<uint32_t>(h)));
            return static_cast<OutS>(r);
        } else {
            return static_cast<OutS>(f32_to_fp8_nosat<E5M2>(f16bits_to_f32(h)));
        }
    }
};
template <bool UP, bool SAT>
struct F16ToE8m0 {  // fp8_e8m0(half): through float
    using InS = uint16_t; using OutS = uint8_t;
    __device__ static OutS one(InS h) { return F32ToE8m0<UP, SAT>::one(f16bits_to_f32(h)); }
};

template <int BYTES> struct VecOf;
template <> struct VecOf<4> { using type = uint32_t; };
template <> struct VecOf<8> { using type = uint2; };
template <> struct VecOf<16> { using type = uint4; };
template <> struct VecOf<32> { using type = Bits256; };
template <> struct Mover<uint32_t> {
    __device__ static uint32_t load(const uint32_t *p) { return __ldcs(p); }
    __device__ static void store(uint32_t *p, const uint32_t &v) { __stcs(p, v); }
};

template <typename C, typename = void> struct HasPair : std::false_type {};
template <typename C> struct HasPair<C, std::void_t<decltype(&C::pair)>> : std::true_type {};

template <typename C>
struct WideOf {
    // elements per thread: the wider side moves as one 256-bit access (128-bit when an
    // 8-byte type is involved, to keep the narrow side at 32 bits or more)
    static constexpr int WIDER = sizeof(typename C::InS) > sizeof(typename C::OutS) ? sizeof(typename C::InS)
                                                                                     : sizeof(typename C::OutS);
    static constexpr int ELEMS = WIDER == 8 ? 4 : 32 / WIDER;
    using In = typename VecOf<ELEMS * sizeof(typename C::InS)>::type;
    using Out = typename VecOf<ELEMS * sizeof(typename C::OutS)>::type;
    __device__ static Out convert(const In &v) {
        union { In raw; typename C::InS e[ELEMS]; } src;
        union { Out raw; typename C::OutS e[ELEMS]; uint16_t two[ELEMS / 2]; } dst;
        src.raw = v;
        if constexpr (HasPair<C>::value) {   // converters of byte codes that do two at a time
#pragma unroll
            for (int k = 0; k < ELEMS; k += 2) dst.two[k / 2] = static_cast<uint16_t>(C::pair(src.e[k], src.e[k + 1]));
        } else {
#pragma unroll
            for (int k = 0; k < ELEMS; ++k) dst.e[k] = C::one(src.e[k]);
        }
        return dst.raw;
    }
};

template <typename C>
__global__ void __launch_bounds__(kThreads)
cast_generic_wide_kernel(const typename WideOf<C>::In *__restrict__ in, typename WideOf<C>::Out *__restrict__ out,
                         int64_t items, int64_t n) {
    using W = WideOf<C>;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
    if (i < items) Mover<typename W::Out>::store(out + i, W::convert(Mover<typename W::In>::load(in + i)));
    if (blockIdx.x == gridDim.x - 1) {  // ragged end
        const int64_t t = items * W::ELEMS + threadIdx.x;
        if (t < n) {
            const auto *in_s = reinterpret_cast<const typename C::InS *>(in);
            auto *out_s = reinterpret_cast<typename C::OutS *>(out);
            out_s[t] = C::one(in_s[t]);
        }
    }
}

template <typename C>
int launch_generic(const void *in, void *out, int64_t n, cudaStream_t stream) {
    if (n == 0) return B2K_OK;
    if (!b2k::aligned_to<void>(in, sizeof(typename C::InS)) || !b2k::aligned_to<void>(out, sizeof(typename C::OutS)))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_cast_ex: pointers must be aligned to the element size");
    using W = WideOf<C>;
    if (b2k::aligned_to<void>(in, sizeof(typename W::In)) && b2k::aligned_to<void>(out, sizeof(typename W::Out))) {
        const int64_t items = n / W::ELEMS;
        int64_t grid = (items + kThreads - 1) / kThreads;
        if (grid < 1) grid = 1;
        if (grid > 0x7FFFFFFFll) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_cast_ex: array too large");
        cast_generic_wide_kernel<C><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const typename W::In *>(in), static_cast<typename W::Out *>(out), items, n);
    } else {
        int64_t grid = (n + kThreads - 1) / kThreads;
        const int64_t cap = static_cast<int64_t>(b2k::sm_count()) * 8;
        if (grid > cap) grid = cap;
        cast_scalar_kernel<C><<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(
            static_cast<const typename C::InS *>(in), static_cast<typename C::OutS *>(out), n);
    }
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_cast_ex launch");
    return B2K_OK;
}

// ---- dispatch of the integer formats ----------------------------------------------
inline bool is_int_format(int f) { return f >= B2K_FMT_I8 && f <= B2K_FMT_U64; }

// `CALL` is an expression that names the integer type as `I`
#define B2K_FOR_WIDE_INT(FMT, CALL)                                         \
    switch (FMT) {                                                          \
        case B2K_FMT_I16: { using I = int16_t; return CALL; }               \
        case B2K_FMT_I32: { using I = int32_t; return CALL; }               \
        case B2K_FMT_I64: { using I = int64_t; return CALL; }               \
        case B2K_FMT_U16: { using I = uint16_t; return CALL; }              \
        case B2K_FMT_U32: { using I = uint32_t; return CALL; }              \
        case B2K_FMT_U64: { using I = uint64_t; return CALL; }              \
        default: break;                                                     \
    }
#define B2K_FOR_ANY_INT(FMT, CALL)                                          \
    switch (FMT) {                                                          \
        case B2K_FMT_I8: { using I = int8_t; return CALL; }                 \
        case B2K_FMT_U8: { using I = uint8_t; return CALL; }                \
        default: break;                                                     \
    }                                                                       \
    B2K_FOR_WIDE_INT(FMT, CALL)

template <int MODE>
int int_to_bf16(int src, const void *in, void *out, int64_t n, cudaStream_t s) {
    B2K_FOR_WIDE_INT(src, (launch_generic<IntToBf16<I, MODE>>(in, out, n, s)))
    return B2K_ERR_UNSUPPORTED;
}
template <int MODE>
int bf16_to_int(int dst, const void *in, void *out, int64_t n, cudaStream_t s) {
    B2K_FOR_WIDE_INT(dst, (launch_generic<Bf16ToInt<I, MODE>>(in, out, n, s)))
    return B2K_ERR_UNSUPPORTED;
}
template <bool E5M2>
int int_to_fp8(int src, const void *in, void *out, int64_t n, cudaStream_t s) {
    B2K_FOR_ANY_INT(src, (launch_generic<IntToFp8<I, E5M2>>(in, out, n, s)))
    return B2K_ERR_UNSUPPORTED;
}
int int_to_e8m0(int src, const void *in, void *out, int64_t n, cudaStream_t s) {
    B2K_FOR_ANY_INT(src, (launch_generic<IntToE8m0<I>>(in, out, n, s)))
    return B2K_ERR_UNSUPPORTED;
}
template <bool E5M2>
int fp8_to_int(int dst, const void *in, void *out, int64_t n, cudaStream_t s) {
    B2K_FOR_ANY_INT(dst, (launch_generic<Fp8ToInt<I, E5M2>>(in, out, n, s)))
    return B2K_ERR_UNSUPPORTED;
}
int e8m0_to_int(int dst, const void *in, void *out, int64_t n, cudaStream_t s) {
    B2K_FOR_ANY_INT(dst, (launch_generic<E8m0ToInt<I>>(in, out, n, s)))
    return B2K_ERR_UNSUPPORTED;
}

// Conversions with an integer or bool side, and the half / bfloat16 / double
// neighbours of the fp8 value types.  Returns B2K_ERR_UNSUPPORTED (without a
// message) for a pair or a mode that is not one of them.
int cast_value_types(int src, int dst, bool sat, int rounding, const void *in, void *out, int64_t n,
                     cudaStream_t s) {
    const bool nearest = rounding == B2K_ROUND_NEAREST;
    const bool e8_mode = rounding == B2K_ROUND_ZERO || rounding == B2K_ROUND_POS_INF;
    if (is_int_format(src) && dst == B2K_FMT_BF16) {
        switch (rounding) {
            case B2K_ROUND_ZERO: return int_to_bf16<1>(src, in, out, n, s);
            case B2K_ROUND_POS_INF: return int_to_bf16<2>(src, in, out, n, s);
            case B2K_ROUND_MIN_INF: return int_to_bf16<3>(src, in, out, n, s);
            default: return int_to_bf16<0>(src, in, out, n, s);
        }
    }
    if (src == B2K_FMT_BF16 && is_int_format(dst)) {
        if (dst == B2K_FMT_I8 && rounding == B2K_ROUND_ZERO) return launch_generic<Bf16ToInt<int8_t, 1>>(in, out, n, s);
        if (dst == B2K_FMT_U8 && rounding == B2K_ROUND_ZERO) return launch_generic<Bf16ToInt<uint8_t, 1>>(in, out, n, s);
        switch (rounding) {
            case B2K_ROUND_ZERO: return bf16_to_int<1>(dst, in, out, n, s);
            case B2K_ROUND_POS_INF: return bf16_to_int<2>(dst, in, out, n, s);
            case B2K_ROUND_MIN_INF: return bf16_to_int<3>(dst, in, out, n, s);
            default: return bf16_to_int<0>(dst, in, out, n, s);
        }
    }
    // constructors of the value types from integers: saturating, to nearest
    // (E4M3 / E5M2) or up to the next power of two (E8M0)
    if (is_int_format(src) && sat) {
        if (dst == B2K_FMT_E4M3 && nearest) return int_to_fp8<false>(src, in, out, n, s);
        if (dst == B2K_FMT_E5M2 && nearest) return int_to_fp8<true>(src, in, out, n, s);
        if (dst == B2K_FMT_E8M0 && rounding == B2K_ROUND_POS_INF) return int_to_e8m0(src, in, out, n, s);
    }
    // conversion operators of the value types to integers: toward zero
    if (is_int_format(dst) && rounding == B2K_ROUND_ZERO) {
        if (src == B2K_FMT_E4M3) return fp8_to_int<false>(dst, in, out, n, s);
        if (src == B2K_FMT_E5M2) return fp8_to_int<true>(dst, in, out, n, s);
        if (src == B2K_FMT_E8M0) return e8m0_to_int(dst, in, out, n, s);
    }
    if (dst == B2K_FMT_BOOL) {
        if (src == B2K_FMT_E4M3) return launch_generic<Fp8ToBool<B2K_FMT_E4M3>>(in, out, n, s);
        if (src == B2K_FMT_E5M2) return launch_generic<Fp8ToBool<B2K_FMT_E5M2>>(in, out, n, s);
        if (src == B2K_FMT_E8M0) return launch_generic<Fp8ToBool<B2K_FMT_E8M0>>(in, out, n, s);
    }
    if (nearest) {
        if (src == B2K_FMT_E4M3 && dst == B2K_FMT_F16) return launch_generic<Fp8ToF16<false>>(in, out, n, s);
        if (src == B2K_FMT_E5M2 && dst == B2K_FMT_F16) return launch_generic<Fp8ToF16<true>>(in, out, n, s);
        if (src == B2K_FMT_E4M3 && dst == B2K_FMT_BF16) return launch_generic<Fp8ToBf16<false>>(in, out, n, s);
        if (src == B2K_FMT_E5M2 && dst == B2K_FMT_BF16) return launch_generic<Fp8ToBf16<true>>(in, out, n, s);
        if (src == B2K_FMT_E4M3 && dst == B2K_FMT_F64) return launch_generic<Fp8ToF64<false>>(in, out, n, s);
        if (src == B2K_FMT_E5M2 && dst == B2K_FMT_F64) return launch_generic<Fp8ToF64<true>>(in, out, n, s);
        if (src == B2K_FMT_E8M0 && dst == B2K_FMT_F64) return launch_generic<E8m0ToF64>(in, out, n, s);
        if (src == B2K_FMT_E8M0 && dst == B2K_FMT_F16) return launch_generic<E8m0ToF16>(in, out, n, s);
        if (src == B2K_FMT_F16 && dst == B2K_FMT_E4M3)
            return sat ? launch_generic<F16ToFp8<false, true>>(in, out, n, s)
                       : launch_generic<F16ToFp8<false, false>>(in, out, n, s);
        if (src == B2K_FMT_F16 && dst == B2K_FMT_E5M2)
            return sat ? launch_generic<F16ToFp8<true, true>>(in, out, n, s)
                       : launch_generic<F16ToFp8<true, false>>(in, out, n, s);
    }
    if (src == B2K_FMT_F16 && dst == B2K_FMT_E8M0 && e8_mode) {
        if (rounding == B2K_ROUND_POS_INF)
            return sat ? launch_generic<F16ToE8m0<true, true>>(in, out, n, s)
                       : launch_generic<F16ToE8m0<true, false>>(in, out, n, s);
        return sat ? launch_generic<F16ToE8m0<false, true>>(in, out, n, s)
                   : launch_generic<F16ToE8m0<false, false>>(in, out, n, s);
    }
    return B2K_ERR_UNSUPPORTED;
}
#undef B2K_FOR_WIDE_INT
#undef B2K_FOR_ANY_INT

}  // namespace

extern "C" int b2k_cast(int src, int dst, int saturate, const void *in_dev, void *out_dev,
                        int64_t n, void *stream) {
    B2K_RANGE("b2k_cast");
    if (n < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_cast: negative length %lld", (long long)n);
    if (n > 0 && (!in_dev || !out_dev)) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_cast: null pointer");
    cudaStream_t s = b2k::as_stream(stream);
    const bool sat = saturate != 0;
    if (src == B2K_FMT_F32 && dst == B2K_FMT_BF16) return launch<F32ToBf16>(in_dev, out_dev, n, s);
    if (src == B2K_FMT_BF16 && dst == B2K_FMT_F32) return launch<Bf16ToF32>(in_dev, out_dev, n, s);
    if (src == B2K_FMT_F32 && dst == B2K_FMT_E4M3)
        return sat ? launch<F32ToFp8<false, true>>(in_dev, out_dev, n, s)
                   : launch<F32ToFp8<false, false>>(in_dev, out_dev, n, s);
    if (src == B2K_FMT_F32 && dst == B2K_FMT_E5M2)
        return sat ? launch<F32ToFp8<true, true>>(in_dev, out_dev, n, s)
                   : launch<F32ToFp8<true, false>>(in_dev, out_dev, n, s);
    if (src == B2K_FMT_E4M3 && dst == B2K_FMT_F32) return launch<Fp8ToF32<false>>(in_dev, out_dev, n, s);
    if (src == B2K_FMT_E5M2 && dst == B2K_FMT_F32) return launch<Fp8ToF32<true>>(in_dev, out_dev, n, s);
    return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_cast: no conversion from format %d to %d", src, dst);
}

extern "C" int b2k_cast_ex(int src, int dst, int saturate, int rounding, const void *in_dev, void *out_dev,
                           int64_t n, void *stream) {
    B2K_RANGE("b2k_cast_ex");
    if (n < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_cast_ex: negative length %lld", (long long)n);
    if (n > 0 && (!in_dev || !out_dev)) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_cast_ex: null pointer");
    if (rounding < B2K_ROUND_NEAREST || rounding > B2K_ROUND_MIN_INF)
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_cast_ex: unknown rounding mode %d", rounding);
    cudaStream_t s = b2k::as_stream(stream);
    const bool sat = saturate != 0;
    // the nearest-even pairs of b2k_cast
    if (rounding == B2K_ROUND_NEAREST &&
        ((src == B2K_FMT_F32 && dst >= B2K_FMT_BF16 && dst <= B2K_FMT_E5M2) ||
         (dst == B2K_FMT_F32 && src >= B2K_FMT_BF16 && src <= B2K_FMT_E5M2)))
        return b2k_cast(src, dst, saturate, in_dev, out_dev, n, stream);
    if (src == B2K_FMT_F32 && dst == B2K_FMT_BF16) {
        if (rounding == B2K_ROUND_ZERO) return launch_generic<F32ToBf16Mode<1>>(in_dev, out_dev, n, s);
        if (rounding == B2K_ROUND_POS_INF) return launch_generic<F32ToBf16Mode<2>>(in_dev, out_dev, n, s);
        return launch_generic<F32ToBf16Mode<3>>(in_dev, out_dev, n, s);
    }
    if (src == B2K_FMT_F64 && dst == B2K_FMT_BF16 && rounding == B2K_ROUND_NEAREST)
        return launch_generic<F64ToBf16>(in_dev, out_dev, n, s);
    const bool e8_mode = rounding == B2K_ROUND_ZERO || rounding == B2K_ROUND_POS_INF;
    const bool up = rounding == B2K_ROUND_POS_INF;
    if (src == B2K_FMT_F32 && dst == B2K_FMT_E8M0 && e8_mode) {
        if (up) return sat ? launch_generic<F32ToE8m0<true, true>>(in_dev, out_dev, n, s)
                           : launch_generic<F32ToE8m0<true, false>>(in_dev, out_dev, n, s);
        return sat ? launch_generic<F32ToE8m0<false, true>>(in_dev, out_dev, n, s)
                   : launch_generic<F32ToE8m0<false, false>>(in_dev, out_dev, n, s);
    }
    if (src == B2K_FMT_BF16 && dst == B2K_FMT_E8M0 && e8_mode) {
        if (up) return sat ? launch_generic<Bf16ToE8m0<true, true>>(in_dev, out_dev, n, s)
                           : launch_generic<Bf16ToE8m0<true, false>>(in_dev, out_dev, n, s);
        return sat ? launch_generic<Bf16ToE8m0<false, true>>(in_dev, out_dev, n, s)
                   : launch_generic<Bf16ToE8m0<false, false>>(in_dev, out_dev, n, s);
    }
    if (src == B2K_FMT_F64 && dst == B2K_FMT_E8M0 && e8_mode) {
        if (up) return sat ? launch_generic<F64ToE8m0<true, true>>(in_dev, out_dev, n, s)
                           : launch_generic<F64ToE8m0<true, false>>(in_dev, out_dev, n, s);
        return sat ? launch_generic<F64ToE8m0<false, true>>(in_dev, out_dev, n, s)
                   : launch_generic<F64ToE8m0<false, false>>(in_dev, out_dev, n, s);
    }
    if (rounding == B2K_ROUND_NEAREST && (dst == B2K_FMT_E4M3 || dst == B2K_FMT_E5M2)) {
        const bool e5 = dst == B2K_FMT_E5M2;
        if (src == B2K_FMT_F64) {
            if (e5) return sat ? launch_generic<F64ToFp8<true, true>>(in_dev, out_dev, n, s)
                               : launch_generic<F64ToFp8<true, false>>(in_dev, out_dev, n, s);
            return sat ? launch_generic<F64ToFp8<false, true>>(in_dev, out_dev, n, s)
                       : launch_generic<F64ToFp8<false, false>>(in_dev, out_dev, n, s);
        }
        if (src == B2K_FMT_BF16) {
            if (e5) return sat ? launch_generic<Bf16ToFp8<true, true>>(in_dev, out_dev, n, s)
                               : launch_generic<Bf16ToFp8<true, false>>(in_dev, out_dev, n, s);
            return sat ? launch_generic<Bf16ToFp8<false, true>>(in_dev, out_dev, n, s)
                       : launch_generic<Bf16ToFp8<false, false>>(in_dev, out_dev, n, s);
        }
    }
    if (rounding == B2K_ROUND_NEAREST) {
        if (src == B2K_FMT_E8M0 && dst == B2K_FMT_BF16) return launch_generic<E8m0ToBf16>(in_dev, out_dev, n, s);
        if (src == B2K_FMT_E8M0 && dst == B2K_FMT_F32) return launch_generic<E8m0ToF32>(in_dev, out_dev, n, s);
        if (src == B2K_FMT_F32 && dst == B2K_FMT_F16) return launch_generic<F32ToF16>(in_dev, out_dev, n, s);
        if (src == B2K_FMT_F16 && dst == B2K_FMT_F32) return launch_generic<F16ToF32>(in_dev, out_dev, n, s);
    }
    {
        const int rc = cast_value_types(src, dst, sat, rounding, in_dev, out_dev, n, s);
        if (rc != B2K_ERR_UNSUPPORTED) return rc;
    }
    return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_cast_ex: no conversion from format %d to %d with rounding %d", src,
                     dst, rounding);
}
