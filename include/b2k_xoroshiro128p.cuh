/*
 * b2k_xoroshiro128p.cuh -- the xoroshiro128+ device functions of numba-cuda's
 * numba/cuda/random.py for CUDA C++ kernels, bit-compatible with the reference:
 * a kernel written against this header consumes the same stream as a
 * @cuda.jit kernel calling the reference functions on the same states array
 * (as created by b2k_xoroshiro128p_init / create_xoroshiro128p_states).
 *
 * Two styles:
 *   - drop-in: xoroshiro128p_uniform_float32(states, index) etc. load and store
 *     the state in global memory on every draw, like random.py:97-115;
 *   - register resident: xoroshiro128p_generator g(states, index); ... g.uniform_float32();
 *     ... g.store(states, index);  -- the state stays in registers between draws.
 *
 * Compile without -use_fast_math: the normals need the IEEE logf / cosf / cos /
 * sqrt of libdevice to match the reference bit for bit.
 */
#ifndef B2K_XOROSHIRO128P_CUH_
#define B2K_XOROSHIRO128P_CUH_

#include <stdint.h>

/* random.py:47-49: {s0: uint64 @0, s1: uint64 @8}, 16 bytes, aligned */
struct alignas(16) xoroshiro128p_state {
    uint64_t s0, s1;
};

struct xoroshiro128p_generator {
    uint64_t s0, s1;

    __device__ __forceinline__ xoroshiro128p_generator() : s0(0), s1(0) {}
    __device__ __forceinline__ xoroshiro128p_generator(uint64_t a, uint64_t b) : s0(a), s1(b) {}
    __device__ __forceinline__ xoroshiro128p_generator(const xoroshiro128p_state *states, int64_t index) {
        const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(states + index);
        s0 = v.x;
        s1 = v.y;
    }
    __device__ __forceinline__ void store(xoroshiro128p_state *states, int64_t index) const {
        *reinterpret_cast<ulonglong2 *>(states + index) = make_ulonglong2(s0, s1);
    }

    /* random.py:97-115: returns s0+s1 of the state before the update.  The two
     * rotations and the shift are spelled as 32-bit funnel shifts (one instruction
     * per output word): rotl(x, 55) = halves swapped then rotated by 23,
     * rotl(x, 36) = halves swapped then rotated by 4. */
    __device__ __forceinline__ uint64_t next() {
        const uint32_t a_lo = static_cast<uint32_t>(s0), a_hi = static_cast<uint32_t>(s0 >> 32);
        const uint64_t out = s0 + s1;
        const uint32_t b_lo = static_cast<uint32_t>(s1) ^ a_lo, b_hi = static_cast<uint32_t>(s1 >> 32) ^ a_hi;
        const uint32_t r_hi = __funnelshift_l(a_hi, a_lo, 23), r_lo = __funnelshift_l(a_lo, a_hi, 23);
        const uint32_t n0_lo = r_lo ^ b_lo ^ (b_lo << 14);
        const uint32_t n0_hi = r_hi ^ b_hi ^ __funnelshift_l(b_lo, b_hi, 14);
        const uint32_t n1_hi = __funnelshift_l(b_hi, b_lo, 4), n1_lo = __funnelshift_l(b_lo, b_hi, 4);
        s0 = (static_cast<uint64_t>(n0_hi) << 32) | n0_lo;
        s1 = (static_cast<uint64_t>(n1_hi) << 32) | n1_lo;
        return out;
    }
    /* random.py:146-156.  (x >> 11) * 2^-53 is exact in float64, so rounding the
     * 53-bit integer to float32 first and scaling by a power of two gives the
     * same bits as rounding the float64 product.  Clearing the low 11 bits and
     * scaling by 2^-64 is the same value again (a power-of-two factor moved from
     * the integer into the scale) and saves the 64-bit shift. */
    __device__ __forceinline__ double uniform_float64() {
        return __ull2double_rn(next() & 0xFFFFFFFFFFFFF800ull) * 0x1p-64;
    }
    __device__ __forceinline__ float uniform_float32() {
        return __ull2float_rn(next() & 0xFFFFFFFFFFFFF800ull) * 0x1p-64f;
    }
    /* random.py:192-238: Box-Muller, cosine branch, from two float32 uniforms */
    __device__ __forceinline__ float normal_float32() {
        const float u1 = uniform_float32();
        const float u2 = uniform_float32();
        return sqrtf(-2.0f * logf(u1)) * cosf(6.2831855f * u2);
    }
    __device__ __forceinline__ double normal_float64() {
        const float u1 = uniform_float32();
        const float u2 = uniform_float32();
        return sqrt(-2.0 * static_cast<double>(logf(u1))) * cos(6.283185307179586 * static_cast<double>(u2));
    }
    /* random.py:119-142: advance by 2^64 steps */
    __device__ __forceinline__ void jump() {
        const uint64_t poly[2] = {0xBEAC0467EBA5FACBull, 0xD86B048B86AA9922ull};
        uint64_t a0 = 0, a1 = 0;
        for (int w = 0; w < 2; ++w)
            for (int b = 0; b < 64; ++b) {
                if ((poly[w] >> b) & 1ull) { a0 ^= s0; a1 ^= s1; }
                (void)next();
            }
        s0 = a0;
        s1 = a1;
    }
};

/* ---- drop-in functions with the reference's names and (states, index) arguments ---- */
#define B2K_XORO_DROP_IN(NAME, TYPE, CALL)                                                   \
    __device__ __forceinline__ TYPE NAME(xoroshiro128p_state *states, int64_t index) {       \
        xoroshiro128p_generator g(states, index);                                            \
        const TYPE r = g.CALL();                                                             \
        g.store(states, index);                                                              \
        return r;                                                                            \
    }
B2K_XORO_DROP_IN(xoroshiro128p_next, uint64_t, next)
B2K_XORO_DROP_IN(xoroshiro128p_uniform_float32, float, uniform_float32)
B2K_XORO_DROP_IN(xoroshiro128p_uniform_float64, double, uniform_float64)
B2K_XORO_DROP_IN(xoroshiro128p_normal_float32, float, normal_float32)
B2K_XORO_DROP_IN(xoroshiro128p_normal_float64, double, normal_float64)
#undef B2K_XORO_DROP_IN

__device__ __forceinline__ void xoroshiro128p_jump(xoroshiro128p_state *states, int64_t index) {
    xoroshiro128p_generator g(states, index);
    g.jump();
    g.store(states, index);
}

#endif /* B2K_XOROSHIRO128P_CUH_ */
