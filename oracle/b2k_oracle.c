/*
 * CPU oracle for the numba-cuda library kernels (TEST INFRASTRUCTURE ONLY).
 *
 * This file is a plain-C restatement of the algorithms the reference runs for
 * reduce / transpose / xoroshiro128p / bf16+fp8 conversion.  It exists so the
 * CUDA kernels can be checked bit for bit on the host.  Nothing in the shipped
 * package may link, load or call it: only the test-suite, the smoke check and
 * the CPU-baseline leg of the benchmark do.
 *
 * Every function names the reference location it follows (paths are relative
 * to the numba-cuda project root).
 *
 * Parity status of this oracle:
 *   - RNG states / uniforms: pinned against values produced by executing the
 *     reference's own CPU-jitted functions (see tests/golden/make_golden.py).
 *   - fp8 / bf16: pinned against the known-answer bytes of the reference's
 *     tests and against the host path of the vendored cuda_fp8.hpp /
 *     cuda_bf16.hpp compiled into oracle/_ref/ (see oracle/Makefile).
 *   - normals: use the host libm (logf / cos / cosf / sqrt); the reference's
 *     GPU kernels use libdevice, so normals from this file are a tolerance
 *     check only.  Bit parity for normals is pinned by GPU-generated fixtures.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stddef.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* xoroshiro128+                                                       */
/* ------------------------------------------------------------------ */

/* numba_cuda/numba/cuda/random.py:47-50 : {s0:u64 @0, s1:u64 @8}, 16 bytes. */
typedef struct { uint64_t s0, s1; } xoro_state;

static inline uint64_t rotl64(uint64_t x, unsigned k) {
    /* random.py:89-93 */
    return (x << k) | (x >> (64u - k));
}

/* random.py:63-85 : SplitMix64 finaliser of the seed, copied into both words. */
ORACLE_API void oracle_xoro_seed(xoro_state *st, uint64_t seed) {
    uint64_t z = seed + UINT64_C(0x9E3779B97F4A7C15);
    z = (z ^ (z >> 30)) * UINT64_C(0xBF58476D1CE4E5B9);
    z = (z ^ (z >> 27)) * UINT64_C(0x94D049BB133111EB);
    z = z ^ (z >> 31);
    st->s0 = z;
    st->s1 = z;
}

/* random.py:97-115 : output is s0+s1 of the state *before* the update. */
ORACLE_API uint64_t oracle_xoro_next(xoro_state *st) {
    uint64_t a = st->s0, b = st->s1;
    uint64_t out = a + b;
    b ^= a;
    st->s0 = rotl64(a, 55) ^ b ^ (b << 14);
    st->s1 = rotl64(b, 36);
    return out;
}

/* random.py:119-142 : advance by 2^64 steps. */
ORACLE_API void oracle_xoro_jump(xoro_state *st) {
    static const uint64_t poly[2] = { UINT64_C(0xBEAC0467EBA5FACB),
                                      UINT64_C(0xD86B048B86AA9922) };
    uint64_t acc0 = 0, acc1 = 0;
    for (int w = 0; w < 2; ++w) {
        for (int bit = 0; bit < 64; ++bit) {
            if ((poly[w] >> bit) & 1u) {
                acc0 ^= st->s0;
                acc1 ^= st->s1;
            }
            (void)oracle_xoro_next(st);
        }
    }
    st->s0 = acc0;
    st->s1 = acc1;
}

/* random.py:242-257 : serial chain, state[i] = jump(state[i-1]). */
ORACLE_API void oracle_xoro_init_states(xoro_state *states, int64_t n,
                                        uint64_t seed, uint64_t subsequence_start) {
    if (n < 1) return;
    oracle_xoro_seed(&states[0], seed);
    for (uint64_t k = 0; k < subsequence_start; ++k) oracle_xoro_jump(&states[0]);
    for (int64_t i = 1; i < n; ++i) {
        states[i] = states[i - 1];
        oracle_xoro_jump(&states[i]);
    }
}

/* random.py:146-149 */
ORACLE_API double oracle_u64_to_unit_f64(uint64_t x) {
    return (double)(x >> 11) * (1.0 / 9007199254740992.0);
}
/* random.py:153-156 : the f64 value rounded (nearest-even) to f32. */
ORACLE_API float oracle_u64_to_unit_f32(uint64_t x) {
    return (float)oracle_u64_to_unit_f64(x);
}

/* random.py:160-184 */
ORACLE_API float oracle_xoro_uniform_f32(xoro_state *st) {
    return oracle_u64_to_unit_f32(oracle_xoro_next(st));
}
ORACLE_API double oracle_xoro_uniform_f64(xoro_state *st) {
    return oracle_u64_to_unit_f64(oracle_xoro_next(st));
}

/* random.py:192-213 : Box-Muller, cosine branch, all-f32 arithmetic. */
ORACLE_API float oracle_xoro_normal_f32(xoro_state *st) {
    float u1 = oracle_xoro_uniform_f32(st);
    float u2 = oracle_xoro_uniform_f32(st);
    const float two_pi = (float)(2.0 * 3.141592653589793);
    return sqrtf(-2.0f * logf(u1)) * cosf(two_pi * u2);
}
/* random.py:217-238 : uniforms are f32; log is the f32 log; the rest is f64. */
ORACLE_API double oracle_xoro_normal_f64(xoro_state *st) {
    float u1 = oracle_xoro_uniform_f32(st);
    float u2 = oracle_xoro_uniform_f32(st);
    const double two_pi = 2.0 * 3.141592653589793;
    return sqrt(-2.0 * (double)logf(u1)) * cos(two_pi * (double)u2);
}

/* Bulk drivers in the layout of the reference's test kernels
 * (tests/cudapy/test_random.py:29-53): out[tid*count + i] = draw(states, tid).
 * kind: 0 uniform f32, 1 uniform f64, 2 normal f32, 3 normal f64. */
ORACLE_API void oracle_xoro_fill(xoro_state *states, int64_t n, int kind,
                                 void *out, int64_t count) {
    for (int64_t t = 0; t < n; ++t) {
        for (int64_t i = 0; i < count; ++i) {
            switch (kind) {
            case 0: ((float *)out)[t * count + i] = oracle_xoro_uniform_f32(&states[t]); break;
            case 1: ((double *)out)[t * count + i] = oracle_xoro_uniform_f64(&states[t]); break;
            case 2: ((float *)out)[t * count + i] = oracle_xoro_normal_f32(&states[t]); break;
            default: ((double *)out)[t * count + i] = oracle_xoro_normal_f64(&states[t]); break;
            }
        }
    }
}

/* ------------------------------------------------------------------ */
/* fp8 (E4M3 / E5M2) and bf16 conversions                              */
/* ------------------------------------------------------------------ */

/* Encode a double to an fp8 code: integer round-to-nearest-even with optional
 * saturation.  Follows numba_cuda/numba/cuda/include/12/cuda_fp8.hpp:119-229.
 * interp: 0 = E4M3, 1 = E5M2.  sat: 0 = NOSAT, 1 = SATFINITE. */
ORACLE_API uint8_t oracle_f64_to_fp8(double x, int sat, int interp) {
    uint64_t bits;
    memcpy(&bits, &x, sizeof bits);

    const int e4m3 = (interp == 0);
    const unsigned bias = e4m3 ? 7u : 15u;
    const unsigned sig_bits = e4m3 ? 4u : 3u; /* significand incl. hidden bit */
    const uint8_t mant_mask = e4m3 ? 0x7u : 0x3u;
    const uint8_t max_norm = e4m3 ? 0x7Eu : 0x7Bu;
    /* |x| at or below half the smallest denormal rounds to zero */
    const uint64_t half_min_denorm = e4m3 ? UINT64_C(0x3F50000000000000)
                                          : UINT64_C(0x3EE0000000000000);
    /* above (max normal + half ulp) is overflow; E5M2 bound is exclusive-1 so
     * one comparison serves both formats */
    const uint64_t overflow_above = e4m3 ? UINT64_C(0x407D000000000000)
                                         : UINT64_C(0x40EE000000000000) - 1u;
    const uint64_t min_norm = e4m3 ? UINT64_C(0x3F90000000000000)
                                   : UINT64_C(0x3F10000000000000);
    const uint64_t inf_bits = UINT64_C(0x7FF0000000000000);
    const uint64_t half_ulp = UINT64_C(1) << (53u - sig_bits - 1u);

    const uint8_t sign = (uint8_t)((bits >> 63) << 7);
    const uint8_t e8 = (uint8_t)((((unsigned)(bits >> 52)) & 0x7FFu) - 1023u + bias);
    uint8_t mant = (uint8_t)(bits >> (53u - sig_bits)) & mant_mask;
    const uint64_t mag = bits & UINT64_C(0x7FFFFFFFFFFFFFFF);
    uint8_t code;

    if (mag <= half_min_denorm) {
        code = 0;
    } else if (mag > inf_bits) {              /* NaN */
        code = e4m3 ? 0x7Fu : (uint8_t)(0x7Eu | mant);
    } else if (mag > overflow_above) {        /* too large, incl. infinities */
        if (sat) code = max_norm;
        else code = e4m3 ? 0x7Fu : 0x7Cu;
    } else if (mag >= min_norm) {             /* normal result */
        code = (uint8_t)((e8 << (sig_bits - 1u)) | mant);
        uint64_t dropped = bits & ((half_ulp << 1) - 1u);
        if (dropped > half_ulp || (dropped == half_ulp && (mant & 1u)))
            code = (uint8_t)(code + 1u);
    } else {                                  /* denormal result */
        uint8_t shift = (uint8_t)(1u - e8);
        mant |= (uint8_t)(1u << (sig_bits - 1u));
        code = (uint8_t)(mant >> shift);
        uint64_t dropped = (bits | (UINT64_C(1) << 52)) &
                           ((half_ulp << (shift + 1u)) - 1u);
        uint64_t mid = half_ulp << shift;
        if (dropped > mid || (dropped == mid && (code & 1u)))
            code = (uint8_t)(code + 1u);
    }
    return (uint8_t)(code | sign);
}

/* cuda_fp8.hpp:245-288 (host branch): canonicalise NaN, widen, encode. */
ORACLE_API uint8_t oracle_f32_to_fp8(float x, int sat, int interp) {
    uint32_t b;
    memcpy(&b, &x, sizeof b);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) b = 0x7FFFFFFFu;
    float fx;
    memcpy(&fx, &b, sizeof fx);
    return oracle_f64_to_fp8((double)fx, sat, interp);
}

/* cuda_fp8.hpp:473-523 (host branch): fp8 code -> IEEE half bit pattern. */
ORACLE_API uint16_t oracle_fp8_to_f16bits(uint8_t code, int interp) {
    uint16_t h = (uint16_t)((uint16_t)code << 8);
    if (interp == 1) {                        /* E5M2 is a truncated half */
        if ((h & 0x7FFFu) > 0x7C00u) h = 0x7FFFu;
        return h;
    }
    uint16_t sign = h & 0x8000u;
    uint16_t expo = (uint16_t)(((h & 0x7800u) >> 1) + 0x2000u);
    uint16_t mant = (uint16_t)((h & 0x0700u) >> 1);
    if ((code & 0x7Fu) == 0x7Fu) return 0x7FFFu;
    if (expo == 0x2000u) {                    /* zero or E4M3 denormal */
        if (mant != 0) {
            mant = (uint16_t)(mant << 1);
            while ((mant & 0x0400u) == 0) {
                mant = (uint16_t)(mant << 1);
                expo = (uint16_t)(expo - 0x0400u);
            }
            mant &= 0x03FFu;
        } else {
            expo = 0;
        }
    }
    return (uint16_t)(sign | expo | mant);
}

/* cuda_fp8.hpp:319-356 (host branch): half bits -> float.  NaN becomes
 * 0x7FFFFFFF with the sign dropped. */
ORACLE_API float oracle_f16bits_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u;
    uint32_t expo = (h >> 10) & 0x1Fu;
    uint32_t mant = (uint32_t)(h & 0x3FFu) << 13;
    if (expo == 0x1Fu) {
        if (mant != 0) { sign = 0; mant = 0x7FFFFFu; }
        expo = 0xFFu;
    } else if (expo == 0) {
        if (mant != 0) {
            uint32_t top;
            expo = 0x71u;
            do {
                top = mant & 0x400000u;
                mant <<= 1;
                --expo;
            } while (top == 0);
            mant &= 0x7FFFFFu;
        }
    } else {
        expo += 0x70u;
    }
    uint32_t u = (sign << 31) | (expo << 23) | mant;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* fp8 value type -> float: cuda_fp8.hpp operator float (12/:1651) =
 * fp8 -> half raw -> float. */
ORACLE_API float oracle_fp8_to_f32(uint8_t code, int interp) {
    return oracle_f16bits_to_f32(oracle_fp8_to_f16bits(code, interp));
}

/* numba_cuda/numba/cuda/include/12/cuda_bf16.hpp:404-503 (host branch):
 * f32 -> bf16, round to nearest even, every NaN becomes 0x7FFF. */
ORACLE_API uint16_t oracle_f32_to_bf16(float x) {
    uint32_t b;
    memcpy(&b, &x, sizeof b);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu;
    uint16_t hi = (uint16_t)(b >> 16);
    uint32_t rest = b << 16;
    if (rest > 0x80000000u || (rest == 0x80000000u && (hi & 1u))) ++hi;
    return hi;
}

/* cuda_bf16.hpp:582-609 (host branch): bf16 -> f32 is a 16-bit left shift. */
ORACLE_API float oracle_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* Bulk cast.  src/dst codes: 0 f32, 1 bf16, 2 fp8 e4m3, 3 fp8 e5m2.
 * Returns 0, or -1 for an unsupported pair. */
ORACLE_API int oracle_cast(int src, int dst, int sat, const void *in, void *out, int64_t n) {
    if (src == 0 && dst == 1) {
        for (int64_t i = 0; i < n; ++i) ((uint16_t *)out)[i] = oracle_f32_to_bf16(((const float *)in)[i]);
    } else if (src == 1 && dst == 0) {
        for (int64_t i = 0; i < n; ++i) ((float *)out)[i] = oracle_bf16_to_f32(((const uint16_t *)in)[i]);
    } else if (src == 0 && (dst == 2 || dst == 3)) {
        for (int64_t i = 0; i < n; ++i) ((uint8_t *)out)[i] = oracle_f32_to_fp8(((const float *)in)[i], sat, dst - 2);
    } else if ((src == 2 || src == 3) && dst == 0) {
        for (int64_t i = 0; i < n; ++i) ((float *)out)[i] = oracle_fp8_to_f32(((const uint8_t *)in)[i], src - 2);
    } else {
        return -1;
    }
    return 0;
}

/* ---- further conversions (rounding modes, f64, E8M0, f16) -------------------- */

/* cuda_bf16.hpp:505-553 (host branches): f32 -> bf16 with directed rounding.
 * mode: 1 = toward zero, 2 = toward +inf, 3 = toward -inf (cudaRoundMode order);
 * 0 = nearest even.  NaN gives 0x7FFF in every mode. */
ORACLE_API uint16_t oracle_f32_to_bf16_mode(float x, int mode) {
    if (mode == 0) return oracle_f32_to_bf16(x);
    uint32_t b;
    memcpy(&b, &x, sizeof b);
    if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu;
    uint16_t hi = (uint16_t)(b >> 16);
    uint32_t rest = b << 16;
    uint32_t negative = b >> 31;
    if (mode == 3 && rest != 0 && negative) ++hi;   /* more negative */
    if (mode == 2 && rest != 0 && !negative) ++hi;  /* more positive */
    return hi;
}

/* cuda_bf16.hpp:452-470 (host branch): f64 -> bf16, nearest even.  The double is
 * first rounded to float "to odd" (sticky bit kept in the last place) so that the
 * second rounding to bf16 sees every discarded bit. */
ORACLE_API uint16_t oracle_f64_to_bf16(double x) {
    float f = (float)x;
    double back = (double)f;
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    int not_nan = ((u << 1) <= 0xFF000000u);
    if (x > 0.0 && back > x) u--;
    if (x < 0.0 && back < x) u--;
    if (back != x && not_nan) u |= 1u;
    memcpy(&f, &u, sizeof f);
    return oracle_f32_to_bf16(f);
}

/* cuda_fp8.hpp:546-589 (host branch): bf16 bits -> E8M0 (an 8-bit biased exponent,
 * 0xFF = NaN).  mode: 1 = toward zero, 2 = toward +inf. */
ORACLE_API uint8_t oracle_bf16_to_e8m0(uint16_t h, int sat, int mode) {
    uint8_t res = (uint8_t)(h >> 7);
    if (mode == 2) {
        if ((h & 0x007Fu) && ((h & 0x7FFFu) > 0x0040u) && ((h & 0x7FFFu) < 0x7F80u)) res++;
    }
    if (sat) {
        if (((h & 0x7FFFu) <= 0x7F80u) && res == 0xFFu) res--;
    }
    return res;
}

/* cuda_fp8.hpp:652-687 (host branches of the bf16 helpers) and :689-740:
 * f32 -> E8M0 goes through bf16 with the same directed rounding (of |x| for
 * the upward mode). */
ORACLE_API uint8_t oracle_f32_to_e8m0(float x, int sat, int mode) {
    uint32_t b;
    memcpy(&b, &x, sizeof b);
    uint16_t h;
    if (mode == 1) {
        h = ((b & 0x7FFFFFFFu) > 0x7F800000u) ? 0x7FFFu : (uint16_t)(b >> 16);
    } else {
        uint32_t a = (b << 1) >> 1;                      /* |x| */
        if (a > 0x7F800000u) h = 0x7FFFu;
        else if (a < 0x7F800000u && (a & 0xFFFFu) != 0) h = (uint16_t)((a >> 16) + 1u);
        else h = (uint16_t)(a >> 16);
    }
    return oracle_bf16_to_e8m0(h, sat, mode);
}

/* cuda_fp8.hpp:817-831: E8M0 -> bf16 bits (2^-127 is the bf16 denormal 0x0040). */
ORACLE_API uint16_t oracle_e8m0_to_bf16(uint8_t e) {
    if (e == 0xFFu) return 0x7FFFu;
    if (e == 0u) return 0x0040u;
    return (uint16_t)((uint16_t)e << 7);
}

/* cuda_fp8.hpp:442-470: bf16 bits -> fp8 goes through float (a 16-bit left shift,
 * exact) and then the float encoder. */
ORACLE_API uint8_t oracle_bf16_to_fp8(uint16_t h, int sat, int interp) {
    return oracle_f32_to_fp8(oracle_bf16_to_f32(h), sat, interp);
}

/* cuda_fp8.hpp:772-806: f64 -> E8M0.  The double is rounded to float "to odd"
 * (the sticky bit of everything discarded is kept in the last place), then the
 * float encoder runs; its directed rounding therefore sees every discarded bit. */
ORACLE_API uint8_t oracle_f64_to_e8m0(double x, int sat, int mode) {
    float f = (float)x;
    double back = (double)f;
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    int not_nan = ((u << 1) <= 0xFF000000u);
    if (x > 0.0 && back > x) u--;
    if (x < 0.0 && back < x) u--;
    if (back != x && not_nan) u |= 1u;
    memcpy(&f, &u, sizeof f);
    return oracle_f32_to_e8m0(f, sat, mode);
}

/* Bulk form of the above.  Formats: 0 f32, 1 bf16, 2 e4m3, 3 e5m2, 4 f64, 6 e8m0. */
ORACLE_API int oracle_cast_ex(int src, int dst, int sat, int mode, const void *in, void *out, int64_t n) {
    if (src == 4 && (dst == 2 || dst == 3)) {
        for (int64_t i = 0; i < n; ++i) ((uint8_t *)out)[i] = oracle_f64_to_fp8(((const double *)in)[i], sat, dst - 2);
    } else if (src == 1 && (dst == 2 || dst == 3)) {
        for (int64_t i = 0; i < n; ++i) ((uint8_t *)out)[i] = oracle_bf16_to_fp8(((const uint16_t *)in)[i], sat, dst - 2);
    } else if (src == 4 && dst == 6) {
        for (int64_t i = 0; i < n; ++i) ((uint8_t *)out)[i] = oracle_f64_to_e8m0(((const double *)in)[i], sat, mode);
    } else if (src == 0 && dst == 1) {
        for (int64_t i = 0; i < n; ++i) ((uint16_t *)out)[i] = oracle_f32_to_bf16_mode(((const float *)in)[i], mode);
    } else if (src == 4 && dst == 1) {
        for (int64_t i = 0; i < n; ++i) ((uint16_t *)out)[i] = oracle_f64_to_bf16(((const double *)in)[i]);
    } else if (src == 0 && dst == 6) {
        for (int64_t i = 0; i < n; ++i) ((uint8_t *)out)[i] = oracle_f32_to_e8m0(((const float *)in)[i], sat, mode);
    } else if (src == 1 && dst == 6) {
        for (int64_t i = 0; i < n; ++i) ((uint8_t *)out)[i] = oracle_bf16_to_e8m0(((const uint16_t *)in)[i], sat, mode);
    } else if (src == 6 && dst == 1) {
        for (int64_t i = 0; i < n; ++i) ((uint16_t *)out)[i] = oracle_e8m0_to_bf16(((const uint8_t *)in)[i]);
    } else if (src == 6 && dst == 0) {
        for (int64_t i = 0; i < n; ++i) ((float *)out)[i] = oracle_bf16_to_f32(oracle_e8m0_to_bf16(((const uint8_t *)in)[i]));
    } else {
        return -1;
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* reduce and transpose                                                */
/* ------------------------------------------------------------------ */

/* The reference's CPU path for cuda.reduce is a sequential left fold that
 * starts from init (numba_cuda/numba/cuda/simulator/reduction.py:7-16).
 * op: 0 add, 1 mul, 2 max, 3 min.  Floating point only (the integer cases are
 * checked with NumPy, where wrap-around is exact). */
ORACLE_API double oracle_fold_f64(const double *x, int64_t n, double init, int op) {
    double acc = init;
    for (int64_t i = 0; i < n; ++i) {
        double v = x[i];
        switch (op) {
        case 0: acc = acc + v; break;
        case 1: acc = acc * v; break;
        case 2: acc = (v > acc) ? v : acc; break;
        default: acc = (v < acc) ? v : acc; break;
        }
    }
    return acc;
}
ORACLE_API float oracle_fold_f32(const float *x, int64_t n, float init, int op) {
    float acc = init;
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i];
        switch (op) {
        case 0: acc = acc + v; break;
        case 1: acc = acc * v; break;
        case 2: acc = (v > acc) ? v : acc; break;
        default: acc = (v < acc) ? v : acc; break;
        }
    }
    return acc;
}

/* numba_cuda/numba/cuda/kernels/transpose.py:42-57 : b[j, i] = a[i, j] for
 * items of any size, arbitrary input byte strides, C-contiguous output. */
ORACLE_API void oracle_transpose2d(const void *in, void *out, int64_t rows, int64_t cols,
                                   int64_t in_stride0, int64_t in_stride1, int64_t itemsize) {
    const char *src = (const char *)in;
    char *dst = (char *)out;
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t j = 0; j < cols; ++j)
            memcpy(dst + (j * rows + i) * itemsize,
                   src + i * in_stride0 + j * in_stride1, (size_t)itemsize);
}
