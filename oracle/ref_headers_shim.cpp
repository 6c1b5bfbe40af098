// Thin C wrappers over the HOST code paths of the reference's vendored CUDA
// headers (numba_cuda/numba/cuda/include/12/cuda_fp8.hpp, cuda_bf16.hpp).
// Compiled with g++ against the headers where they lie in the reference tree;
// the result (oracle/_ref/libb2k_ref_headers.so) is the reference's own CPU
// implementation of the conversion arithmetic.  Test infrastructure only.
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>
#include <cuda_fp8.h>
#include <cuda_bf16.h>


extern "C" {

// __nv_cvt_float_to_fp8  (cuda_fp8.hpp:245-288)
uint8_t ref_cvt_float_to_fp8(float x, int sat, int interp) {
    return (uint8_t)__nv_cvt_float_to_fp8(
        x, sat ? __NV_SATFINITE : __NV_NOSAT, interp ? __NV_E5M2 : __NV_E4M3);
}
// __nv_cvt_double_to_fp8 (cuda_fp8.hpp:119-229)
uint8_t ref_cvt_double_to_fp8(double x, int sat, int interp) {
    return (uint8_t)__nv_cvt_double_to_fp8(
        x, sat ? __NV_SATFINITE : __NV_NOSAT, interp ? __NV_E5M2 : __NV_E4M3);
}
// __nv_cvt_fp8_to_halfraw (cuda_fp8.hpp:473-523)
uint16_t ref_cvt_fp8_to_halfraw(uint8_t code, int interp) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code,
                                           interp ? __NV_E5M2 : __NV_E4M3);
    return h.x;
}
// float(__nv_fp8_e4m3) / float(__nv_fp8_e5m2): the value types' cast operator.
float ref_fp8_to_float(uint8_t code, int interp) {
    if (interp) { __nv_fp8_e5m2 v; v.__x = code; return (float)v; }
    __nv_fp8_e4m3 v; v.__x = code; return (float)v;
}
// __nv_fp8_e4m3(float) / __nv_fp8_e5m2(float): the value types' constructor.
uint8_t ref_fp8_from_float(float x, int interp) {
    if (interp) { __nv_fp8_e5m2 v(x); return v.__x; }
    __nv_fp8_e4m3 v(x); return v.__x;
}
// __float2bfloat16_rn (cuda_bf16.hpp:487-503)
uint16_t ref_float2bfloat16_rn(float x) {
    __nv_bfloat16_raw r = (__nv_bfloat16_raw)__float2bfloat16_rn(x);
    return r.x;
}
// __bfloat162float (cuda_bf16.hpp:606-609)
float ref_bfloat162float(uint16_t bits) {
    __nv_bfloat16_raw r; r.x = bits;
    return __bfloat162float((__nv_bfloat16)r);
}

// __float2bfloat16_rz / _ru / _rd (cuda_bf16.hpp:505-553); mode as cudaRoundMode
uint16_t ref_float2bfloat16_mode(float x, int mode) {
    __nv_bfloat16 v = mode == 1 ? __float2bfloat16_rz(x) : mode == 2 ? __float2bfloat16_ru(x)
                    : mode == 3 ? __float2bfloat16_rd(x) : __float2bfloat16_rn(x);
    return ((__nv_bfloat16_raw)v).x;
}
// __double2bfloat16 (cuda_bf16.hpp:444-470)
uint16_t ref_double2bfloat16(double x) { return ((__nv_bfloat16_raw)__double2bfloat16(x)).x; }
// __nv_cvt_float_to_e8m0 (cuda_fp8.hpp:689-740), __nv_cvt_bfloat16raw_to_e8m0 (:546-589),
// __nv_cvt_e8m0_to_bf16raw (:833-851)
uint8_t ref_cvt_float_to_e8m0(float x, int sat, int mode) {
    return (uint8_t)__nv_cvt_float_to_e8m0(x, sat ? __NV_SATFINITE : __NV_NOSAT,
                                           mode == 2 ? cudaRoundPosInf : cudaRoundZero);
}
uint8_t ref_cvt_bfloat16raw_to_e8m0(uint16_t bits, int sat, int mode) {
    __nv_bfloat16_raw r; r.x = bits;
    return (uint8_t)__nv_cvt_bfloat16raw_to_e8m0(r, sat ? __NV_SATFINITE : __NV_NOSAT,
                                                 mode == 2 ? cudaRoundPosInf : cudaRoundZero);
}
uint16_t ref_cvt_e8m0_to_bf16raw(uint8_t e) { return __nv_cvt_e8m0_to_bf16raw((__nv_fp8_storage_t)e).x; }
// __nv_cvt_bfloat16raw_to_fp8 (cuda_fp8.hpp:442-450)
uint8_t ref_cvt_bfloat16raw_to_fp8(uint16_t bits, int sat, int interp) {
    __nv_bfloat16_raw r; r.x = bits;
    return (uint8_t)__nv_cvt_bfloat16raw_to_fp8(r, sat ? __NV_SATFINITE : __NV_NOSAT,
                                                interp ? __NV_E5M2 : __NV_E4M3);
}
// __nv_cvt_double_to_e8m0 (cuda_fp8.hpp:797-806)
uint8_t ref_cvt_double_to_e8m0(double x, int sat, int mode) {
    return (uint8_t)__nv_cvt_double_to_e8m0(x, sat ? __NV_SATFINITE : __NV_NOSAT,
                                            mode == 2 ? cudaRoundPosInf : cudaRoundZero);
}
// the two-element forms: x in the low byte, y in the high byte
uint16_t ref_cvt_double2_to_fp8x2(double x, double y, int sat, int interp) {
    double2 v; v.x = x; v.y = y;
    return (uint16_t)__nv_cvt_double2_to_fp8x2(v, sat ? __NV_SATFINITE : __NV_NOSAT,
                                               interp ? __NV_E5M2 : __NV_E4M3);
}
uint16_t ref_cvt_float2_to_fp8x2(float x, float y, int sat, int interp) {
    float2 v; v.x = x; v.y = y;
    return (uint16_t)__nv_cvt_float2_to_fp8x2(v, sat ? __NV_SATFINITE : __NV_NOSAT,
                                              interp ? __NV_E5M2 : __NV_E4M3);
}
uint16_t ref_cvt_bfloat16raw2_to_fp8x2(uint16_t x, uint16_t y, int sat, int interp) {
    __nv_bfloat162_raw v; v.x = x; v.y = y;
    return (uint16_t)__nv_cvt_bfloat16raw2_to_fp8x2(v, sat ? __NV_SATFINITE : __NV_NOSAT,
                                                    interp ? __NV_E5M2 : __NV_E4M3);
}
uint16_t ref_cvt_float2_to_e8m0x2(float x, float y, int sat, int mode) {
    float2 v; v.x = x; v.y = y;
    return (uint16_t)__nv_cvt_float2_to_e8m0x2(v, sat ? __NV_SATFINITE : __NV_NOSAT,
                                               mode == 2 ? cudaRoundPosInf : cudaRoundZero);
}
uint16_t ref_cvt_double2_to_e8m0x2(double x, double y, int sat, int mode) {
    double2 v; v.x = x; v.y = y;
    return (uint16_t)__nv_cvt_double2_to_e8m0x2(v, sat ? __NV_SATFINITE : __NV_NOSAT,
                                                mode == 2 ? cudaRoundPosInf : cudaRoundZero);
}
uint16_t ref_cvt_bfloat162raw_to_e8m0x2(uint16_t x, uint16_t y, int sat, int mode) {
    __nv_bfloat162_raw v; v.x = x; v.y = y;
    return (uint16_t)__nv_cvt_bfloat162raw_to_e8m0x2(v, sat ? __NV_SATFINITE : __NV_NOSAT,
                                                     mode == 2 ? cudaRoundPosInf : cudaRoundZero);
}

}  // extern "C"

// Bulk loops split over `threads` host threads (std::thread; <=0 means all cores).
template <class F> static void parallel_for(int64_t n, int threads, F body) {
    int t = threads > 0 ? threads : (int)std::thread::hardware_concurrency();
    if (t < 1) t = 1;
    if (n < 4096 || t == 1) { body(0, n); return; }
    std::vector<std::thread> pool;
    int64_t chunk = (n + t - 1) / t;
    for (int k = 0; k < t; ++k) {
        int64_t lo = k * chunk, hi = lo + chunk < n ? lo + chunk : n;
        if (lo >= hi) break;
        pool.emplace_back([=] { body(lo, hi); });
    }
    for (auto& th : pool) th.join();
}
extern "C" {
void ref_bulk_f32_to_fp8(const float* in, uint8_t* out, int64_t n, int sat, int interp, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_cvt_float_to_fp8(in[i], sat, interp); });
}
void ref_bulk_fp8_to_f32(const uint8_t* in, float* out, int64_t n, int interp, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_fp8_to_float(in[i], interp); });
}
void ref_bulk_f32_to_bf16(const float* in, uint16_t* out, int64_t n, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_float2bfloat16_rn(in[i]); });
}
void ref_bulk_bf16_to_f32(const uint16_t* in, float* out, int64_t n, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_bfloat162float(in[i]); });
}

void ref_bulk_f64_to_fp8(const double* in, uint8_t* out, int64_t n, int sat, int interp, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_cvt_double_to_fp8(in[i], sat, interp); });
}
void ref_bulk_bf16_to_fp8(const uint16_t* in, uint8_t* out, int64_t n, int sat, int interp, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_cvt_bfloat16raw_to_fp8(in[i], sat, interp); });
}
void ref_bulk_f64_to_e8m0(const double* in, uint8_t* out, int64_t n, int sat, int mode, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) out[i] = ref_cvt_double_to_e8m0(in[i], sat, mode); });
}

}  // extern "C"

// ---- the value types' constructors and conversion operators, bulk ----------------
// Format codes as in include/b2k.h: 0 f32, 1 bf16 (raw bits), 2 e4m3, 3 e5m2, 4 f64,
// 5 f16 (raw bits), 6 e8m0, 7..10 int8/16/32/64, 11..14 uint8/16/32/64, 15 bool.
// An 8-bit integer source is widened to 16 bits first, as numba's typing does
// before it picks the constructor (the C++ types have none from char).
#include <cuda_fp16.h>

namespace {
template <class FP8, class Src> inline uint8_t construct(Src v) { FP8 r(v); return r.__x; }

template <class FP8>
void value_from(int src, const void* in, uint8_t* out, int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
        switch (src) {
            case 0: out[i] = construct<FP8>(((const float*)in)[i]); break;
            case 1: { __nv_bfloat16_raw r; r.x = ((const uint16_t*)in)[i];
                      out[i] = construct<FP8>((__nv_bfloat16)r); break; }
            case 4: out[i] = construct<FP8>(((const double*)in)[i]); break;
            case 5: { __half_raw r; r.x = ((const uint16_t*)in)[i];
                      out[i] = construct<FP8>((__half)r); break; }
            case 7: out[i] = construct<FP8>((short)((const int8_t*)in)[i]); break;
            case 8: out[i] = construct<FP8>((short)((const int16_t*)in)[i]); break;
            case 9: out[i] = construct<FP8>((int)((const int32_t*)in)[i]); break;
            case 10: out[i] = construct<FP8>((long long)((const int64_t*)in)[i]); break;
            case 11: out[i] = construct<FP8>((unsigned short)((const uint8_t*)in)[i]); break;
            case 12: out[i] = construct<FP8>((unsigned short)((const uint16_t*)in)[i]); break;
            case 13: out[i] = construct<FP8>((unsigned int)((const uint32_t*)in)[i]); break;
            case 14: out[i] = construct<FP8>((unsigned long long)((const uint64_t*)in)[i]); break;
            default: break;
        }
    }
}

template <class FP8>
void value_to(int dst, const uint8_t* in, void* out, int64_t lo, int64_t hi) {
    for (int64_t i = lo; i < hi; ++i) {
        FP8 v; v.__x = in[i];
        switch (dst) {
            case 0: ((float*)out)[i] = (float)v; break;
            case 1: ((uint16_t*)out)[i] = ((__nv_bfloat16_raw)(__nv_bfloat16)v).x; break;
            case 4: ((double*)out)[i] = (double)v; break;
            case 5: ((uint16_t*)out)[i] = ((__half_raw)(__half)v).x; break;
            case 7: ((int8_t*)out)[i] = (signed char)v; break;
            case 8: ((int16_t*)out)[i] = (short)v; break;
            case 9: ((int32_t*)out)[i] = (int)v; break;
            case 10: ((int64_t*)out)[i] = (long long)v; break;
            case 11: ((uint8_t*)out)[i] = (unsigned char)v; break;
            case 12: ((uint16_t*)out)[i] = (unsigned short)v; break;
            case 13: ((uint32_t*)out)[i] = (unsigned int)v; break;
            case 14: ((uint64_t*)out)[i] = (unsigned long long)v; break;
            case 15: ((uint8_t*)out)[i] = (bool)v ? 1 : 0; break;
            default: break;
        }
    }
}
}  // namespace

extern "C" {
// fp8 value type (format 2, 3 or 6) constructed from `src` items / converted to `dst` items
void ref_bulk_value_from(int src, int fp8, const void* in, uint8_t* out, int64_t n, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        if (fp8 == 2) value_from<__nv_fp8_e4m3>(src, in, out, lo, hi);
        else if (fp8 == 3) value_from<__nv_fp8_e5m2>(src, in, out, lo, hi);
        else value_from<__nv_fp8_e8m0>(src, in, out, lo, hi); });
}
void ref_bulk_value_to(int fp8, int dst, const uint8_t* in, void* out, int64_t n, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        if (fp8 == 2) value_to<__nv_fp8_e4m3>(dst, in, out, lo, hi);
        else if (fp8 == 3) value_to<__nv_fp8_e5m2>(dst, in, out, lo, hi);
        else value_to<__nv_fp8_e8m0>(dst, in, out, lo, hi); });
}
// __nv_cvt_halfraw_to_fp8 (cuda_fp8.hpp:363-388)
void ref_bulk_f16_to_fp8(const uint16_t* in, uint8_t* out, int64_t n, int sat, int interp, int threads) {
    parallel_for(n, threads, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) {
            __half_raw r; r.x = in[i];
            out[i] = (uint8_t)__nv_cvt_halfraw_to_fp8(r, sat ? __NV_SATFINITE : __NV_NOSAT,
                                                      interp ? __NV_E5M2 : __NV_E4M3); } });
}
// __short2bfloat16_rn ... __ull2bfloat16_rn (cuda_bf16.hpp:921, :731, :1448, :1175, :1052, :1307):
// the round-to-nearest forms are the ones with a host path
void ref_bulk_int_to_bf16_rn(int src, const void* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        __nv_bfloat16 v;
        switch (src) {
            case 8: v = __short2bfloat16_rn(((const int16_t*)in)[i]); break;
            case 9: v = __int2bfloat16_rn(((const int32_t*)in)[i]); break;
            case 10: v = __ll2bfloat16_rn(((const int64_t*)in)[i]); break;
            case 12: v = __ushort2bfloat16_rn(((const uint16_t*)in)[i]); break;
            case 13: v = __uint2bfloat16_rn(((const uint32_t*)in)[i]); break;
            default: v = __ull2bfloat16_rn(((const uint64_t*)in)[i]); break;
        }
        out[i] = ((__nv_bfloat16_raw)v).x;
    }
}
// __bfloat162short_rz ... __bfloat162ull_rz, __bfloat162char_rz, __bfloat162uchar_rz
// (cuda_bf16.hpp:867, :680, :1381, :1121, :1002, :1241, :740, :774): the toward-zero
// forms are the ones with a host path
void ref_bulk_bf16_to_int_rz(int dst, const uint16_t* in, void* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        __nv_bfloat16_raw r; r.x = in[i];
        const __nv_bfloat16 h = (__nv_bfloat16)r;
        switch (dst) {
            case 7: ((int8_t*)out)[i] = __bfloat162char_rz(h); break;
            case 8: ((int16_t*)out)[i] = __bfloat162short_rz(h); break;
            case 9: ((int32_t*)out)[i] = __bfloat162int_rz(h); break;
            case 10: ((int64_t*)out)[i] = __bfloat162ll_rz(h); break;
            case 11: ((uint8_t*)out)[i] = __bfloat162uchar_rz(h); break;
            case 12: ((uint16_t*)out)[i] = __bfloat162ushort_rz(h); break;
            case 13: ((uint32_t*)out)[i] = __bfloat162uint_rz(h); break;
            default: ((uint64_t*)out)[i] = __bfloat162ull_rz(h); break;
        }
    }
}
}  // extern "C"
