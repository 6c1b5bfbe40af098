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
