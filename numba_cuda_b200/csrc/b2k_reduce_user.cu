// cuda.reduce with an arbitrary user expression: the reduce kernel is specialised
// at run time.  The reference compiles the user's Python function into its kernel
// with its JIT (numba/cuda/kernels/reduction.py:15-166); here the Python layer
// traces the function into a C++ expression over `a` and `b`, and this file
// compiles the kernel below around it with NVRTC for sm_100a (libnvrtc is loaded
// on first use; without it the call fails -- nothing falls back to the CPU).
//
// An arbitrary op has no known identity element, so the kernel carries a
// "has a value" flag next to every partial instead of seeding accumulators.
// Every block owns one contiguous span of 16-byte vectors (at least one), so all
// block partials are valid; the last block (ticket) folds them in index order and
// folds `init` in, like the table-op kernel.
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "b2k_internal.cuh"

namespace {

const char *kKernelSource = R"b2ksrc(
typedef B2K_T T;
typedef B2K_W W;
#define B2K_INF (__longlong_as_double(0x7ff0000000000000LL))
#define B2K_NAN (__longlong_as_double(0x7ff8000000000000LL))

// Integer operands are 64 bits wide in the expression, as numba types them, but the
// values of 8-, 16- and 32-bit items rarely leave the 32-bit range: division and
// remainder test for that at run time and then take the 32-bit instruction
// sequence, which is several times shorter than the 64-bit one.
__device__ __forceinline__ long long fdiv_(long long a, long long b) {
    if (b == 0) return 0;
    if (a == (long long)(int)a && b == (long long)(int)b && b != -1) {
        const int x = (int)a, y = (int)b;
        int q = x / y;
        if ((x % y != 0) && ((x < 0) != (y < 0))) --q;
        return q;
    }
    long long q = a / b;
    if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
    return q;
}
__device__ __forceinline__ unsigned long long fdiv_(unsigned long long a, unsigned long long b) {
    if (b == 0) return 0;
    if (((a | b) >> 32) == 0) return (unsigned int)a / (unsigned int)b;
    return a / b;
}
__device__ __forceinline__ double fdiv_(double a, double b) { return floor(a / b); }
__device__ __forceinline__ float fdiv_(float a, float b) { return floorf(a / b); }
__device__ __forceinline__ long long mod_(long long a, long long b) {
    if (b == 0) return 0;
    if (a == (long long)(int)a && b == (long long)(int)b && b != -1) {
        const int y = (int)b;
        int r = (int)a % y;
        if (r != 0 && ((r < 0) != (y < 0))) r += y;
        return r;
    }
    long long r = a % b;
    if (r != 0 && ((r < 0) != (b < 0))) r += b;
    return r;
}
__device__ __forceinline__ unsigned long long mod_(unsigned long long a, unsigned long long b) {
    if (b == 0) return 0;
    if (((a | b) >> 32) == 0) return (unsigned int)a % (unsigned int)b;
    return a % b;
}
__device__ __forceinline__ double mod_(double a, double b) {
    double r = fmod(a, b);
    if (r != 0.0 && ((r < 0.0) != (b < 0.0))) r += b;
    return r;
}
__device__ __forceinline__ float mod_(float a, float b) {
    float r = fmodf(a, b);
    if (r != 0.0f && ((r < 0.0f) != (b < 0.0f))) r += b;
    return r;
}
__device__ __forceinline__ double tdiv_(double a, double b) { return a / b; }
__device__ __forceinline__ float tdiv_(float a, float b) { return a / b; }
__device__ __forceinline__ double tdiv_(long long a, long long b) { return (double)a / (double)b; }
__device__ __forceinline__ double tdiv_(unsigned long long a, unsigned long long b) { return (double)a / (double)b; }
// operands of different types meet in their common arithmetic type first
template <class A, class B> __device__ __forceinline__ auto b2k_floordiv(A a, B b) { typedef decltype(a + b) C; return fdiv_((C)a, (C)b); }
template <class A, class B> __device__ __forceinline__ auto b2k_mod(A a, B b) { typedef decltype(a + b) C; return mod_((C)a, (C)b); }
template <class A, class B> __device__ __forceinline__ auto b2k_truediv(A a, B b) { typedef decltype(a + b) C; return tdiv_((C)a, (C)b); }
__device__ __forceinline__ long long b2k_abs(long long a) { return a < 0 ? -a : a; }
__device__ __forceinline__ unsigned long long b2k_abs(unsigned long long a) { return a; }
__device__ __forceinline__ double b2k_abs(double a) { return fabs(a); }
__device__ __forceinline__ float b2k_abs(float a) { return fabsf(a); }

// an unsigned 64-bit value against a signed one, compared as the numbers they are
typedef unsigned long long b2k_u64;
__device__ __forceinline__ bool b2k_lt(b2k_u64 a, long long b) { return b > 0 && a < (b2k_u64)b; }
__device__ __forceinline__ bool b2k_lt(long long a, b2k_u64 b) { return a < 0 || (b2k_u64)a < b; }
__device__ __forceinline__ bool b2k_le(b2k_u64 a, long long b) { return b >= 0 && a <= (b2k_u64)b; }
__device__ __forceinline__ bool b2k_le(long long a, b2k_u64 b) { return a < 0 || (b2k_u64)a <= b; }
__device__ __forceinline__ bool b2k_eq(b2k_u64 a, long long b) { return b >= 0 && a == (b2k_u64)b; }
__device__ __forceinline__ bool b2k_eq(long long a, b2k_u64 b) { return a >= 0 && (b2k_u64)a == b; }

__device__ __forceinline__ T user_op(T a_, T b_) {
    const W a = (W)a_;
    const W b = (W)b_;
    return (T)(B2K_EXPR);
}

#define THREADS 512
// One load per lane and step: 256 bits where the run-time compiler knows the instruction
// (B2K_WIDE, PTX 8.8), else 128 bits.  Read once: no L1 allocation.  (32 bytes per lane as
// two 128-bit loads would touch every sector twice.)
#if B2K_WIDE
#define VECBYTES 32
struct alignas(32) Vec { unsigned int w[8]; };
__device__ __forceinline__ Vec load_vec(const Vec *p) {
    Vec v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]),
                   "=r"(v.w[7])
                 : "l"(p));
    return v;
}
#else
#define VECBYTES 16
struct alignas(16) Vec { unsigned int w[4]; };
__device__ __forceinline__ Vec load_vec(const Vec *p) {
    Vec v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
                 : "l"(p));
    return v;
}
#endif
#define VEC (VECBYTES / (int)sizeof(T))
// the vector folded on its own, left to right
__device__ __forceinline__ T fold_vec(const Vec &raw) {
    union { Vec q; T e[VEC]; } u;
    u.q = raw;
    T t = u.e[0];
#pragma unroll
    for (int k = 1; k < VEC; ++k) t = user_op(t, u.e[k]);
    return t;
}

struct Partial { T v; bool has; };

__device__ __forceinline__ void fold(Partial &p, T x) {
    p.v = p.has ? user_op(p.v, x) : x;
    p.has = true;
}
__device__ __forceinline__ void join(Partial &p, const Partial &q) {
    if (q.has) fold(p, q.v);
}
__device__ __forceinline__ Partial shuffle_xor(const Partial &p, int mask) {
    unsigned long long bits = 0;
    memcpy(&bits, &p.v, sizeof(T));
    bits = __shfl_xor_sync(0xffffffffu, bits, mask);
    Partial q;
    memcpy(&q.v, &bits, sizeof(T));
    q.has = __shfl_xor_sync(0xffffffffu, (int)p.has, mask) != 0;
    return q;
}
// the lane with the lower index keeps the left operand, so the fold stays in index order
__device__ __forceinline__ Partial block_fold(Partial p, Partial *slots) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int m = 1; m < 32; m <<= 1) {
        const Partial q = shuffle_xor(p, m);
        if ((lane & m) == 0) join(p, q);
        else { Partial r = q; join(r, p); p = r; }
    }
    if (lane == 0) slots[warp] = p;
    __syncthreads();
    if (warp == 0) {
        p = (lane < THREADS / 32) ? slots[lane] : Partial{T(), false};
        for (int m = 1; m < 32; m <<= 1) {
            const Partial q = shuffle_xor(p, m);
            if ((lane & m) == 0) join(p, q);
            else { Partial r = q; join(r, p); p = r; }
        }
    }
    __syncthreads();
    return p;
}

extern "C" __global__ void __launch_bounds__(THREADS)
b2k_user_reduce(const T *__restrict__ x, long long n, T init, T *__restrict__ out, T *partials,
                unsigned int *ticket, long long per /* vectors per block; no block is empty */,
                int fold_init) {
    __shared__ Partial slots[THREADS / 32];
    __shared__ bool is_last;

    const unsigned long long addr = (unsigned long long)x;
    long long head = (long long)(((VECBYTES - (addr & (VECBYTES - 1u))) & (VECBYTES - 1u)) / sizeof(T));
    if (head > n) head = n;
    const Vec *xv = (const Vec *)(x + head);
    const long long nvec = (n - head) / VEC;
    const long long tail_begin = head + nvec * VEC;
    // contiguous span of vectors for this block
    const long long vlo = (long long)blockIdx.x * per;
    long long vhi = vlo + per;
    if (vhi > nvec) vhi = nvec;

    Partial acc{T(), false};
    if (blockIdx.x == 0 && threadIdx.x < head) fold(acc, x[threadIdx.x]);
    // A batch of loads is issued before any of its vectors is used, and the vectors fold as
    // independent chains: a user function of tens of instructions per element otherwise
    // leaves each warp with one load in flight, and the SM's warps cannot cover DRAM
    // latency between them.
    long long v = vlo + threadIdx.x;
    for (; v + (B2K_BATCH - 1) * THREADS < vhi; v += B2K_BATCH * THREADS) {
        Vec r[B2K_BATCH];
        T t[B2K_BATCH];
#pragma unroll
        for (int k = 0; k < B2K_BATCH; ++k) r[k] = load_vec(xv + v + k * THREADS);
#pragma unroll
        for (int k = 0; k < B2K_BATCH; ++k) t[k] = fold_vec(r[k]);
#pragma unroll
        for (int k = 0; k < B2K_BATCH; ++k) fold(acc, t[k]);
    }
    for (; v < vhi; v += THREADS) fold(acc, fold_vec(load_vec(xv + v)));
    if (blockIdx.x == gridDim.x - 1) {
        const long long t = tail_begin + threadIdx.x;
        if (t < n) fold(acc, x[t]);
    }
    Partial total = block_fold(acc, slots);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = total.v;   // every block owns at least one element
        __threadfence();
        const unsigned int t = atomicInc(ticket, gridDim.x - 1);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    Partial mine{T(), false};
    // contiguous slices per thread keep the fold in block order
    const unsigned int g = gridDim.x;
    const unsigned int each = (g + THREADS - 1) / THREADS;
    for (unsigned int i = threadIdx.x * each; i < g && i < (threadIdx.x + 1) * each; ++i)
        fold(mine, __ldcg(partials + i));
    total = block_fold(mine, slots);
    if (threadIdx.x == 0) out[0] = fold_init ? user_op(total.v, init) : total.v;
}
)b2ksrc";

// ---- NVRTC, loaded on first use ---------------------------------------------------
struct Nvrtc {
    void *lib = nullptr;
    decltype(&nvrtcCreateProgram) create = nullptr;
    decltype(&nvrtcCompileProgram) compile = nullptr;
    decltype(&nvrtcGetCUBINSize) cubin_size = nullptr;
    decltype(&nvrtcGetCUBIN) cubin = nullptr;
    decltype(&nvrtcGetProgramLogSize) log_size = nullptr;
    decltype(&nvrtcGetProgramLog) log = nullptr;
    decltype(&nvrtcDestroyProgram) destroy = nullptr;
    int version = -1;   // major * 100 + minor
    bool ok = false;
};

Nvrtc &nvrtc() {
    static Nvrtc n;
    static std::once_flag once;
    std::call_once(once, [] {
        // A process can see more than one NVRTC (the toolkit's, and the one a Python
        // package bundles, which the loader hands out under the bare name once that package
        // has loaded it).  The newest one wins: 256-bit loads need its PTX version.
        const char *forced = getenv("B2K_NVRTC_PATH");
        const char *names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                               "/usr/local/cuda/lib64/libnvrtc.so"};
        int best = -1;
        auto consider = [&](const char *name) {
            if (!name || !*name) return;
            void *lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (!lib) return;
            int major = 0, minor = 0;
            auto version = reinterpret_cast<nvrtcResult (*)(int *, int *)>(dlsym(lib, "nvrtcVersion"));
            if (version && version(&major, &minor) == NVRTC_SUCCESS && major * 100 + minor > best) {
                best = major * 100 + minor;
                n.lib = lib;
            }
        };
        if (forced && *forced) consider(forced);
        else for (const char *name : names) consider(name);
        n.version = best;
        if (!n.lib) return;
#define B2K_SYM(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.lib, sym))
        B2K_SYM(create, "nvrtcCreateProgram");
        B2K_SYM(compile, "nvrtcCompileProgram");
        B2K_SYM(cubin_size, "nvrtcGetCUBINSize");
        B2K_SYM(cubin, "nvrtcGetCUBIN");
        B2K_SYM(log_size, "nvrtcGetProgramLogSize");
        B2K_SYM(log, "nvrtcGetProgramLog");
        B2K_SYM(destroy, "nvrtcDestroyProgram");
#undef B2K_SYM
        n.ok = n.create && n.compile && n.cubin_size && n.cubin && n.log_size && n.log && n.destroy;
    });
    return n;
}

struct Driver {
    CUresult (*module_load)(CUmodule *, const void *) = nullptr;
    CUresult (*get_function)(CUfunction *, CUmodule, const char *) = nullptr;
    CUresult (*launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                       void **, void **) = nullptr;
    CUresult (*occupancy)(int *, CUfunction, int, size_t) = nullptr;
    bool ok = false;
};

Driver &driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        auto get = [](const char *name) -> void * {
            void *p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
                return nullptr;
            return p;
        };
        d.module_load = reinterpret_cast<decltype(d.module_load)>(get("cuModuleLoadData"));
        d.get_function = reinterpret_cast<decltype(d.get_function)>(get("cuModuleGetFunction"));
        d.launch = reinterpret_cast<decltype(d.launch)>(get("cuLaunchKernel"));
        d.occupancy = reinterpret_cast<decltype(d.occupancy)>(get("cuOccupancyMaxActiveBlocksPerMultiprocessor"));
        d.ok = d.module_load && d.get_function && d.launch && d.occupancy;
    });
    return d;
}

struct TypeInfo { const char *t; const char *w; const char *ilit; size_t size; };

bool type_info(int dtype, TypeInfo *out) {
    switch (dtype) {
    case B2K_I8: *out = {"signed char", "long long", "((long long)(x))", 1}; return true;
    case B2K_I16: *out = {"short", "long long", "((long long)(x))", 2}; return true;
    case B2K_I32: *out = {"int", "long long", "((long long)(x))", 4}; return true;
    case B2K_I64: *out = {"long long", "long long", "((long long)(x))", 8}; return true;
    case B2K_U8: *out = {"unsigned char", "unsigned long long", "((long long)(x))", 1}; return true;
    case B2K_U16: *out = {"unsigned short", "unsigned long long", "((long long)(x))", 2}; return true;
    case B2K_U32: *out = {"unsigned int", "unsigned long long", "((long long)(x))", 4}; return true;
    case B2K_U64: *out = {"unsigned long long", "unsigned long long", "((long long)(x))", 8}; return true;
    case B2K_F32: *out = {"float", "float", "((double)(x))", 4}; return true;
    case B2K_F64: *out = {"double", "double", "((double)(x))", 8}; return true;
    default: return false;
    }
}

std::mutex g_cache_mutex;
struct Compiled {
    CUfunction fn = nullptr;
    int blocks_per_sm = 1;   // resident CTAs of 512 threads, from the kernel's register count
    int vec_bytes = 16;      // bytes per lane and load the kernel was compiled for
};
std::map<std::string, Compiled> g_cache;  // key: device / dtype / expression

int compile_kernel(const std::string &expr, int dtype, const TypeInfo &ti, Compiled *out) {
    CUfunction *fn = &out->fn;
    Nvrtc &rt = nvrtc();
    if (!rt.ok) return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_expr: libnvrtc could not be loaded");
    Driver &drv = driver();
    if (!drv.ok) return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_expr: driver entry points unavailable");
    cudaFree(nullptr);  // make sure the primary context exists before loading a module
    const std::string dt = std::string("-DB2K_T=") + ti.t;
    const std::string dw = std::string("-DB2K_W=") + ti.w;
    const std::string dl = std::string("-DB2K_ILIT(x)=") + ti.ilit;
    const std::string de = "-DB2K_EXPR=" + expr;
    // 256-bit loads where the run-time compiler knows them (CUDA 12.9 on), 128-bit ones
    // otherwise; 64 bytes in flight per thread either way.  A compiler that refuses the
    // wide form once is not asked again.
    // Functions that divide are bound by instruction issue, not by the loads, and measured
    // 2-4 % faster with four narrow loads (more CTAs resident); the rest gain 4-5 % from
    // the wide ones.
    static std::atomic<int> wide_refused{0};
    const bool divides = expr.find("b2k_mod(") != std::string::npos || expr.find("b2k_floordiv(") != std::string::npos ||
                         expr.find("b2k_truediv(") != std::string::npos;
    const int wide_default = divides ? 0 : 1;
    int wide = (rt.version >= 1209 && !wide_refused.load() &&
                B2K_ENV_INT("B2K_USER_REDUCE_WIDE", wide_default) != 0) ? 1 : 0;
    nvrtcProgram prog;
    for (;;) {
        if (rt.create(&prog, kKernelSource, "b2k_user_reduce.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
            return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_expr: nvrtcCreateProgram failed");
        const std::string dv = std::string("-DB2K_WIDE=") + (wide ? "1" : "0");
        const std::string db = "-DB2K_BATCH=" + std::to_string(B2K_ENV_INT("B2K_USER_REDUCE_BATCH", wide ? 2 : 4));
        const char *opts[] = {"--gpu-architecture=sm_100a", "-std=c++17", "-default-device", dt.c_str(), dw.c_str(),
                              dl.c_str(), de.c_str(), db.c_str(), dv.c_str()};
        if (rt.compile(prog, 9, opts) == NVRTC_SUCCESS) break;
        size_t len = 0;
        rt.log_size(prog, &len);
        std::string log(len, '\0');
        if (len) rt.log(prog, &log[0]);
        rt.destroy(&prog);
        if (wide && log.find("vector") != std::string::npos) {   // "Illegal vector size: 8"
            wide_refused.store(1);
            wide = 0;
            continue;
        }
        if (log.size() > 380) log.resize(380);
        return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_expr: the expression does not compile: %s", log.c_str());
    }
    out->vec_bytes = wide ? 32 : 16;
    size_t size = 0;
    rt.cubin_size(prog, &size);
    std::vector<char> image(size);
    rt.cubin(prog, image.data());
    rt.destroy(&prog);
    CUmodule mod;
    if (drv.module_load(&mod, image.data()) != CUDA_SUCCESS)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_expr: cuModuleLoadData failed");
    if (drv.get_function(fn, mod, "b2k_user_reduce") != CUDA_SUCCESS)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "b2k_reduce_expr: kernel not found in the compiled module");
    // the grid is one wave of resident CTAs: the user's expression decides the register
    // count, and with it how many CTAs of 512 threads an SM holds
    int resident = 0;
    if (drv.occupancy(&resident, *fn, 512, 0) != CUDA_SUCCESS || resident < 1) resident = 1;
    out->blocks_per_sm = resident > 4 ? 4 : resident;
    (void)dtype;
    return B2K_OK;
}

}  // namespace

extern "C" int b2k_reduce_expr(const char *expr, int dtype, const void *x_dev, int64_t n, const void *init_host,
                               void *out_dev, void *scratch_dev, int64_t scratch_bytes, void *stream) {
    B2K_RANGE("b2k_reduce_expr");
    TypeInfo ti;
    if (!type_info(dtype, &ti)) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_expr: unknown dtype %d", dtype);
    if (!expr || !*expr) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_expr: empty expression");
    if (n < 1) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_expr: needs at least one element");
    if (!x_dev || !out_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_reduce_expr: null pointer");
    if (!scratch_dev || scratch_bytes < b2k_reduce_scratch_bytes() || !b2k::aligned_to<void>(scratch_dev, 256))
        return b2k::fail(B2K_ERR_SCRATCH, "b2k_reduce_expr: scratch of %lld bytes (256-byte aligned) required",
                         (long long)b2k_reduce_scratch_bytes());
    if (!b2k::aligned_to<void>(x_dev, ti.size) || !b2k::aligned_to<void>(out_dev, ti.size))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_reduce_expr: pointers must be aligned to the element size");

    int device = 0;
    cudaGetDevice(&device);
    const std::string key = std::to_string(device) + "/" + std::to_string(dtype) + "/" + expr;
    Compiled kernel;
    {
        std::lock_guard<std::mutex> lock(g_cache_mutex);
        auto it = g_cache.find(key);
        if (it == g_cache.end()) {
            const int rc = compile_kernel(expr, dtype, ti, &kernel);
            if (rc != B2K_OK) return rc;
            g_cache.emplace(key, kernel);
        } else {
            kernel = it->second;
        }
    }
    CUfunction fn = kernel.fn;
    // one contiguous span of vectors per block, at least one vector each
    const int64_t vb = kernel.vec_bytes;
    const int64_t vec = vb / static_cast<int64_t>(ti.size);
    const int64_t nvec = n / vec;
    // the head (elements before the first vector boundary) shortens the vector count by at most one
    const int64_t head = ((vb - (reinterpret_cast<uintptr_t>(x_dev) & (vb - 1))) & (vb - 1)) / static_cast<int64_t>(ti.size);
    const int64_t nvec_dev = (n - (head < n ? head : n)) / vec;
    int64_t grid = nvec_dev / (512 * (128 / vb));   // at least 64 KB per block
    const int64_t cap = static_cast<int64_t>(b2k::sm_count()) * kernel.blocks_per_sm;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    long long per = (nvec_dev + grid - 1) / grid;
    if (per > 0) grid = (nvec_dev + per - 1) / per;   // every block gets at least one vector
    if (grid < 1) grid = 1;
    (void)nvec;
    unsigned long long init_bits = 0;
    int fold_init = init_host != nullptr;
    if (fold_init) memcpy(&init_bits, init_host, ti.size);
    long long n_arg = n;
    void *ticket = scratch_dev;
    void *partials = static_cast<char *>(scratch_dev) + 256;
    void *args[] = {const_cast<void **>(&x_dev), &n_arg, &init_bits, &out_dev, &partials, &ticket, &per, &fold_init};
    const CUresult rc = driver().launch(fn, static_cast<unsigned>(grid), 1, 1, 512, 1, 1, 0,
                                        reinterpret_cast<CUstream>(stream), args, nullptr);
    b2k::note_launch();
    if (rc != CUDA_SUCCESS) return b2k::fail(static_cast<int>(cudaErrorLaunchFailure), "b2k_reduce_expr: cuLaunchKernel failed (%d)", (int)rc);
    return B2K_OK;
}
