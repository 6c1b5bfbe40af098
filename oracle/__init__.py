"""CPU oracle for the numba-cuda library kernels -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may import this package.  The shipped package
(``numba_cuda_b200``) never does: it fails loudly if its CUDA library is absent.

Two checkers live here:

* ``libb2k_oracle.so`` -- a plain-C restatement (``b2k_oracle.c``) of the
  reference algorithms, each function citing the reference file:line it follows.
* ``_ref/libb2k_ref_headers.so`` -- the *reference's own* host code for the
  fp8/bf16 arithmetic: its vendored ``cuda_fp8.hpp`` / ``cuda_bf16.hpp`` compiled
  with g++ straight from the reference tree (``oracle/Makefile``).  It is built
  only where the reference tree is present and travels as a binary.

The wrappers below expose both through NumPy arrays.
"""
from __future__ import annotations

import ctypes
import functools
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

#: the RNG state record of numba_cuda/numba/cuda/random.py:47-49
xoroshiro128p_dtype = np.dtype([("s0", np.uint64), ("s1", np.uint64)], align=True)

F32, BF16, E4M3, E5M2, F64, F16, E8M0 = 0, 1, 2, 3, 4, 5, 6
I8, I16, I32, I64, U8, U16, U32, U64, BOOL = 7, 8, 9, 10, 11, 12, 13, 14, 15
RN, RZ, RU, RD = 0, 1, 2, 3   # cudaRoundMode order: nearest, zero, +inf, -inf
OPS = {"add": 0, "mul": 1, "max": 2, "min": 3}


def _older(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force: bool = False, reference_root: str | None = None) -> None:
    """Compile the C restatement and, when the location of a reference source
    tree is given (argument or ``B2K_REFERENCE_ROOT``), the reference-header
    checker.  Without a location a prebuilt ``_ref/`` is kept as it is.
    Building the checker is not using it."""
    target = os.path.join(_HERE, "libb2k_oracle.so")
    src = os.path.join(_HERE, "b2k_oracle.c")
    if force or _older(target, src, os.path.join(_HERE, "Makefile")):
        subprocess.run(["make", "-B", "-C", _HERE, "libb2k_oracle.so", "CC=gcc"], check=True,
                       capture_output=True)
    ref_root = reference_root or os.environ.get("B2K_REFERENCE_ROOT")
    ref_so = os.path.join(_HERE, "_ref", "libb2k_ref_headers.so")
    if ref_root and os.path.isdir(ref_root) and (
            force or _older(ref_so, os.path.join(_HERE, "ref_headers_shim.cpp"))):
        subprocess.run(["make", "-C", _HERE, "ref", "CXX=g++", f"REFERENCE_ROOT={ref_root}"],
                       check=True, capture_output=True)


@functools.lru_cache(maxsize=None)
def lib() -> ctypes.CDLL:
    build()
    L = ctypes.CDLL(os.path.join(_HERE, "libb2k_oracle.so"))
    vp, i64, u64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_int
    L.oracle_xoro_seed.argtypes = [vp, u64]
    L.oracle_xoro_next.argtypes = [vp]
    L.oracle_xoro_next.restype = u64
    L.oracle_xoro_jump.argtypes = [vp]
    L.oracle_xoro_init_states.argtypes = [vp, i64, u64, u64]
    L.oracle_xoro_fill.argtypes = [vp, i64, i32, vp, i64]
    L.oracle_f64_to_fp8.argtypes = [ctypes.c_double, i32, i32]
    L.oracle_f64_to_fp8.restype = ctypes.c_uint8
    L.oracle_f32_to_fp8.argtypes = [ctypes.c_float, i32, i32]
    L.oracle_f32_to_fp8.restype = ctypes.c_uint8
    L.oracle_fp8_to_f16bits.argtypes = [ctypes.c_uint8, i32]
    L.oracle_fp8_to_f16bits.restype = ctypes.c_uint16
    L.oracle_fp8_to_f32.argtypes = [ctypes.c_uint8, i32]
    L.oracle_fp8_to_f32.restype = ctypes.c_float
    L.oracle_f32_to_bf16.argtypes = [ctypes.c_float]
    L.oracle_f32_to_bf16.restype = ctypes.c_uint16
    L.oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
    L.oracle_bf16_to_f32.restype = ctypes.c_float
    L.oracle_cast.argtypes = [i32, i32, i32, vp, vp, i64]
    L.oracle_cast.restype = i32
    L.oracle_f32_to_bf16_mode.argtypes = [ctypes.c_float, i32]
    L.oracle_f32_to_bf16_mode.restype = ctypes.c_uint16
    L.oracle_f64_to_bf16.argtypes = [ctypes.c_double]
    L.oracle_f64_to_bf16.restype = ctypes.c_uint16
    L.oracle_bf16_to_e8m0.argtypes = [ctypes.c_uint16, i32, i32]
    L.oracle_bf16_to_e8m0.restype = ctypes.c_uint8
    L.oracle_f32_to_e8m0.argtypes = [ctypes.c_float, i32, i32]
    L.oracle_f32_to_e8m0.restype = ctypes.c_uint8
    L.oracle_e8m0_to_bf16.argtypes = [ctypes.c_uint8]
    L.oracle_e8m0_to_bf16.restype = ctypes.c_uint16
    L.oracle_bf16_to_fp8.argtypes = [ctypes.c_uint16, i32, i32]
    L.oracle_bf16_to_fp8.restype = ctypes.c_uint8
    L.oracle_f64_to_e8m0.argtypes = [ctypes.c_double, i32, i32]
    L.oracle_f64_to_e8m0.restype = ctypes.c_uint8
    L.oracle_cast_ex.argtypes = [i32, i32, i32, i32, vp, vp, i64]
    L.oracle_cast_ex.restype = i32
    L.oracle_fold_f64.argtypes = [vp, i64, ctypes.c_double, i32]
    L.oracle_fold_f64.restype = ctypes.c_double
    L.oracle_fold_f32.argtypes = [vp, i64, ctypes.c_float, i32]
    L.oracle_fold_f32.restype = ctypes.c_float
    L.oracle_transpose2d.argtypes = [vp, vp, i64, i64, i64, i64, i64]
    return L


def have_ref_headers() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libb2k_ref_headers.so"))


@functools.lru_cache(maxsize=None)
def ref_headers() -> ctypes.CDLL:
    """The reference's vendored fp8/bf16 headers, host path (g++-compiled)."""
    L = ctypes.CDLL(os.path.join(_HERE, "_ref", "libb2k_ref_headers.so"))
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    L.ref_cvt_float_to_fp8.argtypes = [ctypes.c_float, i32, i32]
    L.ref_cvt_float_to_fp8.restype = ctypes.c_uint8
    L.ref_cvt_double_to_fp8.argtypes = [ctypes.c_double, i32, i32]
    L.ref_cvt_double_to_fp8.restype = ctypes.c_uint8
    L.ref_cvt_fp8_to_halfraw.argtypes = [ctypes.c_uint8, i32]
    L.ref_cvt_fp8_to_halfraw.restype = ctypes.c_uint16
    L.ref_fp8_to_float.argtypes = [ctypes.c_uint8, i32]
    L.ref_fp8_to_float.restype = ctypes.c_float
    L.ref_fp8_from_float.argtypes = [ctypes.c_float, i32]
    L.ref_fp8_from_float.restype = ctypes.c_uint8
    L.ref_float2bfloat16_rn.argtypes = [ctypes.c_float]
    L.ref_float2bfloat16_rn.restype = ctypes.c_uint16
    L.ref_bfloat162float.argtypes = [ctypes.c_uint16]
    L.ref_bfloat162float.restype = ctypes.c_float
    L.ref_float2bfloat16_mode.argtypes = [ctypes.c_float, i32]
    L.ref_float2bfloat16_mode.restype = ctypes.c_uint16
    L.ref_double2bfloat16.argtypes = [ctypes.c_double]
    L.ref_double2bfloat16.restype = ctypes.c_uint16
    L.ref_cvt_float_to_e8m0.argtypes = [ctypes.c_float, i32, i32]
    L.ref_cvt_float_to_e8m0.restype = ctypes.c_uint8
    L.ref_cvt_bfloat16raw_to_e8m0.argtypes = [ctypes.c_uint16, i32, i32]
    L.ref_cvt_bfloat16raw_to_e8m0.restype = ctypes.c_uint8
    L.ref_cvt_e8m0_to_bf16raw.argtypes = [ctypes.c_uint8]
    L.ref_cvt_e8m0_to_bf16raw.restype = ctypes.c_uint16
    L.ref_cvt_bfloat16raw_to_fp8.argtypes = [ctypes.c_uint16, i32, i32]
    L.ref_cvt_bfloat16raw_to_fp8.restype = ctypes.c_uint8
    L.ref_cvt_double_to_e8m0.argtypes = [ctypes.c_double, i32, i32]
    L.ref_cvt_double_to_e8m0.restype = ctypes.c_uint8
    for name, scalar in (("ref_cvt_double2_to_fp8x2", ctypes.c_double), ("ref_cvt_float2_to_fp8x2", ctypes.c_float),
                         ("ref_cvt_bfloat16raw2_to_fp8x2", ctypes.c_uint16),
                         ("ref_cvt_float2_to_e8m0x2", ctypes.c_float), ("ref_cvt_double2_to_e8m0x2", ctypes.c_double),
                         ("ref_cvt_bfloat162raw_to_e8m0x2", ctypes.c_uint16)):
        fn = getattr(L, name)
        fn.argtypes = [scalar, scalar, i32, i32]
        fn.restype = ctypes.c_uint16
    L.ref_bulk_f64_to_fp8.argtypes = [vp, vp, i64, i32, i32, i32]
    L.ref_bulk_bf16_to_fp8.argtypes = [vp, vp, i64, i32, i32, i32]
    L.ref_bulk_f64_to_e8m0.argtypes = [vp, vp, i64, i32, i32, i32]
    L.ref_bulk_f32_to_fp8.argtypes = [vp, vp, i64, i32, i32, i32]
    L.ref_bulk_fp8_to_f32.argtypes = [vp, vp, i64, i32, i32]
    L.ref_bulk_f32_to_bf16.argtypes = [vp, vp, i64, i32]
    L.ref_bulk_bf16_to_f32.argtypes = [vp, vp, i64, i32]
    L.ref_bulk_value_from.argtypes = [i32, i32, vp, vp, i64, i32]
    L.ref_bulk_value_to.argtypes = [i32, i32, vp, vp, i64, i32]
    L.ref_bulk_f16_to_fp8.argtypes = [vp, vp, i64, i32, i32, i32]
    L.ref_bulk_int_to_bf16_rn.argtypes = [i32, vp, vp, i64]
    L.ref_bulk_bf16_to_int_rz.argtypes = [i32, vp, vp, i64]
    return L


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


# ---------------------------------------------------------------- RNG
def init_states(n: int, seed: int, subsequence_start: int = 0) -> np.ndarray:
    """Serial state creation, as random.py:242-257."""
    st = np.empty(n, dtype=xoroshiro128p_dtype)
    lib().oracle_xoro_init_states(_ptr(st), n, seed & (2**64 - 1), subsequence_start)
    return st


_KIND = {("uniform", np.dtype(np.float32)): 0, ("uniform", np.dtype(np.float64)): 1,
         ("normal", np.dtype(np.float32)): 2, ("normal", np.dtype(np.float64)): 3}


def fill(states: np.ndarray, dist: str, dtype, count: int, threads: int = 1) -> np.ndarray:
    """out[t, i] = i-th draw of generator t; advances ``states`` in place.
    Generators are independent, so ``threads`` > 1 (0 = all cores) splits them
    into contiguous slices that run side by side (the C call releases the GIL)."""
    dtype = np.dtype(dtype)
    n = states.shape[0]
    out = np.zeros((n, count), dtype=dtype)   # zeros: pages are touched before the timed loops
    assert states.flags.c_contiguous and states.dtype.itemsize == 16
    kind = _KIND[(dist, dtype)]
    if threads == 0:
        threads = os.cpu_count() or 1
    threads = max(1, min(threads, n // 4096 or 1))
    if threads == 1:
        lib().oracle_xoro_fill(_ptr(states), n, kind, _ptr(out), count)
        return out
    import concurrent.futures
    L = lib()
    bounds = np.linspace(0, n, threads + 1).astype(np.int64)

    def piece(k):
        lo, hi = int(bounds[k]), int(bounds[k + 1])
        L.oracle_xoro_fill(_ptr(states) + 16 * lo, hi - lo, kind, _ptr(out) + lo * count * dtype.itemsize, count)

    with concurrent.futures.ThreadPoolExecutor(threads) as pool:
        list(pool.map(piece, range(threads)))
    return out


def jump(state_pair):
    st = np.array([tuple(state_pair)], dtype=xoroshiro128p_dtype)
    lib().oracle_xoro_jump(_ptr(st))
    return int(st[0]["s0"]), int(st[0]["s1"])


def next_u64(state_pair):
    st = np.array([tuple(state_pair)], dtype=xoroshiro128p_dtype)
    r = lib().oracle_xoro_next(_ptr(st))
    return int(r), (int(st[0]["s0"]), int(st[0]["s1"]))


# ---------------------------------------------------------------- casts
_CODE_DTYPE = {F32: np.float32, BF16: np.uint16, E4M3: np.uint8, E5M2: np.uint8, F64: np.float64,
               F16: np.float16, E8M0: np.uint8, I8: np.int8, I16: np.int16, I32: np.int32, I64: np.int64,
               U8: np.uint8, U16: np.uint16, U32: np.uint32, U64: np.uint64, BOOL: np.uint8}
INT_FORMATS = (I8, I16, I32, I64, U8, U16, U32, U64)


def cast(x: np.ndarray, src: int, dst: int, sat: int = 1) -> np.ndarray:
    """Bulk cast with the C restatement.  bf16 travels as uint16 bit patterns,
    fp8 as uint8 codes."""
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    out = np.empty(x.shape, dtype=_CODE_DTYPE[dst])
    rc = lib().oracle_cast(src, dst, sat, _ptr(x), _ptr(out), x.size)
    if rc != 0:
        raise ValueError(f"unsupported cast {src}->{dst}")
    return out


def cast_ex(x: np.ndarray, src: int, dst: int, sat: int = 1, mode: int = RN) -> np.ndarray:
    """Bulk cast for the rounding-mode / f64 / E8M0 / f16 conversions (C restatement;
    f16 uses NumPy's IEEE round-to-nearest-even conversion)."""
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    if (src, dst) == (F32, F16):
        return x.astype(np.float16)
    if (src, dst) == (F16, F32):
        return x.astype(np.float32)
    out = np.empty(x.shape, dtype=_CODE_DTYPE[dst])
    rc = lib().oracle_cast_ex(src, dst, sat, mode, _ptr(x), _ptr(out), x.size)
    if rc != 0:
        raise ValueError(f"unsupported cast {src}->{dst}")
    return out


def ref_cast(x: np.ndarray, src: int, dst: int, sat: int = 1, threads: int = 0, mode: int = RZ) -> np.ndarray:
    """Bulk cast with the reference's own vendored-header host code."""
    R = ref_headers()
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    out = np.empty(x.shape, dtype=_CODE_DTYPE[dst])
    if src == F32 and dst == BF16:
        R.ref_bulk_f32_to_bf16(_ptr(x), _ptr(out), x.size, threads)
    elif src == BF16 and dst == F32:
        R.ref_bulk_bf16_to_f32(_ptr(x), _ptr(out), x.size, threads)
    elif src == F32 and dst in (E4M3, E5M2):
        R.ref_bulk_f32_to_fp8(_ptr(x), _ptr(out), x.size, sat, dst - 2, threads)
    elif src in (E4M3, E5M2) and dst == F32:
        R.ref_bulk_fp8_to_f32(_ptr(x), _ptr(out), x.size, src - 2, threads)
    elif src == F64 and dst in (E4M3, E5M2):
        R.ref_bulk_f64_to_fp8(_ptr(x), _ptr(out), x.size, sat, dst - 2, threads)
    elif src == BF16 and dst in (E4M3, E5M2):
        R.ref_bulk_bf16_to_fp8(_ptr(x), _ptr(out), x.size, sat, dst - 2, threads)
    elif src == F64 and dst == E8M0:
        R.ref_bulk_f64_to_e8m0(_ptr(x), _ptr(out), x.size, sat, mode, threads)
    else:
        raise ValueError(f"unsupported cast {src}->{dst}")
    return out


# ---------------------------------------------------------------- fp8 value types, bf16 <-> integers
def fp8_values(fmt: int) -> np.ndarray:
    """The 256 values of a one-byte format as float64 (NaN where the code is one):
    E4M3 has no infinities and one NaN per sign (0x7F / 0xFF), E5M2 is IEEE-like,
    E8M0 is 2**(code-127) with 0xFF the NaN (cuda_fp8.hpp:473-523, :817-851)."""
    code = np.arange(256)
    if fmt == E8M0:
        v = np.ldexp(1.0, code - 127)
        v[255] = np.nan
        return v
    mbits = 3 if fmt == E4M3 else 2
    bias = 7 if fmt == E4M3 else 15
    sign = np.where(code & 0x80, -1.0, 1.0)
    e = (code & 0x7F) >> mbits
    m = (code & ((1 << mbits) - 1)).astype(np.float64) / (1 << mbits)
    v = np.where(e == 0, np.ldexp(m, 1 - bias), np.ldexp(1.0 + m, e - bias))
    if fmt == E4M3:
        v = np.where((code & 0x7F) == 0x7F, np.nan, v)
    else:
        v = np.where(e == 31, np.where(m == 0, np.inf, np.nan), v)
    return sign * v


def _float_to_int(v: np.ndarray, dst: int, mode: int = RZ) -> np.ndarray:
    """Float64 values to an integer type the way a cvt does it: rounded in the given
    direction, clamped to the ends of the range; a NaN gives 0 in a result of up to
    32 bits and 0x8000000000000000 in one of 64 (cuda_fp8.hpp:1065-1263,
    cuda_bf16.hpp:653-678)."""
    dtype = np.dtype(_CODE_DTYPE[dst])
    info = np.iinfo(dtype)
    rounded = {RN: np.rint, RZ: np.trunc, RU: np.ceil, RD: np.floor}[mode](v)
    nan = np.isnan(v)
    top = rounded >= float(info.max)       # float(max) is max+1 for the 64-bit types: still the right cut
    bottom = rounded <= float(info.min)
    safe = np.where(nan | top | bottom, 0.0, rounded)
    out = safe.astype(dtype)
    out[top] = info.max
    out[bottom] = info.min
    out[nan] = (dtype.type(info.min) if dtype.kind == "i" else dtype.type(1 << 63)) if dtype.itemsize == 8 else 0
    return out


def value_to(codes: np.ndarray, fmt: int, dst: int) -> np.ndarray:
    """Conversion operators of fp8_e4m3 / fp8_e5m2 / fp8_e8m0 (cuda_fp8.hpp:1031-1263,
    :1644-1876, :2260-2494): to f16 / bf16 (raw bits) / f32 / f64, to the integer types
    (toward zero, saturating, NaN as above) and to bool (any non-zero code; always true
    for E8M0)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    table = fp8_values(fmt)
    if dst == BOOL:
        flags = np.ones(256, np.uint8) if fmt == E8M0 else ((np.arange(256) & 0x7F) != 0).astype(np.uint8)
        return flags[codes]
    if dst in INT_FORMATS:
        return _float_to_int(table, dst)[codes]
    if dst == F64:
        return table[codes]
    if dst == F32:
        return table.astype(np.float32)[codes]
    if dst == F16:
        with np.errstate(over="ignore"):
            return table.astype(np.float16)[codes]   # E8M0: to nearest, beyond 2**15 infinity
    if dst == BF16:
        return (table.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)[codes]   # every value fits
    raise ValueError(f"unsupported conversion {fmt}->{dst}")


def value_from(x: np.ndarray, src: int, fmt: int) -> np.ndarray:
    """Constructors of the fp8 value types (cuda_fp8.hpp:918-1023, :1531-1636, :2118-2215).
    E4M3 / E5M2: saturating, to nearest even; an integer is rounded to float32 first.
    E8M0: saturating, up to the next power of two; for an integer that is
    ceil(log2(|v|))."""
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    if fmt in (E4M3, E5M2):
        if src in INT_FORMATS:
            return cast(x.astype(np.float32), F32, fmt, 1)
        if src == F16:
            return cast(x.astype(np.float32), F32, fmt, 1)
        return cast_ex(x, src, fmt, 1, RN) if src in (F64, BF16) else cast(x, src, fmt, 1)
    if src in INT_FORMATS:
        zero = int(cast_ex(np.zeros(1, np.float32), F32, E8M0, 1, RU)[0])
        flat = [int(v) for v in x.reshape(-1)]
        codes = [zero if v == 0 else 127 + (abs(v) - 1).bit_length() for v in flat]
        return np.array(codes, dtype=np.uint8).reshape(x.shape)
    if src == F16:
        return cast_ex(x.astype(np.float32), F32, E8M0, 1, RU)
    return cast_ex(x, src, E8M0, 1, RU)


def int_to_bf16(x: np.ndarray, src: int, mode: int = RN) -> np.ndarray:
    """An integer rounded to bfloat16 (8 significant bits) in one step, in the
    direction asked for: nearest even, toward zero, toward +inf, toward -inf
    (cuda_bf16.hpp:714-738, :807-837 and the 16- and 64-bit siblings)."""
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    out = np.empty(x.size, dtype=np.uint16)
    for i, v in enumerate(int(t) for t in x.reshape(-1)):
        neg, mag = v < 0, abs(v)
        if mag == 0:
            out[i] = 0
            continue
        k = mag.bit_length()
        if k <= 8:
            q = mag << (8 - k)
        else:
            shift = k - 8
            q, rem = mag >> shift, mag & ((1 << shift) - 1)
            half = 1 << (shift - 1)
            up = (rem > half or (rem == half and (q & 1))) if mode == RN else \
                 False if mode == RZ else (rem != 0 and neg == (mode == RD))
            q += int(up)
            if q == 256:
                q, k = 128, k + 1
        out[i] = (int(neg) << 15) | ((126 + k) << 7) | (q & 0x7F)
    return out.reshape(x.shape)


def bf16_to_int(bits: np.ndarray, dst: int, mode: int = RZ) -> np.ndarray:
    """bfloat16 (raw bits) to an integer type: rounded in the direction asked for,
    saturating, NaN to 0 (0x8000000000000000 for 64 bits) (cuda_bf16.hpp:641-712 and
    siblings)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    with np.errstate(invalid="ignore"):     # signalling NaN patterns are converted like the others
        values = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    return _float_to_int(values, dst, mode)


def ref_value_from(x: np.ndarray, src: int, fmt: int, threads: int = 0) -> np.ndarray:
    """Constructors of the value types through the reference's own header (host path)."""
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    out = np.empty(x.shape, dtype=np.uint8)
    ref_headers().ref_bulk_value_from(src, fmt, _ptr(x), _ptr(out), x.size, threads)
    return out


def ref_value_to(codes: np.ndarray, fmt: int, dst: int, threads: int = 0) -> np.ndarray:
    """Conversion operators of the value types through the reference's own header."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    out = np.empty(codes.shape, dtype=_CODE_DTYPE[dst] if dst != F16 else np.uint16)
    ref_headers().ref_bulk_value_to(fmt, dst, _ptr(codes), _ptr(out), codes.size, threads)
    return out.view(np.float16) if dst == F16 else out


def ref_f16_to_fp8(x: np.ndarray, fmt: int, sat: int = 1, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float16)
    out = np.empty(x.shape, dtype=np.uint8)
    ref_headers().ref_bulk_f16_to_fp8(_ptr(x), _ptr(out), x.size, sat, fmt - 2, threads)
    return out


def ref_int_to_bf16_rn(x: np.ndarray, src: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=_CODE_DTYPE[src])
    out = np.empty(x.shape, dtype=np.uint16)
    ref_headers().ref_bulk_int_to_bf16_rn(src, _ptr(x), _ptr(out), x.size)
    return out


def ref_bf16_to_int_rz(bits: np.ndarray, dst: int) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=_CODE_DTYPE[dst])
    ref_headers().ref_bulk_bf16_to_int_rz(dst, _ptr(bits), _ptr(out), bits.size)
    return out


# ---------------------------------------------------------------- reduce / transpose
def fold(x: np.ndarray, op: str, init=0):
    """Sequential left fold from ``init`` -- the reference's CPU path for
    cuda.reduce (simulator/reduction.py:7-16).  Floats go through C so the
    rounding order is exactly left-to-right; integers use NumPy's exact
    wrap-around ufunc reductions."""
    x = np.ascontiguousarray(x)
    if x.dtype == np.float64:
        return np.float64(lib().oracle_fold_f64(_ptr(x), x.size, float(init), OPS[op]))
    if x.dtype == np.float32:
        return np.float32(lib().oracle_fold_f32(_ptr(x), x.size, float(init), OPS[op]))
    t = x.dtype.type
    with np.errstate(over="ignore"):
        if op == "add":
            return t(np.add.reduce(x, dtype=x.dtype, initial=t(init)))
        if op == "mul":
            return t(np.multiply.reduce(x, dtype=x.dtype, initial=t(init)))
        if op == "max":
            return t(max(t(init), x.max())) if x.size else t(init)
        if op == "min":
            return t(min(t(init), x.min())) if x.size else t(init)
        if op == "and":
            return t(np.bitwise_and.reduce(x, initial=t(init)))
        if op == "or":
            return t(np.bitwise_or.reduce(x, initial=t(init)))
        if op == "xor":
            return t(np.bitwise_xor.reduce(x, initial=t(init)))
    raise ValueError(op)


def py_fold(fn, seq, init=0):
    """The simulator's Reduce verbatim in behaviour: functools.reduce(fn, seq, init)
    (simulator/reduction.py:9)."""
    return functools.reduce(fn, seq, init)


def transpose2d(a: np.ndarray) -> np.ndarray:
    """b[j, i] = a[i, j] through the byte-copy loop of b2k_oracle.c (works for any
    itemsize and any input strides)."""
    rows, cols = a.shape
    out = np.empty((cols, rows), dtype=a.dtype)
    base = a
    lib().oracle_transpose2d(base.__array_interface__["data"][0], _ptr(out), rows, cols,
                             a.strides[0], a.strides[1], a.dtype.itemsize)
    return out
