"""Bulk elementwise conversions with the semantics of the reference's conversion
intrinsics and value types: f32 / f64 / f16 / bf16 <-> fp8 (E4M3, E5M2, E8M0), the
fp8 value types' constructors from and conversion operators to every numeric type,
the packed fp8x2 / fp8x4 types, f32 / f64 <-> bf16 and bf16 <-> integers in the four
rounding modes (numba/cuda/_internal/cuda_fp8.py:223-3654; numba/cuda/bf16.py:204-269).

The reference has no bulk cast: a user writes an elementwise ``@cuda.jit``
kernel over the scalar intrinsics.  ``cast`` is that kernel, precompiled.
Storage on the host side: fp8 codes are ``uint8`` (``__nv_fp8_storage_t``),
bf16 is ``ml_dtypes.bfloat16`` (as numba/cuda/np/numpy_support.py:79-84) or
raw ``uint16`` bits.
"""
from __future__ import annotations

import enum

import numpy as np

from . import _lib
from .api import auto_device, device_array
from .devicearray import DeviceNDArray, bfloat16_dtype, stream_ptr


class saturation_t(enum.IntEnum):
    """cuda_fp8.py:223-226"""
    NOSAT = 0
    SATFINITE = 1


class fp8_interpretation_t(enum.IntEnum):
    """cuda_fp8.py:228-230"""
    E4M3 = 0
    E5M2 = 1


class cudaRoundMode(enum.IntEnum):
    """Rounding modes of the conversion intrinsics (cuda_fp8.py / driver_types.h order)."""
    cudaRoundNearest = 0
    cudaRoundZero = 1
    cudaRoundPosInf = 2
    cudaRoundMinInf = 3


FORMATS = {"f64": _lib.FMT_F64, "float64": _lib.FMT_F64, "f16": _lib.FMT_F16, "float16": _lib.FMT_F16,
           "e8m0": _lib.FMT_E8M0, "fp8_e8m0": _lib.FMT_E8M0, "float8_e8m0fnu": _lib.FMT_E8M0,
           "f32": _lib.FMT_F32, "float32": _lib.FMT_F32, "bf16": _lib.FMT_BF16, "bfloat16": _lib.FMT_BF16,
           "e4m3": _lib.FMT_E4M3, "fp8_e4m3": _lib.FMT_E4M3, "float8_e4m3fn": _lib.FMT_E4M3,
           "e5m2": _lib.FMT_E5M2, "fp8_e5m2": _lib.FMT_E5M2, "float8_e5m2": _lib.FMT_E5M2}
_INT_FORMATS = {"int8": _lib.FMT_I8, "int16": _lib.FMT_I16, "int32": _lib.FMT_I32, "int64": _lib.FMT_I64,
                "uint8": _lib.FMT_U8, "uint16": _lib.FMT_U16, "uint32": _lib.FMT_U32, "uint64": _lib.FMT_U64}
FORMATS.update(_INT_FORMATS)
FORMATS.update({"i8": _lib.FMT_I8, "i16": _lib.FMT_I16, "i32": _lib.FMT_I32, "i64": _lib.FMT_I64,
                "u8": _lib.FMT_U8, "u16": _lib.FMT_U16, "u32": _lib.FMT_U32, "u64": _lib.FMT_U64,
                "bool": _lib.FMT_BOOL, "bool_": _lib.FMT_BOOL})
_ITEMSIZE = {_lib.FMT_F32: 4, _lib.FMT_BF16: 2, _lib.FMT_E4M3: 1, _lib.FMT_E5M2: 1,
             _lib.FMT_F64: 8, _lib.FMT_F16: 2, _lib.FMT_E8M0: 1,
             _lib.FMT_I8: 1, _lib.FMT_I16: 2, _lib.FMT_I32: 4, _lib.FMT_I64: 8,
             _lib.FMT_U8: 1, _lib.FMT_U16: 2, _lib.FMT_U32: 4, _lib.FMT_U64: 8, _lib.FMT_BOOL: 1}
_INT_DTYPES = {code: np.dtype(name) for name, code in _INT_FORMATS.items()}


def _format_code(fmt) -> int:
    if isinstance(fmt, (int, np.integer)):
        return int(fmt)
    key = str(getattr(fmt, "name", fmt)).lower()
    if key not in FORMATS:
        raise ValueError(f"unknown format {fmt!r}")
    return FORMATS[key]


def _storage_dtype(code: int):
    if code == _lib.FMT_F32:
        return np.dtype(np.float32)
    if code == _lib.FMT_BF16:
        return bfloat16_dtype()
    if code == _lib.FMT_F64:
        return np.dtype(np.float64)
    if code == _lib.FMT_F16:
        return np.dtype(np.float16)
    if code in _INT_DTYPES:
        return _INT_DTYPES[code]
    if code == _lib.FMT_BOOL:
        return np.dtype(np.bool_)
    return np.dtype(np.uint8)


def cast(src, src_format, dst_format, out=None, saturate=saturation_t.SATFINITE, stream=0,
         rounding=cudaRoundMode.cudaRoundNearest):
    """Convert every element of ``src`` (host or device array holding
    ``src_format`` items) to ``dst_format``; returns a device array of the same
    shape.  Round-to-nearest-even pairs: f32 <-> bf16 / e4m3 / e5m2 / f16,
    f64 / bf16 -> e4m3 / e5m2, f64 -> bf16, e8m0 -> bf16 / f32.  With ``rounding``:
    f32 -> bf16 toward zero, +inf or -inf; f32 / f64 / bf16 -> e8m0 toward zero or
    +inf.  Integer formats: int16/32/64 and uint16/32/64 <-> bf16 in all four modes
    (bf16 -> int8 / uint8 toward zero); integers -> e4m3 / e5m2 (saturating, nearest)
    and -> e8m0 (saturating, toward +inf); e4m3 / e5m2 / e8m0 -> integers (toward
    zero) and -> bool; e4m3 / e5m2 -> f16 / bf16 / f64, e8m0 -> f16 / f64, f16 -> e4m3 /
    e5m2 / e8m0."""
    s, d = _format_code(src_format), _format_code(dst_format)
    dsrc, _ = auto_device(src, stream=stream)
    if dsrc.dtype.itemsize != _ITEMSIZE[s]:
        raise TypeError(f"source items are {dsrc.dtype.itemsize} bytes, format needs {_ITEMSIZE[s]}")
    if dsrc.size and not dsrc.flags["C_CONTIGUOUS"]:
        raise ValueError("cast needs a C-contiguous source")
    if out is None:
        out = device_array(dsrc.shape, dtype=_storage_dtype(d), stream=stream)
    else:
        out, _ = auto_device(out, stream=stream, copy=False)
        if out.dtype.itemsize != _ITEMSIZE[d] or out.size != dsrc.size or not out.flags["C_CONTIGUOUS"]:
            raise ValueError("out must be C-contiguous with the source's size and the target's item size")
    _lib.check(_lib.lib().b2k_cast_ex(s, d, int(saturate), int(rounding), dsrc._ptr, out._ptr, dsrc.size,
                                      stream_ptr(stream)))
    return out


def _scalar_or_bulk(x, s, d, saturate=saturation_t.SATFINITE, rounding=cudaRoundMode.cudaRoundNearest):
    if isinstance(x, DeviceNDArray) or (isinstance(x, np.ndarray) and x.ndim > 0):
        return cast(x, s, d, saturate=saturate, rounding=rounding)
    dtype = getattr(x, "dtype", None)
    if dtype is not None and np.dtype(dtype).itemsize == _ITEMSIZE[s] and np.dtype(dtype).kind in "iu" \
            and _storage_dtype(s).kind not in "iub":
        host = np.array([x])          # an integer scalar of the format's width: raw bits (bf16, f16, fp8 codes)
    else:
        host = np.array([x], dtype=_storage_dtype(s))
    return cast(host, s, d, saturate=saturate, rounding=rounding).copy_to_host()[0]


# ---- fp8 storage intrinsics (cuda_fp8.py:3341-3410) --------------------------
def cvt_float_to_fp8(x, saturate, fp8_interpretation):
    """float32 -> fp8 code (uint8).  A scalar gives a scalar; an array is
    converted in bulk on the device."""
    d = _lib.FMT_E5M2 if int(fp8_interpretation) == fp8_interpretation_t.E5M2 else _lib.FMT_E4M3
    return _scalar_or_bulk(x, _lib.FMT_F32, d, saturate)


def cvt_float2_to_fp8x2(x, saturate, fp8_interpretation):
    """(float32, float32) -> uint16 holding two codes, ``x[0]`` in the low byte."""
    return _pack2(cvt_float_to_fp8(np.asarray(x, dtype=np.float32).reshape(2), saturate, fp8_interpretation))


def _pair(x, dtype):
    pair = np.asarray(x, dtype=dtype).reshape(-1)
    if pair.size != 2:
        raise ValueError("a two-element value is expected")
    return pair


def _pack2(codes) -> np.uint16:
    lo, hi = (int(v) for v in codes.copy_to_host())
    return np.uint16(lo | (hi << 8))


def cvt_double_to_fp8(x, saturate, fp8_interpretation):
    """float64 -> fp8 code (cuda_fp8.py:3269-3302): one rounding straight from the
    double, not through float32."""
    d = _lib.FMT_E5M2 if int(fp8_interpretation) == fp8_interpretation_t.E5M2 else _lib.FMT_E4M3
    return _scalar_or_bulk(x, _lib.FMT_F64, d, saturate)


def cvt_double2_to_fp8x2(x, saturate, fp8_interpretation):
    """(float64, float64) -> uint16 holding two codes, ``x[0]`` in the low byte
    (cuda_fp8.py:3305-3338)."""
    return _pack2(cvt_double_to_fp8(_pair(x, np.float64), saturate, fp8_interpretation))


def cvt_bfloat16raw_to_fp8(x, saturate, fp8_interpretation):
    """bfloat16 (raw ``uint16`` bits or ml_dtypes values) -> fp8 code
    (cuda_fp8.py:3413-3446)."""
    d = _lib.FMT_E5M2 if int(fp8_interpretation) == fp8_interpretation_t.E5M2 else _lib.FMT_E4M3
    return _scalar_or_bulk(x, _lib.FMT_BF16, d, saturate)


# ---- fp8 value types: constructors and conversion operators ---------------------
def _source_format(x) -> int:
    """The format a value-type constructor sees: the array's (or NumPy scalar's) own
    dtype; a Python float is a float64 and a Python int an int64, as numba types
    literals."""
    dtype = getattr(x, "dtype", None)
    if dtype is None:
        if isinstance(x, bool):
            raise TypeError("no fp8 constructor from bool")
        if isinstance(x, int):
            return _lib.FMT_I64
        if isinstance(x, float):
            return _lib.FMT_F64
        dtype = np.asarray(x).dtype
    dtype = np.dtype(dtype)
    if dtype == bfloat16_dtype() and dtype != np.uint16:
        return _lib.FMT_BF16
    for code in (_lib.FMT_F32, _lib.FMT_F64, _lib.FMT_F16, *_INT_DTYPES):
        if dtype == _storage_dtype(code):
            return code
    raise TypeError(f"no fp8 constructor from {dtype}")


def _construct(x, fmt):
    s = _source_format(x)
    e8 = fmt == _lib.FMT_E8M0
    return _scalar_or_bulk(x, s, fmt, saturation_t.SATFINITE,
                           cudaRoundMode.cudaRoundPosInf if e8 else cudaRoundMode.cudaRoundNearest)


def fp8_e4m3(x):
    """``fp8_e4m3(x)`` (cuda_fp8.py:1562-1607): the saturating E4M3 code(s) of a
    float16 / bfloat16 / float32 / float64 or integer value or array, each source
    type through its own constructor (a float64 is rounded once, an integer goes
    through float32)."""
    return _construct(x, _lib.FMT_E4M3)


def fp8_e5m2(x):
    """``fp8_e5m2(x)`` (cuda_fp8.py:568-613): saturating E5M2 code(s)."""
    return _construct(x, _lib.FMT_E5M2)


def fp8_e8m0(x):
    """``fp8_e8m0(x)`` (cuda_fp8.py:2580-2601): the E8M0 code(s) of the smallest power
    of two not below ``|x|`` (saturating; 0xFF for a NaN)."""
    return _construct(x, _lib.FMT_E8M0)


def _convert(codes, fmt, dtype):
    """``dtype(fp8 value)``: the conversion operators of the value types."""
    if dtype is bool or (not isinstance(dtype, str) and np.dtype(dtype) == np.bool_):
        d = _lib.FMT_BOOL
    elif isinstance(dtype, str) and dtype.lower() in ("bf16", "bfloat16"):
        d = _lib.FMT_BF16
    else:
        dtype = np.dtype(dtype)
        if dtype == bfloat16_dtype() and dtype != np.uint16:
            d = _lib.FMT_BF16
        else:
            d = next((c for c in (_lib.FMT_F32, _lib.FMT_F64, _lib.FMT_F16, *_INT_DTYPES)
                      if dtype == _storage_dtype(c)), None)
            if d is None:
                raise TypeError(f"no conversion from an fp8 value to {dtype}")
    rounding = cudaRoundMode.cudaRoundZero if d in _INT_DTYPES else cudaRoundMode.cudaRoundNearest
    return _scalar_or_bulk(codes, fmt, d, rounding=rounding)


def fp8_e4m3_to(codes, dtype):
    """``dtype(fp8_e4m3)`` (cuda_fp8.py:1610-1944): float16 / bfloat16 / float32 /
    float64 exactly; integers toward zero, clamped to the type's range, NaN as 0
    (0x8000000000000000 for 64 bits); bool is true for anything but a zero."""
    return _convert(codes, _lib.FMT_E4M3, dtype)


def fp8_e5m2_to(codes, dtype):
    """``dtype(fp8_e5m2)`` (cuda_fp8.py:616-926)."""
    return _convert(codes, _lib.FMT_E5M2, dtype)


def fp8_e8m0_to(codes, dtype):
    """``dtype(fp8_e8m0)`` (cuda_fp8.py:2604-2962); to float16 the power of two is
    rounded to nearest (infinity above 2**15); bool is always true."""
    return _convert(codes, _lib.FMT_E8M0, dtype)


def fp8_e4m3_to_float32(codes):
    """``float32(fp8_e4m3)`` (cuda_fp8.py:1610-1631)."""
    return _scalar_or_bulk(codes, _lib.FMT_E4M3, _lib.FMT_F32)


def fp8_e5m2_to_float32(codes):
    return _scalar_or_bulk(codes, _lib.FMT_E5M2, _lib.FMT_F32)


# ---- packed value types: two or four codes in one uint16 / uint32 ------------------
def _packed(x, fmt, lanes):
    """``fp8x2_*`` / ``fp8x4_*`` constructors (cuda_fp8.py:1041-1078, :1192-1229 and
    siblings): the last axis of ``x`` holds the 2 or 4 lanes, lane 0 in the lowest
    byte -- the codes in memory order, so the packing is a view."""
    host_scalar = not isinstance(x, DeviceNDArray)
    if host_scalar:
        x = np.asarray(x)
    if x.ndim < 1 or x.shape[-1] != lanes:
        raise ValueError(f"the last axis must hold the {lanes} lanes")
    codes = _construct(x if not host_scalar else np.ascontiguousarray(x), fmt)
    packed = codes.view(np.uint16 if lanes == 2 else np.uint32)
    if x.ndim == 1:                      # one pair / quadruple: a scalar
        return packed.copy_to_host()[0]
    return packed.reshape(x.shape[:-1])


def _unpacked(packed, fmt, lanes, dtype):
    """``float2(fp8x2)`` / ``float4(fp8x4)`` and the half / bfloat16 forms: the lanes
    come back on a new last axis."""
    want = np.uint16 if lanes == 2 else np.uint32
    scalar = not isinstance(packed, DeviceNDArray) and np.ndim(packed) == 0
    if not isinstance(packed, DeviceNDArray):
        packed = np.ascontiguousarray(np.asarray(packed, dtype=want))   # a scalar becomes one item
    elif packed.dtype != want:
        raise TypeError(f"packed codes must be {np.dtype(want)}")
    dev, _ = auto_device(packed)
    if not dev.flags["C_CONTIGUOUS"]:
        raise ValueError("packed codes must be C-contiguous")
    codes = dev.view(np.uint8)
    out = _convert(codes, fmt, dtype)
    return out.copy_to_host() if scalar else out.reshape(tuple(packed.shape) + (lanes,))


def fp8x2_e4m3(x):
    """Two E4M3 codes per ``uint16`` from pairs on the last axis."""
    return _packed(x, _lib.FMT_E4M3, 2)


def fp8x4_e4m3(x):
    """Four E4M3 codes per ``uint32`` from quadruples on the last axis."""
    return _packed(x, _lib.FMT_E4M3, 4)


def fp8x2_e5m2(x):
    return _packed(x, _lib.FMT_E5M2, 2)


def fp8x4_e5m2(x):
    return _packed(x, _lib.FMT_E5M2, 4)


def fp8x2_e8m0(x):
    return _packed(x, _lib.FMT_E8M0, 2)


def fp8x4_e8m0(x):
    return _packed(x, _lib.FMT_E8M0, 4)


def fp8x2_to(packed, fp8_format, dtype=np.float32):
    """``float2(fp8x2_*)`` / ``half2(...)`` / ``bfloat162(...)``: a ``uint16`` array of
    packed pairs to values with the two lanes on a new last axis."""
    return _unpacked(packed, _format_code(fp8_format), 2, dtype)


def fp8x4_to(packed, fp8_format, dtype=np.float32):
    """``float4(fp8x4_*)``: a ``uint32`` array of packed quadruples to values with the
    four lanes on a new last axis."""
    return _unpacked(packed, _format_code(fp8_format), 4, dtype)


# ---- bf16 (bf16.py:204-207) --------------------------------------------------------
def float32_to_bfloat16(x):
    """Round-to-nearest-even float32 -> bfloat16."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_BF16)


float32_to_bfloat16_rn = float32_to_bfloat16


def bfloat16_to_float32(x):
    return _scalar_or_bulk(x, _lib.FMT_BF16, _lib.FMT_F32)


def float32_to_bfloat16_rz(x):
    """float32 -> bfloat16, rounding toward zero (bf16.py:208)."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_BF16, rounding=cudaRoundMode.cudaRoundZero)


def float32_to_bfloat16_rd(x):
    """float32 -> bfloat16, rounding toward -inf (bf16.py:209)."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_BF16, rounding=cudaRoundMode.cudaRoundMinInf)


def float32_to_bfloat16_ru(x):
    """float32 -> bfloat16, rounding toward +inf (bf16.py:210)."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_BF16, rounding=cudaRoundMode.cudaRoundPosInf)


def float64_to_bfloat16(x):
    """float64 -> bfloat16, round to nearest even in one step (bf16.py:205)."""
    return _scalar_or_bulk(x, _lib.FMT_F64, _lib.FMT_BF16)


# ---- bf16 <-> integers (bf16.py:213-263), bit casts (bf16.py:266-269) ------------------
_MODE_SUFFIX = {"rn": cudaRoundMode.cudaRoundNearest, "rz": cudaRoundMode.cudaRoundZero,
                "rd": cudaRoundMode.cudaRoundMinInf, "ru": cudaRoundMode.cudaRoundPosInf}
_BF16_INT_NAMES = []


def _make_int_bf16(name, code, mode):
    def to_bf16(x):
        return _scalar_or_bulk(x, code, _lib.FMT_BF16, rounding=mode)

    def from_bf16(x):
        return _scalar_or_bulk(x, _lib.FMT_BF16, code, rounding=mode)

    suffix = next(k for k, v in _MODE_SUFFIX.items() if v == mode)
    to_bf16.__name__ = f"{name}_to_bfloat16_{suffix}"
    to_bf16.__doc__ = f"{name} -> bfloat16, rounding mode {suffix} (one step, all of the integer's bits seen)."
    from_bf16.__name__ = f"bfloat16_to_{name}_{suffix}"
    from_bf16.__doc__ = (f"bfloat16 -> {name}, rounding mode {suffix}; saturating, NaN gives 0 "
                         "(0x8000000000000000 for 64 bits).")
    return to_bf16, from_bf16


for _name in ("int16", "uint16", "int32", "uint32", "int64", "uint64"):
    for _mode in _MODE_SUFFIX.values():
        _to, _from = _make_int_bf16(_name, _INT_FORMATS[_name], _mode)
        globals()[_to.__name__] = _to
        globals()[_from.__name__] = _from
        _BF16_INT_NAMES += [_to.__name__, _from.__name__]
for _name in ("int8", "uint8"):   # the reference has these toward zero only
    _, _from = _make_int_bf16(_name, _INT_FORMATS[_name], cudaRoundMode.cudaRoundZero)
    globals()[_from.__name__] = _from
    _BF16_INT_NAMES.append(_from.__name__)


def _bits_view(x, dtype):
    if isinstance(x, DeviceNDArray):
        return x.view(dtype)
    return np.asarray(x).view(dtype) if np.ndim(x) else np.array([x]).view(dtype)[0]


def bfloat16_as_int16(x):
    """The bits of a bfloat16 as int16 (no conversion)."""
    return _bits_view(x, np.int16)


def bfloat16_as_uint16(x):
    return _bits_view(x, np.uint16)


def int16_as_bfloat16(x):
    """An int16 bit pattern as bfloat16 (no conversion)."""
    return _bits_view(x if getattr(x, "dtype", None) is not None else np.int16(x), bfloat16_dtype())


def uint16_as_bfloat16(x):
    return _bits_view(x if getattr(x, "dtype", None) is not None else np.uint16(x), bfloat16_dtype())


# ---- E8M0: the 8-bit power-of-two scale type (cuda_fp8.py:3449-3654) -----------------
def _e8m0_rounding(rounding):
    rounding = cudaRoundMode(int(rounding))
    if rounding not in (cudaRoundMode.cudaRoundZero, cudaRoundMode.cudaRoundPosInf):
        raise ValueError("e8m0 conversions round toward zero or toward +inf")
    return rounding


def cvt_float_to_e8m0(x, saturate, rounding):
    """float32 -> E8M0 code (uint8; 0xFF is NaN)."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_E8M0, saturate, _e8m0_rounding(rounding))


def cvt_bfloat16raw_to_e8m0(x, saturate, rounding):
    """bfloat16 (raw bits or ml_dtypes values) -> E8M0 code."""
    return _scalar_or_bulk(x, _lib.FMT_BF16, _lib.FMT_E8M0, saturate, _e8m0_rounding(rounding))


def cvt_double_to_e8m0(x, saturate, rounding):
    """float64 -> E8M0 code (cuda_fp8.py:3557-3590)."""
    return _scalar_or_bulk(x, _lib.FMT_F64, _lib.FMT_E8M0, saturate, _e8m0_rounding(rounding))


def cvt_float2_to_e8m0x2(x, saturate, rounding):
    """(float32, float32) -> uint16 holding two E8M0 codes, ``x[0]`` in the low
    byte (cuda_fp8.py:3521-3554)."""
    return _pack2(cvt_float_to_e8m0(_pair(x, np.float32), saturate, rounding))


def cvt_double2_to_e8m0x2(x, saturate, rounding):
    """(float64, float64) -> uint16 holding two E8M0 codes (cuda_fp8.py:3593-3626)."""
    return _pack2(cvt_double_to_e8m0(_pair(x, np.float64), saturate, rounding))


def cvt_e8m0_to_bf16raw(codes):
    """E8M0 code -> bfloat16 (``2**(code-127)``; code 0 is the bf16 denormal 2**-127)."""
    return _scalar_or_bulk(codes, _lib.FMT_E8M0, _lib.FMT_BF16)


def fp8_e8m0_to_float32(codes):
    """``float32(fp8_e8m0)``."""
    return _scalar_or_bulk(codes, _lib.FMT_E8M0, _lib.FMT_F32)


def float32_to_float16(x):
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_F16)


def float16_to_float32(x):
    return _scalar_or_bulk(x, _lib.FMT_F16, _lib.FMT_F32)


__all__ = [
    "cast", "saturation_t", "fp8_interpretation_t", "cvt_float_to_fp8", "cvt_float2_to_fp8x2",
    "fp8_e4m3", "fp8_e5m2", "fp8_e4m3_to_float32", "fp8_e5m2_to_float32",
    "float32_to_bfloat16", "float32_to_bfloat16_rn", "bfloat16_to_float32",
    "cudaRoundMode", "float32_to_bfloat16_rz", "float32_to_bfloat16_rd", "float32_to_bfloat16_ru",
    "float64_to_bfloat16", "cvt_float_to_e8m0", "cvt_bfloat16raw_to_e8m0", "cvt_e8m0_to_bf16raw",
    "cvt_double_to_fp8", "cvt_double2_to_fp8x2", "cvt_bfloat16raw_to_fp8", "cvt_double_to_e8m0",
    "cvt_float2_to_e8m0x2", "cvt_double2_to_e8m0x2",
    "fp8_e8m0_to_float32", "float32_to_float16", "float16_to_float32",
    "fp8_e8m0", "fp8_e4m3_to", "fp8_e5m2_to", "fp8_e8m0_to",
    "fp8x2_e4m3", "fp8x4_e4m3", "fp8x2_e5m2", "fp8x4_e5m2", "fp8x2_e8m0", "fp8x4_e8m0", "fp8x2_to", "fp8x4_to",
    "bfloat16_as_int16", "bfloat16_as_uint16", "int16_as_bfloat16", "uint16_as_bfloat16",
    *_BF16_INT_NAMES,
]
