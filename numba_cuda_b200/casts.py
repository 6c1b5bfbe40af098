"""Bulk elementwise conversions f32 <-> bf16 / fp8 with the semantics of the
reference's conversion intrinsics (numba/cuda/_internal/cuda_fp8.py:3341-3374,
:1331-1351, :1610-1631; numba/cuda/bf16.py:204-210).

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
_ITEMSIZE = {_lib.FMT_F32: 4, _lib.FMT_BF16: 2, _lib.FMT_E4M3: 1, _lib.FMT_E5M2: 1,
             _lib.FMT_F64: 8, _lib.FMT_F16: 2, _lib.FMT_E8M0: 1}


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
    return np.dtype(np.uint8)


def cast(src, src_format, dst_format, out=None, saturate=saturation_t.SATFINITE, stream=0,
         rounding=cudaRoundMode.cudaRoundNearest):
    """Convert every element of ``src`` (host or device array holding
    ``src_format`` items) to ``dst_format``; returns a device array of the same
    shape.  Round-to-nearest-even pairs: f32 <-> bf16 / e4m3 / e5m2 / f16,
    f64 / bf16 -> e4m3 / e5m2, f64 -> bf16, e8m0 -> bf16 / f32.  With ``rounding``:
    f32 -> bf16 toward zero, +inf or -inf; f32 / f64 / bf16 -> e8m0 toward zero or
    +inf."""
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


# ---- fp8 value types: construct from float (SATFINITE) and convert back --------
def fp8_e4m3(x):
    """``fp8_e4m3(float)`` (cuda_fp8.py:1331-1351): saturating E4M3 code(s)."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_E4M3, saturation_t.SATFINITE)


def fp8_e5m2(x):
    """``fp8_e5m2(float)``: saturating E5M2 code(s)."""
    return _scalar_or_bulk(x, _lib.FMT_F32, _lib.FMT_E5M2, saturation_t.SATFINITE)


def fp8_e4m3_to_float32(codes):
    """``float32(fp8_e4m3)`` (cuda_fp8.py:1610-1631)."""
    return _scalar_or_bulk(codes, _lib.FMT_E4M3, _lib.FMT_F32)


def fp8_e5m2_to_float32(codes):
    return _scalar_or_bulk(codes, _lib.FMT_E5M2, _lib.FMT_F32)


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
]
