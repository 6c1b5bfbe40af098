"""Host API either side of the library kernels: the subset of
numba/cuda/api.py that ``cuda.reduce``, ``transpose`` and the RNG use or that
their callers need to hand arrays over (``to_device`` api.py:117,
``device_array`` :158, ``device_array_like``, ``as_cuda_array`` :67,
``is_cuda_array`` :88, ``stream`` :398, ``synchronize``, capability probes
:100-113)."""
from __future__ import annotations

import os

import numpy as np
import torch

from .devicearray import (DeviceNDArray, Event, Stream, _c_strides, _f_strides, from_cuda_array_interface,
                          stream_ptr)


def _require_cuda():
    if not torch.cuda.is_available():
        raise RuntimeError("numba_cuda_b200 needs a CUDA device: there is no CPU fallback")


def is_available() -> bool:
    return torch.cuda.is_available()


def is_bfloat16_supported() -> bool:
    """True on compute capability >= 8.0 (driver.py:581-583)."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (8, 0)


def is_fp8_supported() -> bool:
    """True on compute capability >= 8.9 (driver.py:585-586)."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability() >= (8, 9)


def synchronize() -> None:
    torch.cuda.synchronize()


def stream() -> Stream:
    """A new CUDA stream."""
    _require_cuda()
    return Stream()


def event(timing=True) -> Event:
    """A new CUDA event (api.py ``event``)."""
    _require_cuda()
    return Event(timing=timing)


def event_elapsed_time(evtstart: Event, evtend: Event) -> float:
    """Milliseconds between two recorded events (api.py ``event_elapsed_time``)."""
    return evtstart.elapsed_time(evtend)


def default_stream() -> Stream:
    _require_cuda()
    return Stream(torch_stream=torch.cuda.default_stream())


def external_stream(ptr: int) -> Stream:
    """Wrap a stream allocated elsewhere (api.py:414)."""
    return Stream(external_ptr=ptr)


def device_array(shape, dtype=np.float64, strides=None, order="C", stream=0) -> DeviceNDArray:
    """Allocate an empty device ndarray (api.py:158-176)."""
    _require_cuda()
    if isinstance(shape, (int, np.integer)):
        shape = (int(shape),)
    shape = tuple(int(s) for s in shape)
    dtype = np.dtype(dtype)
    if strides is None:
        strides = _c_strides(shape, dtype.itemsize) if order == "C" else _f_strides(shape, dtype.itemsize)
    return DeviceNDArray(shape, strides, dtype, stream=stream)


def strides_like(shape, strides, itemsize):
    """Strides of a new dense array "like" one with the given shape and strides
    (api.py:295-328, which follows NumPy's ``zeros_like``): a C- or F-contiguous
    source keeps its order; any other source keeps the ranking of its axes by
    stride, so the axis that was densest in a view stays densest in the copy."""
    shape, strides = tuple(shape), tuple(strides)
    c, f = _c_strides(shape, itemsize), _f_strides(shape, itemsize)
    size = int(np.prod(shape, dtype=np.int64)) if shape else 1
    if len(shape) <= 1 or size == 0 or strides == c or _dense(shape, strides, c):
        return c
    if strides == f or _dense(shape, strides, f):
        return f
    ranking = sorted(range(len(shape)), key=lambda k: strides[k])   # stable: ties keep axis order
    out, step = [0] * len(shape), itemsize
    for k in ranking:
        out[k] = step
        step *= shape[k]
    return tuple(out)


def _dense(shape, strides, want):
    """Same layout as ``want`` once axes of length 1 (whose stride is free) are ignored."""
    return all(n == 1 or a == b for n, a, b in zip(shape, strides, want))


def device_array_like(ary, stream=0) -> DeviceNDArray:
    """Allocate a dense array with the shape, dtype and axis order of ``ary``
    (api.py:331-344)."""
    shape, dtype = tuple(ary.shape), np.dtype(ary.dtype)
    strides = getattr(ary, "strides", None)
    if strides is None:
        strides = _c_strides(shape, dtype.itemsize)
    return device_array(shape, dtype, strides=strides_like(shape, strides, dtype.itemsize), stream=stream)


def pinned_array_like(ary) -> np.ndarray:
    """Page-locked host array with the shape, dtype and axis order of ``ary`` (api.py:365-374)."""
    shape, dtype = tuple(ary.shape), np.dtype(ary.dtype)
    strides = getattr(ary, "strides", None) or _c_strides(shape, dtype.itemsize)
    like = strides_like(shape, strides, dtype.itemsize)
    n = (int(np.prod(shape, dtype=np.int64)) if shape else 1) * dtype.itemsize
    raw = torch.empty(max(n, 1), dtype=torch.uint8, pin_memory=torch.cuda.is_available()).numpy()
    return np.ndarray(shape, dtype=dtype, buffer=raw, strides=like)


def to_device(obj, stream=0, copy=True, to=None) -> DeviceNDArray:
    """Allocate and transfer a host array to the device (api.py:117-155)."""
    _require_cuda()
    if isinstance(obj, DeviceNDArray):
        return obj
    if is_cuda_array(obj):
        return as_cuda_array(obj)
    host = np.asarray(obj)
    if not (host.flags["C_CONTIGUOUS"] or host.flags["F_CONTIGUOUS"]):
        # devicearray.py:904-915
        raise ValueError("Array contains non-contiguous buffer and cannot be transferred as a single memory region. "
                         "Please ensure contiguous buffer with numpy .ascontiguousarray()")
    if to is None:
        to = DeviceNDArray(host.shape, host.strides if host.size else _c_strides(host.shape, host.dtype.itemsize),
                           host.dtype, stream=stream)
    if copy:
        to.copy_to_device(host, stream=stream)
    return to


def is_cuda_array(obj) -> bool:
    return hasattr(obj, "__cuda_array_interface__")


def as_cuda_array(obj, sync=True) -> DeviceNDArray:
    """Zero-copy view of any CUDA-Array-Interface exporter (api.py:67-85).  If
    the exporter names a stream and ``sync`` is true, that stream is
    synchronised first, as the interface asks of a consumer."""
    if not is_cuda_array(obj):
        raise TypeError("*obj* doesn't implement the cuda array interface.")
    if isinstance(obj, DeviceNDArray):
        return obj
    s = obj.__cuda_array_interface__.get("stream")
    # NUMBA_CUDA_ARRAY_INTERFACE_SYNC=0 switches the synchronisation off globally, as the
    # reference's config.CUDA_ARRAY_INTERFACE_SYNC does (api.py:56-60, core/config.py:480)
    if sync and s and os.environ.get("NUMBA_CUDA_ARRAY_INTERFACE_SYNC", "1") not in ("0", ""):
        if s in (1, 2):
            torch.cuda.default_stream().synchronize()
        else:
            torch.cuda.ExternalStream(int(s)).synchronize()
    return from_cuda_array_interface(obj)


def pinned_array(shape, dtype=np.float64, order="C") -> np.ndarray:
    """Host array in page-locked memory (api.py:203-219)."""
    dtype = np.dtype(dtype)
    shape = (shape,) if isinstance(shape, (int, np.integer)) else tuple(shape)
    n = int(np.prod(shape, dtype=np.int64)) * dtype.itemsize
    raw = torch.empty(max(n, 1), dtype=torch.uint8, pin_memory=torch.cuda.is_available()).numpy()
    return np.ndarray(shape, dtype=dtype, buffer=raw, order=order)


def auto_device(obj, stream=0, copy=True):
    """(device array, whether a transfer happened) -- devicearray.py:918-961."""
    if isinstance(obj, DeviceNDArray):
        return obj, False
    if is_cuda_array(obj):
        return as_cuda_array(obj), False
    return to_device(obj, stream=stream, copy=copy), True


__all__ = [
    "is_available", "is_bfloat16_supported", "is_fp8_supported", "synchronize", "stream", "event",
    "event_elapsed_time",
    "default_stream", "external_stream", "device_array", "device_array_like", "to_device",
    "is_cuda_array", "as_cuda_array", "pinned_array", "pinned_array_like", "auto_device", "stream_ptr",
    "strides_like",
]
