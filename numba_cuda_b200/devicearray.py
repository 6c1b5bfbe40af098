"""Device array shim: the attributes and methods of numba-cuda's
``DeviceNDArray`` that the library kernels and their callers touch
(numba/cuda/cudadrv/devicearray.py:60-330, :578-700), over torch-owned memory.

Memory comes from torch's caching allocator as raw bytes, so any NumPy dtype
(records, bool, bfloat16 from ml_dtypes, complex) can be carried.  This is the
boundary plumbing of the drop-in, not a rebuild of numba's array machinery:
basic indexing, contiguity checks, host/device copies, ``.T`` and the CUDA
Array Interface.
"""
from __future__ import annotations

import copy as _copy
import functools
import math
import operator

import numpy as np
import torch


# ------------------------------------------------------------------ streams
class Stream:
    """A CUDA stream handle (numba/cuda/cudadrv/driver.py:1890 has the same
    surface: ``.handle``, ``synchronize()``, context manager ``auto_synchronize``)."""

    def __init__(self, torch_stream=None, external_ptr=None):
        if external_ptr is not None:
            self._ts = torch.cuda.ExternalStream(int(external_ptr))
        elif torch_stream is not None:
            self._ts = torch_stream
        else:
            self._ts = torch.cuda.Stream()

    @property
    def handle(self) -> int:
        return int(self._ts.cuda_stream)

    def __int__(self) -> int:
        return self.handle

    def synchronize(self) -> None:
        self._ts.synchronize()

    def auto_synchronize(self):
        import contextlib

        @contextlib.contextmanager
        def _cm():
            try:
                yield self
            finally:
                self.synchronize()
        return _cm()

    def __repr__(self):
        return f"<b200 CUDA stream {self.handle:#x}>"


class Event:
    """A CUDA event (numba/cuda/cudadrv/driver.py ``Event``: ``record(stream=0)``,
    ``query()``, ``synchronize()``, ``wait(stream=0)``, ``elapsed_time(evtend)``),
    for timing the library calls the way numba-cuda users time kernels."""

    def __init__(self, timing=True):
        self._ev = torch.cuda.Event(enable_timing=bool(timing))

    def record(self, stream=0):
        self._ev.record(_torch_stream(stream))

    def query(self) -> bool:
        return self._ev.query()

    def synchronize(self) -> None:
        self._ev.synchronize()

    def wait(self, stream=0) -> None:
        _torch_stream(stream).wait_event(self._ev)

    def elapsed_time(self, evtend: "Event") -> float:
        """Milliseconds from this event to ``evtend``."""
        return self._ev.elapsed_time(evtend._ev)


def stream_ptr(stream) -> int:
    """0 / Stream / torch stream / raw pointer -> cudaStream_t value."""
    if stream is None or (isinstance(stream, int) and stream == 0):
        return 0
    if isinstance(stream, Stream):
        return stream.handle
    if hasattr(stream, "cuda_stream"):
        return int(stream.cuda_stream)
    if hasattr(stream, "handle"):
        h = stream.handle
        return int(getattr(h, "value", h) or 0)
    return int(stream)


def _torch_stream(stream):
    ptr = stream_ptr(stream)
    if ptr == 0:
        return torch.cuda.default_stream()
    if isinstance(stream, Stream):
        return stream._ts
    if isinstance(stream, torch.cuda.Stream):
        return stream
    return torch.cuda.ExternalStream(ptr)


# ------------------------------------------------------------------ helpers
def _extent_bytes(shape, strides, itemsize) -> int:
    """Bytes spanned from the first to one past the last item."""
    if any(s == 0 for s in shape):
        return 0
    return sum((n - 1) * abs(st) for n, st in zip(shape, strides)) + itemsize


def _c_strides(shape, itemsize):
    strides = []
    acc = itemsize
    for n in reversed(shape):
        strides.append(acc)
        acc *= max(n, 1)
    return tuple(reversed(strides))


def _f_strides(shape, itemsize):
    strides = []
    acc = itemsize
    for n in shape:
        strides.append(acc)
        acc *= max(n, 1)
    return tuple(strides)


def _is_c_contig(shape, strides, itemsize):
    if any(n == 0 for n in shape):
        return True
    acc = itemsize
    for n, st in zip(reversed(shape), reversed(strides)):
        if n != 1 and st != acc:
            return False
        acc *= n
    return True


def _is_f_contig(shape, strides, itemsize):
    return _is_c_contig(tuple(reversed(shape)), tuple(reversed(strides)), itemsize)


def check_array_compatibility(a, b):
    """Same checks and messages as devicearray.py:1104-1119."""
    sa, sb = np.squeeze(_host_view_desc(a)), np.squeeze(_host_view_desc(b))
    if a.dtype != b.dtype:
        raise TypeError("incompatible dtype: %s vs. %s" % (a.dtype, b.dtype))
    if sa.shape != sb.shape:
        raise ValueError("incompatible shape: %s vs. %s" % (sa.shape, sb.shape))
    if sa.size > 1 and sa.strides != sb.strides:
        raise ValueError("incompatible strides: %s vs. %s" % (sa.strides, sb.strides))


def _host_view_desc(a):
    """A zero-memory NumPy stand-in with a's shape and strides (for squeeze etc.)."""
    if isinstance(a, np.ndarray):
        return a
    base = np.empty(1, dtype=a.dtype)
    return np.lib.stride_tricks.as_strided(base, shape=a.shape, strides=a.strides, writeable=False)


# ------------------------------------------------------------------ the array
class DeviceNDArray:
    """An on-GPU N-d array.  Constructor signature follows
    ``DeviceNDArray(shape, strides, dtype, stream=0, gpu_data=None)``
    (devicearray.py:84); ``gpu_data`` here is a ``(torch uint8 tensor, byte offset)``
    pair or ``None`` to allocate."""

    __array_priority__ = 0  # let NumPy defer to our reflected ops where any

    def __init__(self, shape, strides, dtype, stream=0, gpu_data=None):
        if isinstance(shape, (int, np.integer)):
            shape = (int(shape),)
        if isinstance(strides, (int, np.integer)):
            strides = (int(strides),)
        dtype = np.dtype(dtype)
        shape = tuple(int(s) for s in shape)
        strides = tuple(int(s) for s in strides)
        if len(strides) != len(shape):
            raise ValueError("strides not match ndim")
        self.shape = shape
        self.strides = strides
        self.dtype = dtype
        self.ndim = len(shape)
        self.size = int(np.prod(shape, dtype=np.int64)) if shape else 1
        self.alloc_size = _extent_bytes(shape, strides, dtype.itemsize) if self.size else 0
        self.stream = stream
        if gpu_data is None:
            if not torch.cuda.is_available():
                raise RuntimeError("numba_cuda_b200 needs a CUDA device: there is no CPU fallback")
            with torch.cuda.stream(_torch_stream(stream)):
                buf = torch.empty(max(self.alloc_size, 1), dtype=torch.uint8, device="cuda")
            gpu_data = (buf, 0)
        self._buf, self._offset = gpu_data
        self.gpu_data = gpu_data

    # -- basic facts -------------------------------------------------------
    @property
    def nbytes(self):
        return self.dtype.itemsize * self.size

    @property
    def _ptr(self) -> int:
        return (self._buf.data_ptr() + self._offset) if self.size else 0

    @property
    def device_ctypes_pointer(self):
        import ctypes
        return ctypes.c_void_p(self._ptr or None)

    @property
    def device(self):
        return self._buf.device

    @property
    def flags(self):
        return {
            "C_CONTIGUOUS": _is_c_contig(self.shape, self.strides, self.dtype.itemsize),
            "F_CONTIGUOUS": _is_f_contig(self.shape, self.strides, self.dtype.itemsize),
        }

    def is_c_contiguous(self):
        return self.flags["C_CONTIGUOUS"]

    def is_f_contiguous(self):
        return self.flags["F_CONTIGUOUS"]

    @property
    def __cuda_array_interface__(self):
        contiguous = self.flags["C_CONTIGUOUS"]
        s = stream_ptr(self.stream)
        return {
            "shape": self.shape,
            "strides": None if contiguous else tuple(self.strides),
            "data": (self._ptr, False),
            "typestr": self.dtype.str,
            "descr": self.dtype.descr if self.dtype.names else [("", self.dtype.str)],
            "stream": s if s != 0 else None,
            "version": 3,
        }

    def __len__(self):
        if self.ndim == 0:
            raise TypeError("len() of unsized object")
        return self.shape[0]

    def __repr__(self):
        return f"<b200 DeviceNDArray shape={self.shape} strides={self.strides} dtype={self.dtype}>"

    def bind(self, stream=0):
        clone = _copy.copy(self)
        clone.stream = stream
        return clone

    def _default_stream(self, stream):
        return self.stream if not stream else stream

    def _sub(self, shape, strides, byte_offset, dtype=None):
        return DeviceNDArray(shape, strides, dtype or self.dtype, stream=self.stream,
                             gpu_data=(self._buf, self._offset + byte_offset))

    def _bytes_view(self):
        """torch uint8 view of the spanned bytes (requires non-negative strides)."""
        return self._buf[self._offset:self._offset + self.alloc_size]

    # -- transposition -----------------------------------------------------
    @property
    def T(self):
        return self.transpose()

    def transpose(self, axes=None):
        # devicearray.py:157-168
        if axes and tuple(axes) == tuple(range(self.ndim)):
            return self
        elif self.ndim != 2:
            raise NotImplementedError("transposing a non-2D DeviceNDArray isn't supported")
        elif axes is not None and set(axes) != set(range(self.ndim)):
            raise ValueError("invalid axes list %r" % (axes,))
        else:
            from .kernels.transpose import transpose
            return transpose(self)

    # -- copies --------------------------------------------------------------
    def copy_to_host(self, ary=None, stream=0):
        """Copy to ``ary`` or to a new ndarray with this array's strides
        (devicearray.py:249-304).  Synchronous unless a stream is given."""
        if any(s < 0 for s in self.strides):
            raise NotImplementedError(
                "D->H copy not implemented for negative strides: {}".format(self.strides))
        stream = self._default_stream(stream)
        if ary is not None:
            check_array_compatibility(self, ary)
        if self.alloc_size == 0:
            return ary if ary is not None else np.empty(self.shape, dtype=self.dtype)
        raw = np.empty(self.alloc_size, dtype=np.uint8)
        with torch.cuda.stream(_torch_stream(stream)):
            # a copy into pageable host memory returns once the bytes have landed
            torch.from_numpy(raw).copy_(self._bytes_view())
        view = np.ndarray(shape=self.shape, dtype=self.dtype, strides=self.strides, buffer=raw)
        if ary is None:
            return view
        ary[...] = view
        return ary

    def copy_to_device(self, ary, stream=0):
        """Copy ``ary`` (host ndarray or device array) into self
        (devicearray.py:214-247): self must be contiguous; dtype, squeezed
        shape and strides must agree."""
        if getattr(ary, "size", 1) == 0:
            return
        if not (self.flags["C_CONTIGUOUS"] or self.flags["F_CONTIGUOUS"]):
            raise ValueError("Array contains non-contiguous buffer and cannot be transferred as a single memory region. "
                             "Please ensure contiguous buffer with numpy .ascontiguousarray()")
        stream = self._default_stream(stream)
        ts = _torch_stream(stream)
        if isinstance(ary, DeviceNDArray) or hasattr(ary, "__cuda_array_interface__"):
            src = ary if isinstance(ary, DeviceNDArray) else from_cuda_array_interface(ary)
            if not (src.flags["C_CONTIGUOUS"] or src.flags["F_CONTIGUOUS"]):
                raise ValueError("Array contains non-contiguous buffer and cannot be transferred as a single memory region.")
            check_array_compatibility(self, src)
            with torch.cuda.stream(ts):
                self._bytes_view().copy_(src._bytes_view(), non_blocking=True)
            return
        host = np.asarray(ary)
        host = np.array(host, order="C" if self.flags["C_CONTIGUOUS"] else "F", copy=None)
        check_array_compatibility(self, host)
        raw = _host_bytes(host)
        with torch.cuda.stream(ts):
            self._bytes_view()[: raw.size].copy_(torch.from_numpy(raw))

    # -- views ---------------------------------------------------------------
    def __getitem__(self, item):
        shape, strides, offset = _basic_index(self.shape, self.strides, item)
        if len(shape) == 0 and not _has_slice(item):
            # scalar read: synchronous one-item copy, returns a NumPy scalar
            sub = self._sub((1,), (self.dtype.itemsize,), offset)
            val = sub.copy_to_host()[0]
            return val
        return self._sub(shape, strides, offset)

    def getitem(self, item, stream=0):
        return self.__getitem__(item)

    def __setitem__(self, key, value):
        return self._do_setitem(key, value)

    def setitem(self, key, value, stream=0):
        """Do `__setitem__(key, value)` with CUDA stream"""
        return self._do_setitem(key, value, stream=stream)

    def _do_setitem(self, key, value, stream=0):
        """Broadcasting assignment on the device (devicearray.py:735-791): the
        left side is the indexed view, the right side any device array, host
        array or scalar with at most as many axes; axes of length 1 repeat.
        One ``b2k_assign`` launch; synchronous when no stream is involved."""
        stream = self._default_stream(stream)
        synchronous = not stream
        shape, strides, offset = _basic_index(self.shape, self.strides, key)
        lhs = self._sub(shape, strides, offset)

        if isinstance(value, DeviceNDArray) or hasattr(value, "__cuda_array_interface__"):
            rhs = value if isinstance(value, DeviceNDArray) else from_cuda_array_interface(value)
            if rhs.dtype != self.dtype:
                # values are converted like a NumPy assignment would; on the host
                rhs = _upload(np.asarray(rhs.copy_to_host()).astype(self.dtype), stream)
        else:
            host = np.asarray(value)
            if host.dtype != self.dtype:
                host = host.astype(self.dtype)
            if host.ndim == 0 and 0 < self.dtype.itemsize <= 16:
                fill_strided(lhs._ptr, lhs.shape, lhs.strides, host, stream)
                if synchronous:
                    torch.cuda.current_stream().synchronize()
                return
            rhs = _upload(host, stream)
        if rhs.ndim > lhs.ndim:
            raise ValueError("Can't assign %s-D array to %s-D self" % (rhs.ndim, lhs.ndim))
        lead = lhs.ndim - rhs.ndim
        rhs_shape = (1,) * lead + tuple(rhs.shape)
        rhs_strides = (0,) * lead + tuple(rhs.strides)
        for i, (l, r) in enumerate(zip(lhs.shape, rhs_shape)):
            if r != 1 and l != r:
                raise ValueError("Can't copy sequence with size %d to array axis %d with dimension %d" % (r, i, l))
        src_strides = tuple(0 if r == 1 else st for r, st in zip(rhs_shape, rhs_strides))
        assign_strided(lhs._ptr, rhs._ptr, lhs.shape, lhs.strides, src_strides, self.dtype.itemsize, stream)
        if synchronous:
            torch.cuda.current_stream().synchronize()

    def reshape(self, *newshape, order="C"):
        if len(newshape) == 1 and isinstance(newshape[0], (tuple, list)):
            newshape = tuple(newshape[0])
        newshape = list(int(s) for s in newshape)
        if -1 in newshape:
            known = -int(np.prod(newshape))
            newshape[newshape.index(-1)] = self.size // known if known else 0
        newshape = tuple(newshape)
        if int(np.prod(newshape, dtype=np.int64)) != self.size:
            raise ValueError("total size of new array must be unchanged")
        if order == "C" and self.flags["C_CONTIGUOUS"]:
            return self._sub(newshape, _c_strides(newshape, self.dtype.itemsize), 0)
        if order == "F" and self.flags["F_CONTIGUOUS"]:
            return self._sub(newshape, _f_strides(newshape, self.dtype.itemsize), 0)
        raise NotImplementedError("operation requires copying")

    def ravel(self, order="C"):
        return self.reshape(self.size, order=order)

    def view(self, dtype):
        """Reinterpret the bytes with another dtype (last axis must be contiguous)."""
        dtype = np.dtype(dtype)
        if dtype.itemsize == self.dtype.itemsize:
            return self._sub(self.shape, self.strides, 0, dtype)
        if not self.flags["C_CONTIGUOUS"]:
            raise ValueError("To change to a dtype of a different size, the array must be C-contiguous")
        last_bytes = self.shape[-1] * self.dtype.itemsize
        if last_bytes % dtype.itemsize:
            raise ValueError("When changing to a larger dtype, its size must be a divisor of the total size "
                             "in bytes of the last axis of the array.")
        shape = self.shape[:-1] + (last_bytes // dtype.itemsize,)
        return self._sub(shape, _c_strides(shape, dtype.itemsize), 0, dtype)

    def squeeze(self, axis=None):
        desc = np.squeeze(_host_view_desc(self), axis=axis)
        return self._sub(desc.shape, desc.strides, 0)

    def split(self, section, stream=0):
        """Equal 1-D partitions of ``section`` items (devicearray.py:306-327)."""
        if self.ndim != 1:
            raise ValueError("only support 1d array")
        if self.strides[0] != self.dtype.itemsize:
            raise ValueError("only support unit stride")
        for i in range(int(math.ceil(float(self.size) / section))):
            begin, end = i * section, min((i + 1) * section, self.size)
            yield self._sub((end - begin,), self.strides, begin * self.dtype.itemsize)

    def as_torch(self):
        """Typed torch view (dtypes torch knows; C-contiguous only)."""
        tdt = _TORCH_DTYPES.get(self.dtype.str) or _TORCH_DTYPES.get(self.dtype.name)
        if tdt is None or not self.flags["C_CONTIGUOUS"]:
            raise TypeError(f"no torch view for dtype {self.dtype} / this layout")
        return self._bytes_view()[: self.nbytes].view(tdt).reshape(self.shape)


_TORCH_DTYPES = {
    "|i1": torch.int8, "|u1": torch.uint8, "<i2": torch.int16, "<i4": torch.int32, "<i8": torch.int64,
    "<u2": torch.uint16, "<u4": torch.uint32, "<u8": torch.uint64,
    "<f2": torch.float16, "<f4": torch.float32, "<f8": torch.float64, "|b1": torch.bool,
    "<c8": torch.complex64, "<c16": torch.complex128, "bfloat16": torch.bfloat16,
}


def fill_strided(dst_ptr, shape, dst_strides, value: np.ndarray, stream=0):
    """``dst[idx] = value`` for one item of at most 16 bytes: one ``b2k_fill``
    launch, the item travels in the kernel parameters."""
    import ctypes
    from . import _lib
    nd = len(shape)
    if any(int(n) == 0 for n in shape):
        return
    arr = ctypes.c_int64 * max(nd, 1)
    raw = value.tobytes()
    _lib.check(_lib.lib().b2k_fill(dst_ptr, nd, arr(*[int(v) for v in shape]), arr(*[int(v) for v in dst_strides]),
                                   raw, len(raw), stream_ptr(stream)))


def _upload(host: np.ndarray, stream=0) -> "DeviceNDArray":
    """A C-contiguous host array (0-d included) as a new device array."""
    if not host.flags["C_CONTIGUOUS"]:      # (ascontiguousarray would turn a 0-d array into a 1-d one)
        host = np.ascontiguousarray(host)
    dev = DeviceNDArray(host.shape, _c_strides(host.shape, host.dtype.itemsize), host.dtype, stream=stream)
    if host.size:
        raw = host.reshape(-1).view(np.uint8) if host.dtype.itemsize else host.reshape(-1)
        with torch.cuda.stream(_torch_stream(stream)):
            dev._buf[dev._offset:dev._offset + raw.size].copy_(
                torch.from_numpy(raw if raw.flags.writeable else raw.copy()))
    return dev


def assign_strided(dst_ptr, src_ptr, shape, dst_strides, src_strides, itemsize, stream=0):
    """``dst[idx] = src[idx]`` over ``shape`` with byte strides on both sides
    (source stride 0 = broadcast): one ``b2k_assign`` launch."""
    import ctypes
    from . import _lib
    nd = len(shape)
    if any(int(n) == 0 for n in shape):
        return
    arr = ctypes.c_int64 * max(nd, 1)
    _lib.check(_lib.lib().b2k_assign(
        dst_ptr, src_ptr, nd, arr(*[int(v) for v in shape]), arr(*[int(v) for v in dst_strides]),
        arr(*[int(v) for v in src_strides]), int(itemsize), stream_ptr(stream)))


def _host_bytes(host: np.ndarray) -> np.ndarray:
    """The bytes of a contiguous (C or F) host array, without copying when possible."""
    flat = host.reshape(-1, order="A")
    if not flat.flags["C_CONTIGUOUS"]:
        flat = np.ascontiguousarray(flat)
    if not flat.flags["WRITEABLE"]:
        flat = flat.copy()
    return flat.view(np.uint8) if flat.dtype.itemsize else flat


def _has_slice(item):
    items = item if isinstance(item, tuple) else (item,)
    return any(isinstance(i, slice) or i is Ellipsis for i in items)


def _basic_index(shape, strides, item):
    """Basic (int / slice / Ellipsis) indexing -> (shape, strides, byte offset)."""
    items = list(item) if isinstance(item, tuple) else [item]
    if sum(1 for i in items if i is Ellipsis) > 1:
        raise IndexError("an index can only have a single ellipsis ('...')")
    n_real = sum(1 for i in items if i is not Ellipsis)
    if n_real > len(shape):
        raise IndexError("too many indices for array")
    if Ellipsis in items:
        k = items.index(Ellipsis)
        items[k:k + 1] = [slice(None)] * (len(shape) - n_real)
    items += [slice(None)] * (len(shape) - len(items))
    out_shape, out_strides, offset = [], [], 0
    for idx, n, st in zip(items, shape, strides):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(n)
            length = len(range(start, stop, step))
            offset += start * st if length else 0
            out_shape.append(length)
            out_strides.append(st * step)
        else:
            i = operator.index(idx)
            if i < 0:
                i += n
            if not 0 <= i < n:
                raise IndexError("index out of bounds")
            offset += i * st
    return tuple(out_shape), tuple(out_strides), offset


# ------------------------------------------------------------------ constructors
def from_cuda_array_interface(obj, owner=None) -> DeviceNDArray:
    """Wrap any object exporting ``__cuda_array_interface__`` without copying
    (the import side of numba/cuda/api.py:24-64)."""
    if isinstance(obj, DeviceNDArray):
        return obj
    desc = obj.__cuda_array_interface__
    shape = tuple(desc["shape"])
    dtype = np.dtype(desc.get("descr")) if (desc.get("descr") and len(desc["descr"]) > 1) else np.dtype(desc["typestr"])
    strides = desc.get("strides") or _c_strides(shape, dtype.itemsize)
    ptr = desc["data"][0]
    nbytes = _extent_bytes(shape, strides, dtype.itemsize)
    buf = _ForeignBuffer(ptr, nbytes, obj if owner is None else owner)
    return DeviceNDArray(shape, strides, dtype, stream=desc.get("stream") or 0, gpu_data=(buf.tensor, 0))


class _ForeignBuffer:
    """Keeps a foreign allocation alive and exposes it as a torch uint8 tensor."""

    def __init__(self, ptr, nbytes, owner):
        self.owner = owner
        self.ptr = int(ptr or 0)
        self.nbytes = int(nbytes)
        iface = {"shape": (max(self.nbytes, 1),), "typestr": "|u1", "data": (self.ptr, False), "version": 3}
        holder = type("_CAI", (), {"__cuda_array_interface__": iface, "_owner": owner})()
        self.tensor = torch.as_tensor(holder, device="cuda") if self.ptr else torch.empty(1, dtype=torch.uint8, device="cuda")
        self.tensor._b2k_owner = owner  # lifetime


@functools.lru_cache(maxsize=None)
def bfloat16_dtype():
    """NumPy dtype used for bf16 arrays: ml_dtypes.bfloat16 when importable
    (as numba/cuda/np/numpy_support.py:79-84 does), else raw uint16 bits."""
    try:
        import ml_dtypes
        return np.dtype(ml_dtypes.bfloat16)
    except Exception:  # pragma: no cover
        return np.dtype(np.uint16)
