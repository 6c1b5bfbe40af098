"""2-D device-array transpose, same call surface as
numba/cuda/kernels/transpose.py:10-65: ``transpose(a, b=None)``.

``a`` may be a host ndarray (copied to the device first) or any device array;
``b`` is allocated C-contiguous with shape ``(a.shape[1], a.shape[0])`` on
``a``'s stream when not given.  Any dtype (records, bool, complex, bfloat16)
and any input strides are accepted; the work is done by ``b2k_transpose2d``
(TMA tile kernel for contiguous 1/2/4/8/16-byte items, general kernels
otherwise)."""
from __future__ import annotations

from .. import _lib
from ..api import auto_device
from ..devicearray import DeviceNDArray, stream_ptr


def transpose(a, b=None):
    """Compute the transpose of 'a' and store it into 'b', if given, and
    return it.  If 'b' is not given, allocate a new array and return that."""
    stream = getattr(a, "stream", 0)
    a, _ = auto_device(a, stream=stream)
    if a.ndim != 2:
        raise NotImplementedError("transposing a non-2D DeviceNDArray isn't supported")

    if b is None:
        rows_in, cols_in = a.shape
        item = a.dtype.itemsize
        b = DeviceNDArray((cols_in, rows_in), (item * rows_in, item), dtype=a.dtype, stream=stream)
    else:
        b, _ = auto_device(b, stream=stream, copy=False)
        if b.dtype != a.dtype:
            raise TypeError("incompatible dtype: %s vs. %s" % (b.dtype, a.dtype))
        if tuple(b.shape) != (a.shape[1], a.shape[0]):
            raise ValueError("incompatible shape: %s vs. %s" % (b.shape, (a.shape[1], a.shape[0])))

    if a.size:
        _lib.check(_lib.lib().b2k_transpose2d(
            a._ptr, b._ptr, a.shape[0], a.shape[1], a.strides[0], a.strides[1],
            b.strides[0], b.strides[1], a.dtype.itemsize, stream_ptr(stream)))
    return b
