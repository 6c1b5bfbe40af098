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


def permute(a, axes=None, b=None):
    """Materialise ``a.transpose(axes)`` for an array of any rank: returns ``b``
    (allocated C-contiguous when not given) with ``b.shape[k] == a.shape[axes[k]]``;
    ``axes=None`` reverses the axes, as NumPy does.  The reference stops at two
    axes (``DeviceNDArrayBase.transpose`` raises for other ranks,
    numba/cuda/cudadrv/devicearray.py:157-168); this is the N-D step after it.
    Two-axis swaps of a C-contiguous array go to the 2-D transpose kernels, every
    other permutation is one ``b2k_assign`` launch."""
    from ..devicearray import _c_strides, assign_strided
    stream = getattr(a, "stream", 0)
    a, _ = auto_device(a, stream=stream)
    nd = a.ndim
    axes = tuple(range(nd))[::-1] if axes is None else tuple(int(x) % nd if nd else int(x) for x in axes)
    if sorted(axes) != list(range(nd)):
        raise ValueError("invalid axes list %r" % (axes,))
    shape = tuple(a.shape[x] for x in axes)
    if b is None:
        b = DeviceNDArray(shape, _c_strides(shape, a.dtype.itemsize), dtype=a.dtype, stream=stream)
    else:
        b, _ = auto_device(b, stream=stream, copy=False)
        if b.dtype != a.dtype:
            raise TypeError("incompatible dtype: %s vs. %s" % (b.dtype, a.dtype))
        if tuple(b.shape) != shape:
            raise ValueError("incompatible shape: %s vs. %s" % (b.shape, shape))
    if a.size == 0:
        return b
    if nd == 2 and axes == (1, 0):
        return transpose(a, b)
    src_strides = tuple(a.strides[x] for x in axes)
    assign_strided(b._ptr, a._ptr, shape, b.strides, src_strides, a.dtype.itemsize, stream)
    return b
