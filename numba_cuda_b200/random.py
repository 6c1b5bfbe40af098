"""xoroshiro128+ random numbers, same names and meaning as numba/cuda/random.py.

State creation runs on the device (every thread jumps straight to its own
subsequence), unlike the reference's serial CPU chain + upload
(random.py:242-282).  Draws: the reference's ``xoroshiro128p_*`` functions are
device functions a user inlines into a ``@cuda.jit`` kernel; here the bulk
equivalent of such a kernel is ``xoroshiro128p_fill`` (one generator per
thread, ``out[t*count + i]`` layout of tests/cudapy/test_random.py:29-53), and
the four scalar names are kept as host-callable functions that draw one value
from ``states[index]`` on the device and return it.
"""
from __future__ import annotations

import threading

import numpy as np
import torch

from . import _lib
from .api import device_array
from .devicearray import DeviceNDArray, _torch_stream, from_cuda_array_interface, stream_ptr

#: random.py:47-49
xoroshiro128p_dtype = np.dtype([("s0", np.uint64), ("s1", np.uint64)], align=True)

_DRAWS = {
    ("uniform", np.dtype(np.float32)): _lib.UNIFORM_F32,
    ("uniform", np.dtype(np.float64)): _lib.UNIFORM_F64,
    ("normal", np.dtype(np.float32)): _lib.NORMAL_F32,
    ("normal", np.dtype(np.float64)): _lib.NORMAL_F64,
}
_DRAW_DTYPE = {_lib.UNIFORM_F32: np.float32, _lib.UNIFORM_F64: np.float64,
               _lib.NORMAL_F32: np.float32, _lib.NORMAL_F64: np.float64}

_tables_lock = threading.Lock()
_tables: dict = {}


def _jump_tables(stream):
    """Seed-independent jump tables, built once per device."""
    dev = torch.cuda.current_device()
    with _tables_lock:
        t = _tables.get(dev)
        if t is None:
            nbytes = int(_lib.lib().b2k_xoroshiro128p_tables_bytes())
            t = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            _lib.check(_lib.lib().b2k_xoroshiro128p_build_tables(t.data_ptr(), nbytes, 0))
            torch.cuda.default_stream().synchronize()
            _tables[dev] = t
        return t


def _as_states(states) -> DeviceNDArray:
    d = states if isinstance(states, DeviceNDArray) else from_cuda_array_interface(states)
    if d.dtype.itemsize != 16 or d.ndim != 1 or d.strides[0] != 16:
        raise TypeError("states must be a 1-D contiguous array of xoroshiro128p_dtype")
    return d


def init_xoroshiro128p_states(states, seed, subsequence_start=0, stream=0):
    """Initialize RNG states on the GPU for parallel generators: state ``i`` is
    ``2**64 * (subsequence_start + i)`` steps into the sequence of ``seed``."""
    d = _as_states(states)
    tables = _jump_tables(stream)
    _lib.check(_lib.lib().b2k_xoroshiro128p_init(
        d._ptr, d.size, int(seed) & (2**64 - 1), int(subsequence_start) & (2**64 - 1),
        tables.data_ptr(), tables.numel(), stream_ptr(stream)))


def create_xoroshiro128p_states(n, seed, subsequence_start=0, stream=0):
    """Returns a new device array initialized for n random number generators."""
    states = device_array(n, dtype=xoroshiro128p_dtype, stream=stream)
    init_xoroshiro128p_states(states, seed, subsequence_start, stream)
    return states


def xoroshiro128p_fill(states, dist, out=None, count=None, dtype=np.float32, stream=0,
                       then=None):
    """Bulk draws: for every generator ``t``, ``out[t, i] = draw(states, t)`` for
    ``i`` in ``range(count)``; ``states`` is advanced in place.

    ``dist`` is ``"uniform"`` or ``"normal"``.  ``out`` (device array of shape
    ``(n, count)``, float32 or float64, C-contiguous) is allocated when absent.
    ``then=(dist2, out2_or_count2, dtype2)`` draws a second block per generator
    right after the first in the same launch (e.g. 64 uniforms then 16 normals).
    Returns ``out`` or ``(out, out2)``."""
    d = _as_states(states)

    def prepare(dist_, out_, count_, dtype_):
        if out_ is None:
            out_ = device_array((d.size, int(count_)), dtype=dtype_, stream=stream)
        elif not isinstance(out_, DeviceNDArray):
            out_ = from_cuda_array_interface(out_)
        if out_.size and not out_.flags["C_CONTIGUOUS"]:
            raise ValueError("output must be C-contiguous")
        cnt = out_.size // d.size if d.size else 0
        if cnt * d.size != out_.size:
            raise ValueError("output size must be a multiple of the number of generators")
        key = (dist_, np.dtype(out_.dtype))
        if key not in _DRAWS:
            raise TypeError(f"no {dist_} draw for dtype {out_.dtype}")
        return out_, cnt, _DRAWS[key]

    out, cnt0, draw0 = prepare(dist, out, count, dtype)
    out2, cnt1, draw1, ptr1 = None, 0, 0, 0
    if then is not None:
        dist2, second, dtype2 = then
        if isinstance(second, (int, np.integer)):
            out2, cnt1, draw1 = prepare(dist2, None, second, dtype2)
        else:
            out2, cnt1, draw1 = prepare(dist2, second, None, dtype2)
        ptr1 = out2._ptr
    _lib.check(_lib.lib().b2k_xoroshiro128p_fill(
        d._ptr, d.size, draw0, out._ptr, cnt0, draw1, ptr1, cnt1, stream_ptr(stream)))
    return out if then is None else (out, out2)


def _draw_one(states, index, draw):
    d = _as_states(states)
    index = int(index)
    if not 0 <= index < d.size:
        raise IndexError("generator index out of range")
    one = d[index:index + 1]
    slot = device_array(1, dtype=_DRAW_DTYPE[draw], stream=d.stream)
    _lib.check(_lib.lib().b2k_xoroshiro128p_fill(one._ptr, 1, draw, slot._ptr, 1, 0, 0, 0,
                                                 stream_ptr(d.stream)))
    return slot.copy_to_host()[0]


def xoroshiro128p_uniform_float32(states, index):
    """Return a float32 in range [0.0, 1.0) and advance ``states[index]``."""
    return _draw_one(states, index, _lib.UNIFORM_F32)


def xoroshiro128p_uniform_float64(states, index):
    """Return a float64 in range [0.0, 1.0) and advance ``states[index]``."""
    return _draw_one(states, index, _lib.UNIFORM_F64)


def xoroshiro128p_normal_float32(states, index):
    """Return a normally distributed float32 and advance ``states[index]``
    (Box-Muller; advances the sequence by two steps)."""
    return _draw_one(states, index, _lib.NORMAL_F32)


def xoroshiro128p_normal_float64(states, index):
    """Return a normally distributed float64 and advance ``states[index]``
    (Box-Muller; advances the sequence by two steps)."""
    return _draw_one(states, index, _lib.NORMAL_F64)


__all__ = [
    "xoroshiro128p_dtype", "init_xoroshiro128p_states", "create_xoroshiro128p_states",
    "xoroshiro128p_fill", "xoroshiro128p_uniform_float32", "xoroshiro128p_uniform_float64",
    "xoroshiro128p_normal_float32", "xoroshiro128p_normal_float64",
]
