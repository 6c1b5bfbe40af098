"""``cuda.reduce`` / ``Reduce``: full reduction of a 1-D array with a user's
binary function, on one sm_100a kernel launch.

Same call surface as numba/cuda/kernels/reduction.py:169-265:
``Reduce(functor)(arr, size=None, res=None, init=0, stream=0)``.

The reference JIT-compiles the Python functor into its kernel.  Here the
functor is traced into a C++ expression (``_trace.py``).  When that expression is
one of the plain forms of the ops the precompiled kernels carry (add, mul, max,
min, and, or, xor) and the functor also agrees with that op on a fixed set of
sample pairs, the precompiled kernel runs.  Any other traceable functor has the
reduce kernel compiled around its expression at run time with NVRTC
(``b2k_reduce_expr``).  A functor that cannot be traced raises
``NotImplementedError`` -- nothing is ever computed on the CPU instead.
"""
from __future__ import annotations

import random
import threading

import numpy as np
import torch

from .. import _lib
from ..api import auto_device
from ..devicearray import DeviceNDArray, _torch_stream, check_array_compatibility, stream_ptr

_WARPSIZE = 32
_NUMWARPS = 4

_DTYPE_CODES = {
    np.dtype(np.int8): _lib.I8, np.dtype(np.int16): _lib.I16, np.dtype(np.int32): _lib.I32,
    np.dtype(np.int64): _lib.I64, np.dtype(np.uint8): _lib.U8, np.dtype(np.uint16): _lib.U16,
    np.dtype(np.uint32): _lib.U32, np.dtype(np.uint64): _lib.U64,
    np.dtype(np.float32): _lib.F32, np.dtype(np.float64): _lib.F64,
}

_OP_TABLE = [
    ("add", _lib.ADD, lambda a, b: a + b),
    ("mul", _lib.MUL, lambda a, b: a * b),
    ("max", _lib.MAX, lambda a, b: b if b > a else a),
    ("min", _lib.MIN, lambda a, b: b if b < a else a),
    ("and", _lib.AND, lambda a, b: a & b),
    ("or", _lib.OR, lambda a, b: a | b),
    ("xor", _lib.XOR, lambda a, b: a ^ b),
]
OP_NAMES = {code: name for name, code, _ in _OP_TABLE}


def _sample_pairs(kind: str):
    rng = random.Random(0xB200)
    if kind == "f":
        fixed = [(0.0, 0.0), (1.0, 1.0), (0.0, 3.5), (3.5, 0.0), (-2.25, 7.5), (7.5, -2.25),
                 (-1.5, -4.0), (0.5, 0.25), (2.0, 2.0)]
        rnd = [(rng.uniform(-50, 50), rng.uniform(-50, 50)) for _ in range(40)]
    elif kind == "u":
        fixed = [(0, 0), (1, 1), (0, 5), (5, 0), (12, 10), (10, 12), (255, 1), (6, 3), (7, 7)]
        rnd = [(rng.randrange(0, 1000), rng.randrange(0, 1000)) for _ in range(40)]
    else:
        fixed = [(0, 0), (1, 1), (0, 5), (5, 0), (-3, 7), (7, -3), (-4, -9), (12, 10), (6, 3), (-1, -1)]
        rnd = [(rng.randrange(-1000, 1000), rng.randrange(-1000, 1000)) for _ in range(40)]
    return fixed + rnd


def classify_functor(functor, dtype) -> int:
    """Return the table op code ``functor`` computes on ``dtype`` or raise
    ``NotImplementedError``.  Pure host logic: probes the functor on Python
    scalars (ints for integer dtypes, floats for float dtypes)."""
    dtype = np.dtype(dtype)
    if dtype not in _DTYPE_CODES:
        raise NotImplementedError(f"cuda.reduce: dtype {dtype} has no precompiled kernel")
    kind = dtype.kind
    pairs = _sample_pairs(kind)
    matches = []
    for name, code, ref in _OP_TABLE:
        if kind == "f" and name in ("and", "or", "xor"):
            continue
        ok = True
        for a, b in pairs:
            try:
                got = functor(a, b)
            except Exception:
                ok = False
                break
            want = ref(a, b)
            if isinstance(got, (bool, np.bool_)) or got != want:
                ok = False
                break
        if ok:
            matches.append(code)
    if len(matches) == 1:
        return matches[0]
    raise NotImplementedError(
        "cuda.reduce: the binary function is not one of the precompiled ops "
        "(a+b, a*b, max(a,b), min(a,b), a&b, a|b, a^b)")


def _canonical_forms():
    """The expressions the tracer produces for the table ops themselves."""
    forms = {code: set() for _, code, _ in _OP_TABLE}
    for sym, code in (("+", _lib.ADD), ("*", _lib.MUL), ("&", _lib.AND), ("|", _lib.OR), ("^", _lib.XOR)):
        forms[code] |= {f"(a {sym} b)", f"(b {sym} a)"}
    picks_a = ["(a > b)", "(a >= b)", "(b < a)", "(b <= a)"]      # true when a is the larger
    picks_b = ["(b > a)", "(b >= a)", "(a < b)", "(a <= b)"]
    for cond in picks_a:
        forms[_lib.MAX].add(f"({cond} ? a : b)")
        forms[_lib.MIN].add(f"({cond} ? b : a)")
    for cond in picks_b:
        forms[_lib.MAX].add(f"({cond} ? b : a)")
        forms[_lib.MIN].add(f"({cond} ? a : b)")
    return forms


_CANONICAL = _canonical_forms()


class _Scratch:
    """Kernel scratch (ticket + partials) per (device, stream): zero-filled once, the
    kernel leaves it reusable, and calls on one stream are ordered, so every host
    thread may share it.  The result slot and its page-locked landing buffer are
    per (device, stream, host thread): two threads reducing on one stream must not
    read each other's result (the reference allocates fresh partials per call,
    reduction.py:236-241)."""

    _lock = threading.Lock()
    _pool: dict = {}
    _local = threading.local()

    @classmethod
    def get(cls, stream):
        key = (torch.cuda.current_device(), stream_ptr(stream))
        with cls._lock:
            entry = cls._pool.get(key)
            if entry is None:
                nbytes = int(_lib.lib().b2k_reduce_scratch_bytes())
                with torch.cuda.stream(_torch_stream(stream)):
                    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
                entry = (scratch, nbytes)
                cls._pool[key] = entry
        mine = cls._local.__dict__.setdefault("slots", {})
        own = mine.get(key)
        if own is None:
            with torch.cuda.stream(_torch_stream(stream)):
                own = (torch.zeros(16, dtype=torch.uint8, device="cuda"),
                       torch.zeros(16, dtype=torch.uint8, pin_memory=True))
            mine[key] = own
        return entry[0], own[0], entry[1], own[1]


class Reduce:
    """Create a reduction object that reduces values using a given binary
    function.  The classification of the function is cached per
    ``(functor, dtype)`` on the class, like the reference's kernel cache
    (reduction.py:175-192)."""

    _cache: dict = {}

    def __init__(self, functor):
        self._functor = functor

    def _compile(self, dtype):
        """Table op code for ``(functor, dtype)``, or a C++ expression string when the
        functor is not a table op (it is then compiled into the kernel at run time)."""
        key = self._functor, np.dtype(dtype)
        op = self._cache.get(key)
        if op is None:
            from ._trace import trace_functor
            if np.dtype(dtype) not in _DTYPE_CODES:
                raise NotImplementedError(f"cuda.reduce: dtype {np.dtype(dtype)} has no kernel")
            try:
                expr = trace_functor(self._functor, dtype)
            except NotImplementedError:
                expr = None
            try:
                table = classify_functor(self._functor, dtype)
            except NotImplementedError:
                table = None
            if table is not None and expr in _CANONICAL[table]:
                # the samples AND the function's own structure say it is this op
                op = table
            elif expr is not None:
                # anything else that can be followed runs as what it is (a function that
                # only looks like a table op on the samples -- a cap, a modulus, a
                # threshold -- included)
                op = expr
            else:
                # Not followable (math.*, float(), NumPy calls ...): agreeing with a table
                # op on the samples proves nothing about the values not sampled.
                raise NotImplementedError(
                    "cuda.reduce: the binary function can be neither traced nor identified as one of "
                    "a+b, a*b, max(a,b), min(a,b), a&b, a|b, a^b")
            self._cache[key] = op
        return op

    def __call__(self, arr, size=None, res=None, init=0, stream=0, _fold_init=True, *, input_ready=False):
        """Performs a full reduction.

        :param arr: A host or device array (1-D).
        :param size: Optional number of leading elements to reduce.
        :param res: Optional device array; the result is written to its first
                    element and nothing is copied back to the host.
        :param init: Initial value; it is always folded into the result.
        :param stream: Optional CUDA stream (0 = default stream).
        :param input_ready: (not in the reference) promise that ``arr`` is not written by
                    the kernel that precedes this call on ``stream``: a run of reductions
                    with ``res`` given then overlap, each reading its input while the one
                    before finishes.  Table ops on device arrays only; ignored otherwise.
        :return: ``None`` if ``res`` is given, else a NumPy scalar of ``arr.dtype``.
        """
        # reduction.py:217-228
        if arr.ndim != 1:
            raise TypeError("only support 1D array")
        if size is not None:
            arr = arr[:size]
        init = arr.dtype.type(init)
        if arr.size < 1:
            return init

        op = self._compile(arr.dtype)
        darr, staged = auto_device(arr, stream=stream)
        if darr.strides[0] != darr.dtype.itemsize:
            darr, staged = _gather_contiguous(darr, stream), True

        scratch, slot, scratch_bytes, landing = _Scratch.get(stream)
        if res is not None:
            dres, _ = auto_device(res, stream=stream)
            if not (dres.ndim == 1 and dres.shape[0] >= 1 and dres.dtype == arr.dtype):
                # the reference copies partials[:1] into res[:1] (reduction.py:260-261)
                check_array_compatibility(dres[:1], _OneItem(arr.dtype))
            out_ptr = dres._ptr
        else:
            out_ptr = slot.data_ptr()

        init_host = np.array([init], dtype=arr.dtype)
        if isinstance(op, str):
            # a traced function has no identity; the sharded wrapper asks for the bare fold
            _lib.check(_lib.lib().b2k_reduce_expr(
                op.encode(), _DTYPE_CODES[np.dtype(arr.dtype)], darr._ptr, darr.size,
                init_host.ctypes.data if _fold_init else None,
                out_ptr, scratch.data_ptr(), scratch_bytes, stream_ptr(stream)))
        else:
            # a host array was copied by this call, a strided one gathered: both are written
            # by the work just before the kernel, so the promise cannot hold for them
            ready = bool(input_ready) and not staged
            _lib.check(_lib.lib().b2k_reduce_ex(
                op, _DTYPE_CODES[np.dtype(arr.dtype)], darr._ptr, darr.size, init_host.ctypes.data,
                out_ptr, scratch.data_ptr(), scratch_bytes, _lib.REDUCE_INPUT_READY if ready else 0,
                stream_ptr(stream)))
        if res is not None:
            return None
        # one item back through a page-locked landing buffer, ordered on the call's stream
        ts = _torch_stream(stream)
        if torch.cuda.current_stream() == ts:
            landing.copy_(slot, non_blocking=True)
        else:
            with torch.cuda.stream(ts):
                landing.copy_(slot, non_blocking=True)
        ts.synchronize()
        return landing.numpy()[: arr.dtype.itemsize].view(arr.dtype)[0]


    def along_axis(self, arr, axis, res=None, init=0, stream=0):
        """Reduce a 2-D array along ``axis`` (0: over rows, one result per column;
        1: over columns, one result per row).  ``init`` is folded into every
        result, as ``__call__`` folds it into its one.  Returns a 1-D device array
        (``res`` if given).  C-contiguous arrays of more than two axes are reduced
        along one axis too and give an array of the remaining shape.  The reference
        stops at 1-D arrays (reduction.py:217-218); table ops only."""
        if arr.ndim > 2:
            return self._along_axis_nd(arr, axis, res, init, stream)
        if arr.ndim != 2:
            raise TypeError("only support 2D array")
        if axis not in (0, 1, -1, -2):
            raise ValueError("axis %r is out of bounds for a 2D array" % (axis,))
        axis %= 2
        dtype = np.dtype(arr.dtype)
        op = self._compile(dtype)
        if isinstance(op, str):
            raise NotImplementedError("axis-wise reduction supports the precompiled table ops only")
        darr, _ = auto_device(arr, stream=stream)
        item = dtype.itemsize
        rows, cols = darr.shape
        if darr.strides[1] == item or cols <= 1:
            pitch = darr.strides[0] if rows > 1 else max(cols, 1) * item
        elif darr.strides[0] == item or rows <= 1:
            # columns are the contiguous runs: the same bytes are a row-major matrix
            # of the transposed shape, reduced along the other axis
            rows, cols, axis = cols, rows, 1 - axis
            pitch = darr.strides[1] if rows > 1 else max(cols, 1) * item
        else:
            raise ValueError("one axis of the array must be contiguous")
        if pitch < cols * item:
            raise ValueError("rows of the array overlap")
        outputs = cols if axis == 0 else rows
        if res is None:
            from ..api import device_array
            dres = device_array(outputs, dtype, stream=stream)
        else:
            dres, _ = auto_device(res, stream=stream, copy=False)
            if np.dtype(dres.dtype) != dtype:
                raise TypeError("incompatible dtype: %s vs. %s" % (dres.dtype, dtype))
            if dres.ndim != 1 or dres.shape[0] != outputs or (outputs > 1 and dres.strides[0] != item):
                raise ValueError("incompatible shape: res must be a contiguous 1-D array of %d items" % outputs)
        L = _lib.lib()
        need = int(L.b2k_reduce_axis_scratch_bytes(rows, cols, _DTYPE_CODES[dtype], axis))
        scratch = _AxisScratch.get(stream, need)
        init_host = np.array([init], dtype=dtype)
        _lib.check(L.b2k_reduce_axis(op, _DTYPE_CODES[dtype], darr._ptr, rows, cols, pitch, axis,
                                     init_host.ctypes.data, dres._ptr, scratch.data_ptr() if need else None,
                                     need, stream_ptr(stream)))
        return dres


    def _along_axis_nd(self, arr, axis, res, init, stream):
        """One axis of a C-contiguous N-D array: the axes before it fold into an outer
        count, the axes behind it into an inner run.  inner == 1 or outer == 1 is one
        matrix reduction; otherwise every outer slab is a (length x inner) matrix
        reduced along its rows."""
        from ..api import device_array
        nd = arr.ndim
        if not -nd <= axis < nd:
            raise ValueError("axis %r is out of bounds for an array of %d axes" % (axis, nd))
        axis %= nd
        darr, _ = auto_device(arr, stream=stream)
        if not darr.flags["C_CONTIGUOUS"]:
            raise ValueError("arrays of more than two axes must be C-contiguous")
        dtype, item = np.dtype(darr.dtype), np.dtype(darr.dtype).itemsize
        shape = darr.shape
        outer = int(np.prod(shape[:axis], dtype=np.int64))
        length = shape[axis]
        inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
        out_shape = shape[:axis] + shape[axis + 1:]
        if res is None:
            dres = device_array(out_shape, dtype, stream=stream)
        else:
            dres, _ = auto_device(res, stream=stream, copy=False)
            if np.dtype(dres.dtype) != dtype:
                raise TypeError("incompatible dtype: %s vs. %s" % (dres.dtype, dtype))
            if tuple(dres.shape) != tuple(out_shape) or not dres.flags["C_CONTIGUOUS"]:
                raise ValueError("incompatible shape: res must be a C-contiguous array of shape %s" % (out_shape,))
        if outer * inner == 0:
            return dres
        flat = dres._sub((outer * inner,), (item,), 0)
        if inner == 1:
            self.along_axis(darr._sub((outer, length), (length * item, item), 0), 1, res=flat, init=init, stream=stream)
        elif outer == 1:
            self.along_axis(darr._sub((length, inner), (inner * item, item), 0), 0, res=flat, init=init, stream=stream)
        else:
            # every outer slab is a (length x inner) matrix reduced along its rows: one launch
            # over the batch of slabs (65535 per launch)
            op = self._compile(dtype)
            if isinstance(op, str):
                raise NotImplementedError("axis-wise reduction supports the precompiled table ops only")
            L = _lib.lib()
            code = _DTYPE_CODES[dtype]
            slab = length * inner * item
            init_host = np.array([init], dtype=dtype)
            for first in range(0, outer, 65535):
                count = min(65535, outer - first)
                need = int(L.b2k_reduce_cols_batched_scratch_bytes(count, length, inner, code))
                scratch = _AxisScratch.get(stream, need)
                _lib.check(L.b2k_reduce_cols_batched(
                    op, code, darr._ptr + first * slab, count, length, inner, inner * item, slab,
                    init_host.ctypes.data, flat._ptr + first * inner * item,
                    scratch.data_ptr() if need else None, need, stream_ptr(stream)))
        return dres


class _AxisScratch:
    """Per (device, stream) zero-initialised scratch for the axis-wise kernels,
    regrown when a shape needs more (the kernels leave it zeroed where it must be)."""

    _lock = threading.Lock()
    _pool: dict = {}

    @classmethod
    def get(cls, stream, nbytes):
        key = (torch.cuda.current_device(), stream_ptr(stream))
        with cls._lock:
            buf = cls._pool.get(key)
            if buf is None or buf.numel() < nbytes:
                with torch.cuda.stream(_torch_stream(stream)):
                    buf = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device="cuda")
                cls._pool[key] = buf
            return buf


class _OneItem:
    """Shape/stride descriptor of ``partials[:1]`` for the compatibility check."""

    def __init__(self, dtype):
        self.dtype = np.dtype(dtype)
        self.shape = (1,)
        self.strides = (self.dtype.itemsize,)
        self.size = 1


def _gather_contiguous(darr: DeviceNDArray, stream) -> DeviceNDArray:
    """Unit-stride copy of a strided 1-D device view (device-side gather)."""
    step = darr.strides[0]
    item = darr.dtype.itemsize
    if step <= 0 or step % item:
        raise NotImplementedError("cuda.reduce: only positive item-multiple strides are supported")
    from ..api import device_array
    from ..devicearray import assign_strided
    out = device_array(darr.size, darr.dtype, stream=stream)
    assign_strided(out._ptr, darr._ptr, (darr.size,), (item,), (step,), item, stream)
    return out


reduce = Reduce
