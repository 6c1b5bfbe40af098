"""Axis-wise reduction of a matrix (b2k_reduce_axis) against NumPy's
``ufunc.reduce(..., axis=..., dtype=x.dtype)``: exact for integers (wrap-around at
the dtype's width, like b2k_reduce), within 1e-12 (float64) / 1e-5 (float32)
relative for floating-point sums and products."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

import numba_cuda_b200 as cuda  # noqa: E402

FUNCTORS = {
    "add": (lambda a, b: a + b, np.add),
    "mul": (lambda a, b: a * b, np.multiply),
    "max": (lambda a, b: max(a, b), np.maximum),
    "min": (lambda a, b: min(a, b), np.minimum),
    "and": (lambda a, b: a & b, np.bitwise_and),
    "or": (lambda a, b: a | b, np.bitwise_or),
    "xor": (lambda a, b: a ^ b, np.bitwise_xor),
}
REDUCERS = {k: cuda.Reduce(f) for k, (f, _) in FUNCTORS.items()}
INT_DTYPES = [np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64]


def _data(shape, dtype, seed, op="add"):
    rng = np.random.default_rng(seed)
    dtype = np.dtype(dtype)
    if dtype.kind == "f":
        if op == "mul":
            return (1.0 + 0.01 * rng.standard_normal(shape)).astype(dtype)
        return rng.standard_normal(shape).astype(dtype)
    info = np.iinfo(dtype)
    return rng.integers(info.min, info.max, size=shape, dtype=dtype, endpoint=True)


def _want(name, host, axis, init):
    ufunc = FUNCTORS[name][1]
    with np.errstate(over="ignore"):
        if host.shape[axis] == 0:
            return np.full(host.shape[1 - axis], init, dtype=host.dtype)
        red = ufunc.reduce(host, axis=axis, dtype=host.dtype)
        return ufunc(red, host.dtype.type(init), dtype=host.dtype)


def _check(name, host, axis, init=0, dev=None):
    got = REDUCERS[name].along_axis(host if dev is None else dev, axis, init=init).copy_to_host()
    want = _want(name, host, axis, init)
    assert got.shape == want.shape and got.dtype == want.dtype
    if host.dtype.kind == "f" and name in ("add", "mul"):
        tol = 1e-12 if host.dtype == np.float64 else 1e-5
        scale = np.abs(host.astype(np.float64)).sum(axis=axis) if name == "add" else np.abs(want)
        assert (np.abs(got.astype(np.float64) - want.astype(np.float64)) <= tol * np.maximum(scale, 1e-300)).all()
    else:
        assert got.tobytes() == want.tobytes()


SHAPES = [(1, 1), (1, 7), (7, 1), (3, 4), (5, 16), (33, 65), (64, 128), (257, 130), (1000, 36), (36, 1000),
          (2, 5000), (5000, 2), (129, 4096), (4096, 12), (300, 1027)]


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("dtype", INT_DTYPES)
@pytest.mark.parametrize("name", list(FUNCTORS))
def test_integer_ops_every_dtype_exact(name, dtype, axis):
    for k, shape in enumerate(SHAPES):
        host = _data(shape, dtype, 100 + k)
        _check(name, host, axis, init={"and": -1 if np.dtype(dtype).kind == "i" else np.iinfo(dtype).max,
                                       "mul": 1, "min": np.iinfo(dtype).max, "max": np.iinfo(dtype).min}.get(name, 0))


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("name", ["add", "mul", "max", "min"])
def test_float_ops(name, dtype, axis):
    for k, shape in enumerate(SHAPES):
        host = _data(shape, dtype, 200 + k, name)
        _check(name, host, axis, init={"mul": 1, "min": np.inf, "max": -np.inf}.get(name, 0))


@pytest.mark.parametrize("axis", [0, 1])
def test_init_is_folded_into_every_output(axis):
    host = _data((50, 70), np.int32, 1)
    _check("add", host, axis, init=12345)
    _check("max", host, axis, init=2 ** 31 - 5)
    f = _data((50, 70), np.float64, 2)
    _check("add", f, axis, init=-3.5)


def test_empty_axes():
    for shape in ((0, 5), (5, 0)):
        host = np.zeros(shape, dtype=np.int32)
        for axis in (0, 1):
            _check("add", host, axis, init=7)
            _check("max", host, axis, init=-4)


@pytest.mark.parametrize("axis", [0, 1])
def test_views_pitched_unaligned_and_fortran_order(axis):
    base = _data((300, 517), np.float32, 3)
    dev = cuda.to_device(base)
    _check("add", base[:, 3:260], axis, dev=dev[:, 3:260])          # 4-byte aligned rows only: item path
    _check("max", base[10:290, 4:260], axis, dev=dev[10:290, 4:260])  # 16-byte aligned columns, pitched rows
    _check("min", base[::3, 8:72], axis, dev=dev[::3, 8:72])          # row step folded into the pitch
    fort = np.asfortranarray(_data((130, 70), np.int64, 4))
    _check("add", fort, axis, dev=cuda.to_device(fort))
    with pytest.raises(ValueError, match="contiguous"):
        REDUCERS["add"].along_axis(dev[::2, ::2], axis)


def test_every_plan_shape_through_one_reused_scratch():
    # tall + narrow (many row chunks), wide (one chunk), few very long rows (split rows),
    # many short rows, back to tall: the same scratch buffer serves all of them in turn
    for k, shape in enumerate([(1 << 16, 8), (64, 1 << 15), (4, 1 << 20), (1 << 17, 3), (1 << 15, 40),
                               (3, (1 << 20) + 16), (1 << 14, 100)]):
        host = _data(shape, np.int32, 300 + k)
        for axis in (0, 1):
            _check("add", host, axis)
            _check("xor", host, axis)
        f = _data(shape, np.float64, 400 + k)
        for axis in (0, 1):
            _check("add", f, axis)


def test_results_are_reproducible_and_res_is_used():
    host = _data((20000, 300), np.float32, 5)
    dev = cuda.to_device(host)
    for axis in (0, 1):
        a = REDUCERS["add"].along_axis(dev, axis).copy_to_host()
        b = REDUCERS["add"].along_axis(dev, axis).copy_to_host()
        assert a.tobytes() == b.tobytes()
        res = cuda.device_array(host.shape[1 - axis], dtype=np.float32)
        assert REDUCERS["add"].along_axis(dev, axis, res=res) is res
        assert res.copy_to_host().tobytes() == a.tobytes()


@pytest.mark.parametrize("shape", [(5, 6, 7), (3, 1, 9), (2, 3, 4, 5), (40, 33, 17), (1, 50, 64), (64, 50, 1)])
def test_one_axis_of_an_nd_array(shape):
    host = _data(shape, np.int32, 11)
    dev = cuda.to_device(host)
    for axis in range(-1, len(shape)):
        got = REDUCERS["add"].along_axis(dev, axis, init=3).copy_to_host()
        with np.errstate(over="ignore"):
            want = np.add.reduce(host, axis=axis, dtype=np.int32) + np.int32(3)
        assert got.shape == want.shape and got.tobytes() == want.tobytes()
    f = _data(shape, np.float64, 12)
    got = REDUCERS["max"].along_axis(cuda.to_device(f), 1, init=-np.inf).copy_to_host()
    assert got.tobytes() == f.max(axis=1).tobytes()
    out = cuda.device_array(shape[:1] + shape[2:], dtype=np.int32)
    assert REDUCERS["xor"].along_axis(dev, 1, res=out) is out
    assert out.copy_to_host().tobytes() == np.bitwise_xor.reduce(host, axis=1).tobytes()
    with pytest.raises(ValueError, match="out of bounds"):
        REDUCERS["add"].along_axis(dev, len(shape))
    with pytest.raises(ValueError, match="C-contiguous"):
        REDUCERS["add"].along_axis(cuda.to_device(np.zeros((4, 6, 8), dtype=np.int32))[:, ::2], 0)


def test_argument_errors():
    r = REDUCERS["add"]
    with pytest.raises(TypeError, match="only support 2D array"):
        r.along_axis(np.zeros(4, dtype=np.int32), 0)
    with pytest.raises(ValueError, match="out of bounds"):
        r.along_axis(np.zeros((4, 4), dtype=np.int32), 2)
    with pytest.raises(TypeError, match="incompatible dtype"):
        r.along_axis(np.zeros((4, 4), dtype=np.int32), 0, res=cuda.device_array(4, dtype=np.int64))
    with pytest.raises(ValueError, match="incompatible shape"):
        r.along_axis(np.zeros((4, 6), dtype=np.int32), 0, res=cuda.device_array(4, dtype=np.int32))
    with pytest.raises(NotImplementedError):
        cuda.Reduce(lambda a, b: (a + b) % 7).along_axis(np.zeros((4, 4), dtype=np.int32), 0)
    with pytest.raises((NotImplementedError, TypeError, cuda._lib.B2KError)):
        REDUCERS["and"].along_axis(np.zeros((4, 4), dtype=np.float32), 0)


@pytest.mark.parametrize("shape,dtype", [((6, 5000, 130), np.int32), ((300, 700, 48), np.uint8),
                                         ((5000, 37, 24), np.float64), ((3, 20011, 1000), np.int16),
                                         ((70000, 3, 8), np.int32)])
def test_middle_axis_of_a_batch_is_one_launch(shape, dtype):
    """outer x length x inner with outer, inner > 1: every slab is reduced along its rows
    by ONE launch over the batch of slabs (many tiles, rows cut into chunks, packed small
    items, more slabs than one launch's 65535)."""
    from numba_cuda_b200 import _lib
    host = _data(shape, dtype, 13)
    dev = cuda.to_device(host)
    before = _lib.launch_count()
    got = REDUCERS["add"].along_axis(dev, 1, init=2)
    launches = _lib.launch_count() - before
    assert launches == -(-shape[0] // 65535)
    with np.errstate(over="ignore"):
        want = np.add.reduce(host, axis=1, dtype=dtype) + np.dtype(dtype).type(2)
    if np.dtype(dtype).kind == "f":
        scale = np.abs(host).sum(axis=1)                      # sums of mixed signs cancel
        assert (np.abs(got.copy_to_host() - want) <= 1e-12 * scale).all()
    else:
        assert got.copy_to_host().tobytes() == want.tobytes()
    got = REDUCERS["max"].along_axis(dev, 1, init=host.min()).copy_to_host()
    assert got.tobytes() == host.max(axis=1).tobytes()
