"""Host-side logic of the drop-in: functor classification, indexing math,
shard bounds, identities.  No GPU."""
import os

import numpy as np
import pytest

from numba_cuda_b200 import _lib, casts, sharded
from numba_cuda_b200.devicearray import (_basic_index, _c_strides, _extent_bytes, _f_strides,
                                         _is_c_contig, _is_f_contig, stream_ptr)
from numba_cuda_b200.kernels.reduction import Reduce, classify_functor


@pytest.mark.parametrize("fn,code", [
    (lambda a, b: a + b, _lib.ADD), (lambda a, b: b + a, _lib.ADD), (lambda a, b: a * b, _lib.MUL),
    (lambda a, b: max(a, b), _lib.MAX), (lambda a, b: min(a, b), _lib.MIN),
    (lambda a, b: a if a > b else b, _lib.MAX), (lambda a, b: a if a < b else b, _lib.MIN)])
@pytest.mark.parametrize("dtype", [np.int8, np.int32, np.uint64, np.float32, np.float64])
def test_classify_arithmetic(fn, code, dtype):
    assert classify_functor(fn, dtype) == code


@pytest.mark.parametrize("fn,code", [(lambda a, b: a & b, _lib.AND), (lambda a, b: a | b, _lib.OR),
                                     (lambda a, b: a ^ b, _lib.XOR)])
def test_classify_bitwise(fn, code):
    assert classify_functor(fn, np.int32) == code
    assert classify_functor(fn, np.uint8) == code
    with pytest.raises(NotImplementedError):
        classify_functor(fn, np.float32)


def test_classify_rejects_what_it_cannot_run():
    for fn in (lambda a, b: a - b, lambda a, b: a + 2 * b, lambda a, b: a > b, lambda a, b: a / (b + 1e9),
               lambda a, b: a + b if a < 40 else a):
        with pytest.raises(NotImplementedError):
            classify_functor(fn, np.float64)
    with pytest.raises(NotImplementedError):
        classify_functor(lambda a, b: a + b, np.complex128)


def test_functors_with_constants_take_the_traced_path():
    # agrees with a+b on every probe sample, but is not a+b
    def capped(a, b):
        s = a + b
        if s > 100000:
            return 100000
        return s
    assert classify_functor(capped, np.int32) == _lib.ADD          # what the probe alone would say
    op = Reduce(capped)._compile(np.dtype(np.int32))
    assert isinstance(op, str) and "100000" in op
    assert Reduce(lambda a, b: a + b)._compile(np.dtype(np.int32)) == _lib.ADD
    assert Reduce(lambda a, b: max(a, b))._compile(np.dtype(np.float64)) == _lib.MAX
    assert isinstance(Reduce(lambda a, b: (a + b) % 7)._compile(np.dtype(np.int64)), str)
    import math
    with pytest.raises(NotImplementedError):
        Reduce(lambda a, b: math.sqrt(a) + b)._compile(np.dtype(np.float64))


def test_tracer_follows_branches_and_numba_typing():
    from numba_cuda_b200.kernels._trace import trace_functor
    assert trace_functor(lambda a, b: a + b) == "(a + b)"
    assert trace_functor(lambda a, b: max(a, b)) == "((b > a) ? b : a)"
    assert trace_functor(lambda a, b: a // b) == "b2k_floordiv(a, b)"
    assert trace_functor(lambda a, b: a * 1.5 + b) == "((a * 1.5) + b)"
    assert trace_functor(lambda a, b: 3) == "B2K_ILIT(3LL)"

    def three_way(a, b):
        if a > b:
            return a - b
        elif a == b:
            return 0
        return b - a
    assert trace_functor(three_way) == "((a > b) ? (a - b) : ((a == b) ? B2K_ILIT(0LL) : (b - a)))"
    with pytest.raises(NotImplementedError):
        trace_functor(lambda a, b: [a, b][a])


def test_reduce_argument_checks_come_first():
    # reduction.py:217-228: ndim check, then empty -> init, all before any device work
    r = Reduce(lambda a, b: a + b)
    with pytest.raises(TypeError, match="only support 1D array"):
        r(np.zeros((2, 2)))
    assert r(np.zeros(0, dtype=np.float64)) == 0.0
    got = r(np.zeros(0, dtype=np.int32), init=7)
    assert got == 7 and got.dtype == np.int32
    assert r(np.arange(10.0), size=0, init=3) == 3.0


def test_basic_index():
    shape, strides = (10, 12), (96, 8)
    assert _basic_index(shape, strides, (slice(None, None, 2), slice(None, None, 2))) == ((5, 6), (192, 16), 0)
    assert _basic_index(shape, strides, 3) == ((12,), (8,), 288)
    assert _basic_index(shape, strides, (3, 4)) == ((), (), 288 + 32)
    assert _basic_index(shape, strides, (-1, slice(2, 5))) == ((3,), (8,), 9 * 96 + 16)
    assert _basic_index(shape, strides, (Ellipsis, 1)) == ((10,), (96,), 8)
    assert _basic_index((7,), (4,), slice(5, 2)) == ((0,), (4,), 0)
    with pytest.raises(IndexError):
        _basic_index(shape, strides, (10, 0))
    with pytest.raises(IndexError):
        _basic_index(shape, strides, (0, 0, 0))


def test_layout_helpers():
    assert _c_strides((3, 4), 8) == (32, 8) and _f_strides((3, 4), 8) == (8, 24)
    assert _is_c_contig((3, 4), (32, 8), 8) and not _is_c_contig((3, 4), (64, 8), 8)
    assert _is_f_contig((3, 4), (8, 24), 8) and _is_c_contig((1, 4), (999, 8), 8)
    assert _extent_bytes((5, 6), (192, 16), 8) == 4 * 192 + 5 * 16 + 8
    assert _extent_bytes((0, 6), (192, 16), 8) == 0
    assert stream_ptr(0) == 0 and stream_ptr(None) == 0 and stream_ptr(0x1234) == 0x1234


def test_shard_bounds_partition():
    for n in (0, 1, 7, 1 << 20, (1 << 20) + 13):
        for world in (1, 2, 4, 8):
            for align in (1, 16):
                pieces = [sharded.shard_bounds(n, world, r, align) for r in range(world)]
                assert pieces[0][0] == 0 and pieces[-1][1] == n
                for (lo, hi), (lo2, _) in zip(pieces, pieces[1:]):
                    assert hi == lo2 and lo % align == 0 and lo <= hi
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 2, 2)


def test_identities_and_host_fold():
    for dt in (np.int8, np.uint16, np.int32, np.uint64, np.float32, np.float64):
        x = (np.random.default_rng(3).integers(0, 100, size=17)).astype(dt)
        ops = [_lib.ADD, _lib.MUL, _lib.MAX, _lib.MIN] + ([] if np.dtype(dt).kind == "f" else [_lib.AND, _lib.OR, _lib.XOR])
        for op in ops:
            ident = sharded.op_identity(op, dt)
            assert ident.dtype == np.dtype(dt)
            assert sharded.host_fold(op, x[:1], ident) == x[0]
    x = np.array([200, 100, 7], dtype=np.uint8)
    assert sharded.host_fold(_lib.ADD, x, np.uint8(0)) == np.uint8((200 + 100 + 7) % 256)
    assert sharded.host_fold(_lib.MAX, np.array([-5, -9], dtype=np.int32), np.int32(0)) == 0


def test_format_names():
    assert casts._format_code("e4m3") == _lib.FMT_E4M3 and casts._format_code("bfloat16") == _lib.FMT_BF16
    assert casts._format_code(_lib.FMT_F32) == _lib.FMT_F32
    assert casts.saturation_t.SATFINITE == 1 and casts.fp8_interpretation_t.E5M2 == 1
    with pytest.raises(ValueError):
        casts._format_code("fp4")


def test_array_like_strides_follow_numpy_zeros_like():
    # numba/cuda/tests/cudapy/test_array.py:100-263 compares device_array_like with
    # np.zeros_like on contiguous arrays and on views; the rule itself needs no GPU
    from numba_cuda_b200.api import strides_like
    rng = np.random.default_rng(0)
    checked = 0
    for _ in range(2000):
        nd = int(rng.integers(1, 5))
        shape = tuple(int(x) for x in rng.integers(2, 7, size=nd))
        base = np.zeros(shape, dtype=rng.choice([np.float32, np.float64, np.int8]), order=rng.choice(["C", "F"]))
        view = base[tuple(slice(None, None, int(rng.choice([1, 1, 2, 3]))) for _ in range(nd))]
        if rng.random() < 0.3:
            view = view.T
        if min(view.shape) < 2:
            continue
        assert strides_like(view.shape, view.strides, view.dtype.itemsize) == np.zeros_like(view).strides
        checked += 1
    assert checked > 1000
    for shape, order in (((10,), "C"), ((10, 12), "C"), ((10, 12, 14), "C"), ((10,), "F"), ((10, 12), "F"),
                         ((10, 12, 14), "F")):
        a = np.zeros(shape, order=order)
        assert strides_like(a.shape, a.strides, 8) == a.strides
        assert strides_like(a.T.shape, a.T.strides, 8) == a.T.strides
    # a signed sort, as the reference does: a reversed axis ranks first
    assert strides_like((3, 4), (-32, 8), 8) == (8, 24)


def test_basic_indexing_matches_numpy_views():
    # shape, strides and byte offset of every view numba's dummy array would give
    # (numba/cuda/tests/nocuda/test_dummyarray.py compares against NumPy the same way)
    from numba_cuda_b200.devicearray import _basic_index
    rng = np.random.default_rng(1)

    def one_slice(dim):
        def bound():
            return None if rng.random() < 0.3 else int(rng.integers(-dim - 2, dim + 3))
        step = None if rng.random() < 0.4 else int(rng.choice([1, 2, 3, -1, -2, -3]))
        return slice(bound(), bound(), step)

    def one_item(dim):
        return int(rng.integers(-dim, dim)) if rng.random() < 0.4 else one_slice(dim)

    views = 0
    for _ in range(4000):
        nd = int(rng.integers(1, 5))
        shape = tuple(int(x) for x in rng.integers(1, 6, size=nd))
        base = np.zeros(shape, dtype=np.int32)
        head = [one_item(shape[d]) for d in range(int(rng.integers(0, nd + 1)))]
        key = head
        if rng.random() < 0.3 and len(head) < nd:
            tail_len = int(rng.integers(0, nd - len(head) + 1))
            key = head + [Ellipsis] + [one_item(shape[nd - tail_len + j]) for j in range(tail_len)]
        key = tuple(key)
        want = base[key]
        got_shape, got_strides, got_offset = _basic_index(base.shape, base.strides, key)
        assert got_shape == want.shape
        if not isinstance(want, np.ndarray) or want.size == 0:
            continue
        assert all(a == b for a, b, n in zip(got_strides, want.strides, got_shape) if n > 1)
        assert got_offset == want.__array_interface__["data"][0] - base.__array_interface__["data"][0]
        views += 1
    assert views > 2000
    with pytest.raises(IndexError):
        _basic_index((3, 4), (16, 4), (0, 4))
    with pytest.raises(IndexError):
        _basic_index((3, 4), (16, 4), (0, 0, 0))
    with pytest.raises(IndexError):
        _basic_index((3, 4), (16, 4), (Ellipsis, Ellipsis))


def test_table_ops_are_recognised_in_every_usual_spelling():
    import operator
    spellings = {
        _lib.ADD: [lambda a, b: a + b, lambda a, b: b + a, operator.add],
        _lib.MUL: [lambda a, b: a * b, operator.mul],
        _lib.MAX: [lambda a, b: max(a, b), max, lambda a, b: a if a > b else b, lambda a, b: b if a < b else a,
                   lambda a, b: a if a >= b else b],
        _lib.MIN: [lambda a, b: min(a, b), min, lambda a, b: a if a < b else b, lambda a, b: b if b <= a else a],
        _lib.AND: [lambda a, b: a & b, operator.and_],
        _lib.OR: [lambda a, b: a | b],
        _lib.XOR: [lambda a, b: a ^ b, operator.xor],
    }
    for code, fns in spellings.items():
        for fn in fns:
            for dt in (np.int8, np.uint16, np.int32, np.uint64) + (() if code >= _lib.AND else (np.float32, np.float64)):
                assert Reduce(fn)._compile(np.dtype(dt)) == code, (code, dt)


def test_a_look_alike_that_cannot_be_traced_is_refused():
    LIMIT = 10 ** 9

    def looks_like_add(a, b):
        return float(min(a + b, LIMIT))       # equals a+b on every probe sample

    assert classify_functor(lambda a, b: min(a + b, LIMIT), np.float64) == _lib.ADD
    with pytest.raises(NotImplementedError):
        Reduce(looks_like_add)._compile(np.dtype(np.float64))
    # the traceable form of the same function runs as what it is
    op = Reduce(lambda a, b: min(a + b, LIMIT))._compile(np.dtype(np.int64))
    assert isinstance(op, str) and "1000000000" in op


def test_unsigned_items_widen_to_uint64_and_mix_as_int64():
    from numba_cuda_b200.kernels._trace import trace_functor
    # uint - uint stays unsigned (wraps), and is compared with the signed literal as a number
    assert trace_functor(lambda a, b: a if a - b > 0 else b, np.uint32) == \
        "(b2k_lt(B2K_ILIT(0LL), (a - b)) ? a : b)"
    # signed items: plain comparison
    assert trace_functor(lambda a, b: a if a - b > 0 else b, np.int32) == "(((a - b) > B2K_ILIT(0LL)) ? a : b)"
    # unsigned with a signed constant: the operation is done in int64
    assert trace_functor(lambda a, b: (a + b) % 7, np.uint8) == "b2k_mod(((long long)(a + b)), ((long long)B2K_ILIT(7LL)))"
    assert trace_functor(lambda a, b: -a + b, np.uint16) == "(((long long)(-(long long)a)) + ((long long)b))"
    # floats are untouched by the integer rule
    assert trace_functor(lambda a, b: a + b * 2, np.float32) == "(a + (b * B2K_ILIT(2LL)))"


def test_stats_and_nvtx_switch_need_no_device():
    """``cuda.stats()`` reads host-side counters only; with B2K_NVTX=1 an entry point that
    has no work to launch still returns 0 (the range opens and closes around nothing)."""
    import subprocess
    import sys
    import numba_cuda_b200 as cuda
    s = cuda.stats()
    assert set(s) == {"kernel_launches", "nvtx_ranges", "library"} and s["kernel_launches"] >= 0
    code = ("from numba_cuda_b200 import _lib; L = _lib.lib(); "
            "import numba_cuda_b200 as cuda; "
            "assert L.b2k_cast(0, 1, 1, None, None, 0, None) == 0; "
            "assert L.b2k_transpose2d(None, None, 0, 4, 16, 4, 0, 4, 4, None) == 0; "
            "assert cuda.stats()['nvtx_ranges'] is True; print('ok')")
    env = dict(os.environ, B2K_NVTX="1")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stderr[-500:]
