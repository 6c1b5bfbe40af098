"""cuda.reduce with functors outside the precompiled op table: the function is
traced to a C++ expression and compiled into the kernel at run time.  Checked
against a sequential fold of the same Python function (what the reference's
simulator does, numba/cuda/simulator/reduction.py:7-16); the functors are
associative and commutative, as cuda.reduce requires."""
import functools

import numpy as np
import pytest

import numba_cuda_b200 as cuda
from numba_cuda_b200.kernels._trace import trace_functor

pytestmark = pytest.mark.gpu

MOD = 1000003
mod_add = lambda a, b: (a + b) % MOD                      # noqa: E731
mod_mul = lambda a, b: (a * b) % 251                      # noqa: E731
abs_max = lambda a, b: max(abs(a), abs(b))                # noqa: E731
capped = lambda a, b: min(a + b, 100000)                  # noqa: E731
or_one = lambda a, b: a | b | 1                           # noqa: E731


def py_fold(fn, x, init):
    return functools.reduce(fn, [v.item() for v in x], init)


@pytest.mark.parametrize("n", [1, 2, 3, 15, 16, 17, 511, 4096, 100003, (1 << 20) + 3])
def test_modular_sum_int64(n):
    x = np.random.default_rng(n).integers(0, MOD, size=n, dtype=np.int64)
    got = cuda.reduce(mod_add)(x, init=5)
    assert got == (int(x.sum()) + 5) % MOD and got.dtype == np.int64


@pytest.mark.parametrize("dtype", [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64])
def test_every_integer_dtype(dtype):
    x = np.random.default_rng(1).integers(1, 100, size=50021).astype(dtype)
    fn = lambda a, b: (a * b) % 97                         # noqa: E731
    want = functools.reduce(lambda a, b: (a * b) % 97, [int(v) for v in x], 1)
    assert cuda.reduce(fn)(x, init=1) == want
    assert cuda.reduce(or_one)(x) == functools.reduce(or_one, [int(v) for v in x], 0)


def test_branching_functors():
    x = np.random.default_rng(3).integers(-10 ** 6, 10 ** 6, size=200001).astype(np.int32)
    assert cuda.reduce(abs_max)(x) == np.abs(x.astype(np.int64)).max()

    def manhattan_cap(a, b):
        s = a + b
        if s > 100000:
            return 100000
        return s
    y = np.random.default_rng(4).integers(0, 50, size=30011).astype(np.int32)
    assert cuda.reduce(manhattan_cap)(y) == min(int(y.sum()), 100000)
    assert cuda.reduce(capped)(y[:100]) == min(int(y[:100].sum()), 100000)


def test_float_functors():
    x = np.random.default_rng(5).standard_normal(100001)
    got = cuda.reduce(abs_max)(x)
    assert got == np.abs(x).max()
    # float32 meeting a Python float is evaluated in double and rounded on store, as numba types it
    f = np.random.default_rng(6).random(1000, dtype=np.float32)
    scaled_max = lambda a, b: max(a, b) * 1.0              # noqa: E731  (not a table op: result differs in type)
    assert cuda.reduce(lambda a, b: max(a * 1.0, b * 1.0))(f) == f.max()
    assert np.isfinite(cuda.reduce(scaled_max)(f))


def test_res_init_size_and_unaligned_views():
    x = np.random.default_rng(7).integers(0, MOD, size=5000, dtype=np.int64)
    d = cuda.to_device(x)
    res = cuda.device_array(1, dtype=np.int64)
    assert cuda.reduce(mod_add)(d, res=res, init=11) is None
    assert res.copy_to_host()[0] == (int(x.sum()) + 11) % MOD
    assert cuda.reduce(mod_add)(d, size=77) == int(x[:77].sum()) % MOD
    for off in (1, 2, 3):
        assert cuda.reduce(mod_add)(d[off:off + 1001]) == int(x[off:off + 1001].sum()) % MOD
    x8 = np.random.default_rng(8).integers(1, 100, size=3001).astype(np.uint8)
    d8 = cuda.to_device(x8)
    for off in range(0, 18):
        want = functools.reduce(mod_mul, [int(v) for v in x8[off:off + 1500]], 1)
        assert cuda.reduce(mod_mul)(d8[off:off + 1500], init=1) == want


def test_large_input_and_cache():
    n = 1 << 26
    x = np.random.default_rng(9).integers(0, MOD, size=n, dtype=np.int32)
    r = cuda.reduce(mod_add)
    d = cuda.to_device(x)
    a, b = r(d), r(d)
    assert a == b == int(x.astype(np.int64).sum()) % MOD


def test_trace_output_is_plain_cpp():
    assert trace_functor(mod_add) == "b2k_mod((a + b), B2K_ILIT(1000003LL))"
    assert trace_functor(lambda a, b: a if a < b else b) == "((a < b) ? a : b)"


def test_floor_remainder_on_the_32_bit_and_the_64_bit_instruction_paths():
    rng = np.random.default_rng(10)
    # operands within 32 bits, negative modulus: Python's sign rule, short path
    x = rng.integers(-10 ** 6, 10 ** 6, size=40001).astype(np.int32)
    neg_mod = lambda a, b: (a + b) % -1009                 # noqa: E731
    assert cuda.reduce(neg_mod)(x) == int(x.astype(np.int64).sum()) % -1009
    # the same remainder spelled with floor division
    via_div = lambda a, b: (a + b) - ((a + b) // 1009) * 1009   # noqa: E731
    assert cuda.reduce(via_div)(x) == int(x.astype(np.int64).sum()) % 1009
    # operands far outside 32 bits: the 64-bit path
    big = rng.integers(-2 ** 45, 2 ** 45, size=30011, dtype=np.int64)
    big_mod = lambda a, b: (a + b) % 1000000007            # noqa: E731
    assert cuda.reduce(big_mod)(big, init=3) == (sum(int(v) for v in big) + 3) % 1000000007
    # a divisor of -1 (the one case the 32-bit instructions cannot take)
    minus_one = lambda a, b: (a + b) % -1                  # noqa: E731
    assert cuda.reduce(minus_one)(x[:1000]) == 0
    u = rng.integers(0, 2 ** 32, size=20001, dtype=np.uint64).astype(np.uint32)
    assert cuda.reduce(lambda a, b: (a + b) % 65521)(u) == int(u.astype(np.uint64).sum()) % 65521


def test_unsigned_items_follow_the_integer_rule():
    """uint32 - uint32 is a uint64 that wraps, and comparing it with the signed 0 is done
    by value (numba's typing of the same function): a - b > 0 holds whenever a != b."""
    u = np.random.default_rng(11).integers(0, 2 ** 32, size=100003, dtype=np.uint64).astype(np.uint32)
    fn = lambda a, b: max(a, b) if a - b > 0 else min(a, b)      # noqa: E731
    assert cuda.reduce(fn)(u) == u.max()
    s = u.astype(np.int64).astype(np.int32)                      # signed items: a - b > 0 only when a > b
    assert cuda.reduce(lambda a, b: a if a - b > 0 else b)(s) == s.max()


def test_operands_that_leave_the_32_bit_range_in_small_items():
    """Items of up to 32 bits take the 32-bit division sequence only while the operands
    fit; a sum of two int32 may not.  The result must not depend on which sequence ran."""
    rng = np.random.default_rng(13)
    # half of all pair sums overflow int32
    wide = rng.integers(-2 ** 31, 2 ** 31, size=100003, dtype=np.int64).astype(np.int32)
    fn = lambda a, b: (a + b) % 1000003                    # noqa: E731
    assert cuda.reduce(fn)(wide, init=7) == (int(wide.astype(np.int64).sum()) + 7) % 1000003
    # a single overflowing pair in an otherwise small array, at every position of a vector
    for pos in range(0, 9):
        x = rng.integers(0, 1000, size=4099).astype(np.int32)
        x[2048 + pos] = 2 ** 31 - 1
        x[2049 + pos] = 2 ** 31 - 5
        assert cuda.reduce(fn)(x) == int(x.astype(np.int64).sum()) % 1000003, pos
    m8 = rng.integers(1, 100, size=5000).astype(np.uint8)
    assert cuda.reduce(lambda a, b: (a + b) % 101)(m8) == int(m8.astype(np.int64).sum()) % 101
    # a divisor of -1 that comes from the data (the case the 32-bit instructions cannot take)
    d = rng.integers(1, 50, size=2000).astype(np.int16)
    d[::7] = -1
    keep = lambda a, b: (a % b) * 0 + max(a, b)            # noqa: E731
    assert cuda.reduce(keep)(d, init=-5) == d.max()
