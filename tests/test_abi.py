"""The C-ABI library loads and exports every symbol include/b2k.h declares, and
rejects bad arguments on the host before any CUDA call.  No GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from numba_cuda_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b2k.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2k_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_bound():
    names = declared_symbols()
    assert "b2k_reduce" in names and "b2k_cast" in names and len(names) >= 10
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    for name in declared_symbols():
        assert getattr(L, name) is not None
    assert L.b2k_version() >= 100
    assert L.b2k_reduce_scratch_bytes() >= 256 + 8 * 1024
    assert L.b2k_xoroshiro128p_tables_bytes() == 8 * 256 * 16


def test_argument_errors_are_reported_on_host():
    L = _lib.lib()
    init = np.zeros(1, dtype=np.float64)
    # unknown dtype / op, negative length, null pointers: all before any launch
    assert L.b2k_reduce(_lib.ADD, 99, None, 0, init.ctypes.data, 8, 256, 1 << 20, None) == _lib.ERR_INVALID_ARG
    assert b"dtype" in L.b2k_last_error()
    assert L.b2k_reduce(42, _lib.F64, None, 0, init.ctypes.data, 8, 256, 1 << 20, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce(_lib.ADD, _lib.F64, None, -1, init.ctypes.data, 8, 256, 1 << 20, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce(_lib.ADD, _lib.F64, None, 4, init.ctypes.data, 8, 256, 1 << 20, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce(_lib.ADD, _lib.F64, 1024, 4, init.ctypes.data, 8, None, 0, None) == _lib.ERR_SCRATCH
    assert L.b2k_reduce(_lib.ADD, _lib.F64, 1028, 4, init.ctypes.data, 8, 256, 1 << 20, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_reduce(_lib.AND, _lib.F32, 1024, 4, init.ctypes.data, 8, 256, 1 << 20, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast(_lib.FMT_BF16, _lib.FMT_E4M3, 1, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast(_lib.FMT_F32, _lib.FMT_BF16, 1, 1024, 2048, -5, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_cast(_lib.FMT_F32, _lib.FMT_BF16, 1, None, 2048, 16, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_cast(_lib.FMT_F32, _lib.FMT_BF16, 1, 1026, 2048, 16, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_transpose2d(None, None, 4, 4, 16, 4, 16, 4, 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_transpose2d(1024, 2048, -1, 4, 16, 4, 16, 4, 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_xoroshiro128p_init(1024, 8, 1, 0, None, 0, None) == _lib.ERR_SCRATCH
    assert L.b2k_xoroshiro128p_init(1028, 8, 1, 0, 4096, 1 << 20, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_xoroshiro128p_fill(1024, 8, 7, 2048, 4, 0, None, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_xoroshiro128p_fill(1024, -8, 0, 2048, 4, 0, None, 0, None) == _lib.ERR_INVALID_ARG
    # strided assignment and axis-wise reduce
    arr2 = ctypes.c_int64 * 2
    assert L.b2k_assign(1024, 2048, 40, None, None, None, 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_assign(1024, 2048, 2, arr2(4, 4), arr2(16, 4), arr2(16, 4), 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_assign(1024, 2048, 2, arr2(4, -4), arr2(16, 4), arr2(16, 4), 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_assign(1024, 2048, 2, arr2(4, 4), arr2(16, 0), arr2(16, 4), 4, None) == _lib.ERR_INVALID_ARG
    assert b"destination stride 0" in L.b2k_last_error()
    assert L.b2k_assign(None, 2048, 2, arr2(4, 4), arr2(16, 4), arr2(16, 4), 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_assign(None, None, 2, arr2(4, 0), arr2(16, 4), arr2(16, 4), 4, None) == 0          # empty
    four = np.float32(1.5).tobytes()
    assert L.b2k_fill(1024, 2, arr2(4, 4), arr2(16, 4), None, 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_fill(1024, 2, arr2(4, 4), arr2(16, 4), four, 17, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_fill(None, 2, arr2(4, 4), arr2(16, 4), four, 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_fill(1024, 2, arr2(4, 4), arr2(0, 4), four, 4, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_fill(None, 2, arr2(0, 4), arr2(16, 4), four, 4, None) == 0                        # empty
    assert L.b2k_reduce_axis(_lib.ADD, 99, 1024, 4, 4, 16, 0, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_axis(_lib.ADD, _lib.F32, 1024, 4, 4, 16, 2, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_axis(_lib.ADD, _lib.F32, 1024, -4, 4, 16, 0, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_axis(_lib.ADD, _lib.F32, 1024, 4, 4, 8, 0, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_INVALID_ARG
    assert b"pitch" in L.b2k_last_error()
    assert L.b2k_reduce_axis(_lib.ADD, _lib.F32, 1026, 4, 4, 16, 0, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_reduce_axis(_lib.XOR, _lib.F64, 1024, 4, 4, 32, 1, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_reduce_axis(_lib.ADD, _lib.F32, 1024, 1 << 20, 8, 32, 0, init.ctypes.data, 2048, None, 0, None) == _lib.ERR_SCRATCH
    assert L.b2k_reduce_axis(_lib.ADD, _lib.F32, None, 0, 0, 0, 0, init.ctypes.data, None, None, 0, None) == 0   # no outputs
    assert L.b2k_reduce_axis_scratch_bytes(1 << 20, 8, _lib.F32, 0) > 16384
    assert L.b2k_reduce_axis_scratch_bytes(64, 64, _lib.F32, 1) == 0
    assert L.b2k_reduce_axis_scratch_bytes(64, 64, 99, 1) == 0
    # a batch of matrices reduced along their rows, the flags of b2k_reduce_ex, the new cast pairs
    assert L.b2k_reduce_cols_batched(_lib.ADD, _lib.F32, 1024, 70000, 4, 4, 16, 64, init.ctypes.data, 2048, None, 0,
                                     None) == _lib.ERR_TOO_LARGE
    assert L.b2k_reduce_cols_batched(_lib.ADD, _lib.F32, 1024, 3, 4, 4, 16, -64, init.ctypes.data, 2048, None, 0,
                                     None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_cols_batched(_lib.ADD, _lib.F32, 1024, 3, 4, 4, 16, 66, init.ctypes.data, 2048, None, 0,
                                     None) == _lib.ERR_ALIGNMENT
    assert L.b2k_reduce_cols_batched(_lib.ADD, _lib.F32, 1024, 4, 1 << 20, 8, 32, 1 << 25, init.ctypes.data, 2048,
                                     None, 0, None) == _lib.ERR_SCRATCH
    assert L.b2k_reduce_cols_batched(_lib.ADD, _lib.F32, None, 0, 4, 4, 16, 64, init.ctypes.data, None, None, 0,
                                     None) == 0                                                   # no matrices
    assert L.b2k_reduce_cols_batched_scratch_bytes(4, 1 << 20, 8, _lib.F32) > \
        L.b2k_reduce_axis_scratch_bytes(1 << 20, 8, _lib.F32, 0)
    assert L.b2k_reduce_ex(_lib.ADD, _lib.F64, 1024, 4, init.ctypes.data, 8, 256, 1 << 20, 2, None) == _lib.ERR_INVALID_ARG
    assert b"flag" in L.b2k_last_error()
    assert L.b2k_reduce(_lib.ADD, _lib.F64, 1024, 4, init.ctypes.data, 8, 256, 1000, None) == _lib.ERR_SCRATCH
    assert L.b2k_cast_ex(_lib.FMT_F64, _lib.FMT_E4M3, 1, _lib.ROUND_ZERO, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_F64, _lib.FMT_E4M3, 1, _lib.ROUND_NEAREST, 1028, 2048, 16, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_cast_ex(_lib.FMT_F64, _lib.FMT_E8M0, 1, _lib.ROUND_NEAREST, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_BF16, _lib.FMT_E5M2, 0, _lib.ROUND_NEAREST, None, None, 0, None) == 0
    # integer sides: the constructors saturate and round to nearest (E8M0: up); the operators truncate
    assert L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_E4M3, 0, _lib.ROUND_NEAREST, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_E8M0, 1, _lib.ROUND_ZERO, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_E5M2, _lib.FMT_U16, 1, _lib.ROUND_NEAREST, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_BF16, _lib.FMT_I8, 1, _lib.ROUND_POS_INF, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_U8, _lib.FMT_BF16, 1, _lib.ROUND_NEAREST, 1024, 2048, 16, None) == _lib.ERR_UNSUPPORTED
    assert L.b2k_cast_ex(_lib.FMT_I64, _lib.FMT_BF16, 1, _lib.ROUND_MIN_INF, 1028, 2048, 16, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_cast_ex(_lib.FMT_E8M0, _lib.FMT_U64, 1, _lib.ROUND_ZERO, 1024, 2052, 16, None) == _lib.ERR_ALIGNMENT
    assert L.b2k_cast_ex(_lib.FMT_I16, _lib.FMT_E5M2, 1, _lib.ROUND_NEAREST, None, None, 0, None) == 0
    # empty work is a no-op that needs no device
    assert L.b2k_cast(_lib.FMT_F32, _lib.FMT_BF16, 1, None, None, 0, None) == 0
    assert L.b2k_transpose2d(None, None, 0, 4, 16, 4, 0, 4, 4, None) == 0
    assert L.b2k_xoroshiro128p_init(None, 0, 1, 0, None, 0, None) == 0


def test_status_maps_to_python_exceptions():
    L = _lib.lib()
    with pytest.raises(NotImplementedError):
        _lib.check(L.b2k_cast(_lib.FMT_BF16, _lib.FMT_E4M3, 1, 1024, 2048, 16, None))
    with pytest.raises(ValueError):
        _lib.check(L.b2k_cast(_lib.FMT_F32, _lib.FMT_BF16, 1, 1024, 2048, -5, None))
    _lib.check(0)


def test_no_cpu_fallback_without_device():
    """Without a GPU the public API must raise, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import numba_cuda_b200 as cuda
    with pytest.raises(RuntimeError):
        cuda.to_device(np.arange(4.0))
    with pytest.raises(RuntimeError):
        cuda.reduce(lambda a, b: a + b)(np.arange(4.0))
    with pytest.raises(RuntimeError):
        cuda.random.create_xoroshiro128p_states(4, 1)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No library, no work: the binding raises instead of finding another way."""
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libb2k.so"))
    _lib.lib.cache_clear()
    try:
        with pytest.raises(ImportError, match="no CPU fallback"):
            _lib.lib()
    finally:
        monkeypatch.undo()
        _lib.lib.cache_clear()
        assert _lib.lib().b2k_version() >= 100


def test_package_never_touches_the_oracle():
    """The CPU oracle is test infrastructure: nothing under the package imports,
    loads or names it."""
    pkg = os.path.join(ROOT, "numba_cuda_b200")
    for dirpath, _, files in os.walk(pkg):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, name)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, name)
