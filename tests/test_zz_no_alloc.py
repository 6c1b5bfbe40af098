"""``b2k_reduce_noalloc``: the reduction for callers that may not allocate device
memory (their memory belongs to an external pool, or they are plain C callers
with only an input and an output buffer).  Its scratch is an array built into
the library, so this test checks, through the C ABI, that it gives exactly what
``b2k_reduce`` gives with caller scratch -- twice in a row, because the built-in
array is shared by all calls and keeps the previous call's contents.

Collected last on purpose: a run that stops at the first failure has already
run every other test by the time it gets here.
"""
import numpy as np
import pytest

from numba_cuda_b200 import _lib


def test_oversize_is_refused_before_any_device_work():
    L = _lib.lib()
    limit = L.b2k_reduce_noalloc_max_elements()
    assert limit == 1 << 32
    init = np.zeros(1, dtype=np.int32)
    rc = L.b2k_reduce_noalloc(_lib.ADD, _lib.I32, 4096, limit + 1, init.ctypes.data, 8192, None)
    assert rc == _lib.ERR_TOO_LARGE
    assert b"exceed the limit" in L.b2k_last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)


@pytest.mark.gpu
def test_matches_caller_scratch_entry_point_twice_in_a_row():
    import torch
    L = _lib.lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(7)
    cases = [
        (_lib.MAX, _lib.I32, torch.int32, 1 << 24, -2 ** 31),
        (_lib.ADD, _lib.F64, torch.float64, (1 << 22) + 5, 0.0),
        (_lib.ADD, _lib.F32, torch.float32, 1000003, 3.0),
        (_lib.MIN, _lib.I64, torch.int64, 77, 2 ** 62),
        (_lib.XOR, _lib.U8, torch.uint8, 123457, 0),
        (_lib.ADD, _lib.I32, torch.int32, 0, 9),
    ]
    for op, code, tdt, n, init_value in cases:
        if tdt.is_floating_point:
            x = torch.rand(max(n, 1), dtype=tdt, device="cuda", generator=g)[:n]
        else:
            info = torch.iinfo(tdt)
            x = torch.randint(info.min, info.max, (max(n, 1),), dtype=tdt, device="cuda", generator=g)[:n]
        ndt = np.dtype(str(tdt).replace("torch.", ""))
        init = np.array([init_value], dtype=ndt)
        want = torch.zeros(1, dtype=tdt, device="cuda")
        rc = L.b2k_reduce(op, code, x.data_ptr(), n, init.ctypes.data, want.data_ptr(),
                          scratch.data_ptr(), scratch.numel(), stream)
        assert rc == 0, L.b2k_last_error()
        expected = want.cpu().numpy().tobytes()
        for attempt in range(2):       # the second call meets the first call's leftovers
            got = torch.full((1,), 1, dtype=tdt, device="cuda")
            rc = L.b2k_reduce_noalloc(op, code, x.data_ptr(), n, init.ctypes.data, got.data_ptr(), stream)
            assert rc == 0, L.b2k_last_error()
            # same kernel, same grid, same fold order: the tolerance is zero, floats included
            assert got.cpu().numpy().tobytes() == expected, (op, code, n, attempt)
    # different inputs back to back through the shared array
    a = torch.arange(1, 100001, dtype=torch.int64, device="cuda")
    b = torch.arange(1, 11, dtype=torch.int64, device="cuda")
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    zero = np.zeros(1, dtype=np.int64)
    assert L.b2k_reduce_noalloc(_lib.ADD, _lib.I64, a.data_ptr(), a.numel(), zero.ctypes.data, out.data_ptr(), stream) == 0
    assert L.b2k_reduce_noalloc(_lib.ADD, _lib.I64, b.data_ptr(), b.numel(), zero.ctypes.data, out.data_ptr() + 8, stream) == 0
    assert out.tolist() == [100000 * 100001 // 2, 55]
