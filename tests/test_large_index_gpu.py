"""Arrays with more than 2^31 / 2^32 items: every kernel family once, so that an
index that was computed in 32 bits somewhere shows up.  Results are checked on the
device with torch (moving these arrays to the host would dominate the test time);
the kernels themselves are checked against the CPU oracle at ordinary sizes in the
other test files."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import numba_cuda_b200 as cuda  # noqa: E402
from numba_cuda_b200 import _lib  # noqa: E402


def _need(gigabytes):
    free, _ = torch.cuda.mem_get_info()
    if free < gigabytes * (1 << 30):
        pytest.skip(f"needs {gigabytes} GiB of free device memory")


def _check(rc):
    assert rc == 0, _lib.lib().b2k_last_error()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_reduce_over_more_than_2_32_items():
    _need(8)
    L = _lib.lib()
    n = (1 << 32) + 7
    x = torch.ones(n, dtype=torch.int8, device="cuda")
    x[n - 3] = 100           # beyond item 2^32
    x[1 << 31] = -128
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    out = torch.zeros(1, dtype=torch.int8, device="cuda")
    init = np.zeros(1, dtype=np.int8)
    for op, want in ((_lib.MAX, 100), (_lib.MIN, -128),
                     (_lib.ADD, int(np.int64(n - 2 + 100 - 128).astype(np.int8)))):
        _check(L.b2k_reduce(op, _lib.I8, x.data_ptr(), n, init.ctypes.data, out.data_ptr(), scratch.data_ptr(),
                            scratch.numel(), _stream()))
        assert int(out.item()) == want, (op, int(out.item()), want)


def test_cast_over_more_than_2_31_items():
    _need(16)
    L = _lib.lib()
    n = (1 << 31) + 48
    x = torch.full((n,), 1.5, dtype=torch.float32, device="cuda")
    x[-5:] = torch.tensor([2.0, -3.0, 0.5, 448.0, 1e9], device="cuda")
    x[1 << 31] = 7.0
    codes = torch.empty(n, dtype=torch.uint8, device="cuda")
    _check(L.b2k_cast(_lib.FMT_F32, _lib.FMT_E4M3, 1, x.data_ptr(), codes.data_ptr(), n, _stream()))
    assert int((codes[:-5] != 0x3C).sum().item()) == 1 and int(codes[1 << 31].item()) == 0x4E   # 1.5 -> 0x3C, 7.0 -> 0x4E
    assert codes[-5:].tolist() == [0x40, 0xC4, 0x30, 0x7E, 0x7E]
    half = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    _check(L.b2k_cast(_lib.FMT_F32, _lib.FMT_BF16, 1, x.data_ptr(), half.data_ptr(), n, _stream()))
    assert torch.equal(half[-64:], x[-64:].to(torch.bfloat16)) and float(half[1 << 31]) == 7.0
    assert torch.equal(half[:1 << 20], x[:1 << 20].to(torch.bfloat16))


def test_assign_over_more_than_2_32_units():
    _need(16)
    L = _lib.lib()
    n = (1 << 32) + 1024
    src = torch.randint(0, 256, (2 * n,), dtype=torch.uint8, device="cuda")
    src[2 * (n - 1)] = 77
    dst = torch.zeros(n, dtype=torch.uint8, device="cuda")
    one = ctypes.c_int64 * 1
    # every second byte: nothing merges, 1-byte units, more than 2^32 of them
    _check(L.b2k_assign(dst.data_ptr(), src.data_ptr(), 1, one(n), one(1), one(2), 1, _stream()))
    assert int(dst[-1].item()) == 77
    for lo in (0, (1 << 31) - 512, (1 << 32) - 512, n - 1024):
        assert torch.equal(dst[lo:lo + 1024], src[2 * lo:2 * lo + 2048:2])
    # scalar fill of the same length: the widened 16-byte path
    _check(L.b2k_assign(dst.data_ptr(), src.data_ptr() + 2 * (n - 1), 1, one(n), one(1), one(0), 1, _stream()))
    assert int(dst.min().item()) == 77 and int(dst.max().item()) == 77


def test_transpose_and_permute_over_more_than_2_32_items():
    _need(12)
    L = _lib.lib()
    rows, cols = 65536 + 128, 65536
    a = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, device="cuda")
    b = torch.empty(cols, rows, dtype=torch.uint8, device="cuda")
    _check(L.b2k_transpose2d(a.data_ptr(), b.data_ptr(), rows, cols, cols, 1, rows, 1, 1, _stream()))
    for r0, c0 in ((0, 0), (rows - 256, cols - 256), (rows - 300, 17), (32768, 40000)):
        assert torch.equal(b[c0:c0 + 256, r0:r0 + 256], a[r0:r0 + 256, c0:c0 + 256].t())
    # the same problem through the strided-assignment entry point (stacked TMA path)
    b.zero_()
    two = ctypes.c_int64 * 2
    _check(L.b2k_assign(b.data_ptr(), a.data_ptr(), 2, two(cols, rows), two(rows, 1), two(1, cols), 1, _stream()))
    for r0, c0 in ((0, 0), (rows - 256, cols - 256), (50000, 123)):
        assert torch.equal(b[c0:c0 + 256, r0:r0 + 256], a[r0:r0 + 256, c0:c0 + 256].t())


def test_axis_reduce_over_more_than_2_32_items():
    _need(8)
    rows, cols = 65536 + 64, 65536
    m = torch.ones(rows, cols, dtype=torch.uint8, device="cuda")
    m[rows - 1, cols - 1] = 5
    m[40000, 3] = 9
    red = cuda.Reduce(lambda a, b: a + b)
    dev = cuda.as_cuda_array(m)
    col_sums = torch.as_tensor(red.along_axis(dev, 0), device="cuda")
    want = torch.full((cols,), rows % 256, dtype=torch.uint8, device="cuda")
    want[cols - 1] = (rows + 4) % 256
    want[3] = (rows + 8) % 256
    assert torch.equal(col_sums, want)
    row_sums = torch.as_tensor(red.along_axis(dev, 1), device="cuda")
    want = torch.full((rows,), cols % 256, dtype=torch.uint8, device="cuda")
    want[rows - 1] = (cols + 4) % 256
    want[40000] = (cols + 8) % 256
    assert torch.equal(row_sums, want)


def test_rng_fill_over_more_than_2_32_samples():
    _need(24)
    from numba_cuda_b200.random import create_xoroshiro128p_states, xoroshiro128p_fill
    n, count = 1 << 24, 260           # 4.36e9 float32 samples
    states = create_xoroshiro128p_states(n, seed=7)
    out = xoroshiro128p_fill(states, "uniform", count=count, dtype=np.float32)
    big = torch.as_tensor(out, device="cuda")
    # the last generators again, created by their subsequence numbers: same rows
    for lo in (n - 64, (1 << 23) + 5, 0):
        few = create_xoroshiro128p_states(64, seed=7, subsequence_start=lo)
        small = torch.as_tensor(xoroshiro128p_fill(few, "uniform", count=count, dtype=np.float32), device="cuda")
        assert torch.equal(big[lo:lo + 64], small)
