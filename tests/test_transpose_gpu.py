"""Device-array transpose on the GPU, bit-exact against NumPy ``.T``.  Restates
numba/cuda/tests/cudapy/test_transpose.py and the transpose cases of
tests/cudadrv/test_cuda_ndarray.py, then adds every item size, edge tiles and
the benchmark shapes."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib
from numba_cuda_b200.kernels.transpose import transpose

pytestmark = pytest.mark.gpu


def no_timeouts():
    c = ctypes.c_uint(123)
    assert _lib.lib().b2k_transpose_wait_timeouts(ctypes.byref(c)) == 0
    return c.value == 0


@pytest.mark.parametrize("rows,cols,dtype", [(5, 6, np.float64), (128, 128, np.complex128), (1025, 512, np.float64)])
def test_transpose(rows, cols, dtype):
    # test_transpose.py:16-31
    n = np.arange(rows * cols).reshape(rows, cols).astype(dtype)
    dx = cuda.to_device(n)
    dy = cuda.device_array((cols, rows), dtype=dtype)
    ret = transpose(dx, dy)
    assert ret is dy
    np.testing.assert_array_equal(dy.copy_to_host(), n.T)
    np.testing.assert_array_equal(transpose(dx).copy_to_host(), n.T)


@pytest.mark.parametrize("shape", [(1, 1), (1, 5), (5, 1), (3, 2), (2, 3), (33, 65), (64, 32)])
def test_transpose_record(shape):
    # test_transpose.py:43-58: a 28-byte record
    rec = np.dtype([("i", np.int32), ("j", np.float32, (3, 2))], align=True)
    arr = np.zeros(shape, dtype=rec)
    arr["i"] = np.arange(arr.size).reshape(shape)
    arr["j"] = np.random.default_rng(0).random(shape + (3, 2))
    out = cuda.to_device(arr).T.copy_to_host()
    assert out.shape == shape[::-1]
    np.testing.assert_array_equal(out, arr.T)


def test_transpose_bool():
    for rows, cols in ((1, 1), (5, 6), (128, 128), (1025, 512)):
        arr = np.random.default_rng(1).integers(0, 2, size=(rows, cols)).astype(np.bool_)
        np.testing.assert_array_equal(transpose(cuda.to_device(arr)).copy_to_host(), arr.T)


def test_transpose_view():
    # test_transpose.py:73-86
    a = np.arange(120, dtype=np.int64).reshape((10, 12))
    a_view_t = a[::2, ::2].T
    d_a = cuda.to_device(a)
    d_a_view_t = d_a[::2, ::2].T
    assert d_a_view_t.shape == (6, 5)
    assert d_a_view_t.strides == (40, 8)
    np.testing.assert_array_equal(d_a_view_t.copy_to_host(), a_view_t)


def test_transpose_api_errors_and_identities():
    # test_cuda_ndarray.py:143-244
    d3 = cuda.to_device(np.zeros((2, 3, 4)))
    with pytest.raises(NotImplementedError, match="non-2D"):
        d3.transpose()
    assert d3.transpose((0, 1, 2)) is d3
    d2 = cuda.to_device(np.arange(6.0).reshape(2, 3))
    assert d2.transpose((0, 1)) is d2
    with pytest.raises(ValueError, match="invalid axes"):
        d2.transpose((0, 2))
    np.testing.assert_array_equal(d2.transpose((1, 0)).copy_to_host(), np.arange(6.0).reshape(2, 3).T)
    np.testing.assert_array_equal(d2.T.copy_to_host(), np.arange(6.0).reshape(2, 3).T)
    with pytest.raises(ValueError):
        transpose(d2, cuda.device_array((2, 3), dtype=np.float64))
    with pytest.raises(TypeError):
        transpose(d2, cuda.device_array((3, 2), dtype=np.float32))


def test_host_input_is_copied_and_result_stays_on_device():
    a = np.random.default_rng(3).random((40, 24))
    out = transpose(a)
    assert isinstance(out, cuda.DeviceNDArray)
    np.testing.assert_array_equal(out.copy_to_host(), a.T)


SIZES = [1, 2, 3, 7, 8, 15, 16, 17, 31, 32, 33, 63, 64, 65, 70]


@pytest.mark.parametrize("itemsize", [1, 2, 4, 8, 16])
def test_small_shapes_every_itemsize(itemsize):
    dt = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64, 16: np.complex128}[itemsize]
    rng = np.random.default_rng(itemsize)
    for r in SIZES:
        for c in SIZES:
            a = rng.integers(0, 255, size=(r, c)).astype(dt)
            if itemsize == 16:
                a = a + 1j * rng.integers(0, 255, size=(r, c))
            got = transpose(cuda.to_device(a)).copy_to_host()
            assert got.tobytes() == np.ascontiguousarray(a.T).tobytes(), (r, c)


@pytest.mark.parametrize("rows,cols,dtype", [
    (512, 1024, np.float32), (1028, 516, np.float32), (64, 32, np.uint32), (1, 4096 * 8, np.uint32),
    (4096 * 8, 4, np.uint32), (300, 4104, np.uint16), (264, 136, np.uint16), (528, 1040, np.uint8),
    (1024, 2048, np.uint8), (514, 258, np.uint64), (520, 130, np.complex128), (1000, 2000, np.float32),
    (2049, 4100, np.float32), (1999, 3000, np.float64), (4097, 1032, np.uint16), (777, 1008, np.int8),
    (1024, 2048, np.uint16), (448, 320, np.uint16), (1088, 960, np.int16), (640, 1152, np.uint8),
    # single bytes on pitches that rule out the TMA path: the aligned-word byte tiles
    (777, 1001, np.uint8), (1001, 515, np.int8), (130, 4099, np.uint8), (4099, 130, np.bool_), (33, 35, np.uint8),
    (129, 131, np.uint8), (255, 257, np.int8), (2047, 2049, np.uint8)])
def test_tma_tile_path_shapes(rows, cols, dtype):
    rng = np.random.default_rng(rows * 7 + cols)
    a = rng.integers(0, 1 << 30, size=(rows, cols)).astype(dtype)
    before = _lib.launch_count()
    got = transpose(cuda.to_device(a)).copy_to_host()
    assert _lib.launch_count() == before + 1
    assert got.tobytes() == np.ascontiguousarray(a.T).tobytes()
    assert no_timeouts()


def test_tma_and_general_kernels_agree(monkeypatch):
    a = np.random.default_rng(0).integers(0, 1 << 30, size=(1500, 2052)).astype(np.uint32)
    d = cuda.to_device(a)
    fast = transpose(d).copy_to_host()
    # an input pitch that is not a multiple of 16 bytes forces the general kernel
    wide = np.zeros((1500, 2053), dtype=np.uint32)
    wide[:, :2052] = a
    slow = transpose(cuda.to_device(wide)[:, :2052]).copy_to_host()
    assert fast.tobytes() == slow.tobytes() == np.ascontiguousarray(a.T).tobytes()


def test_padded_pitches_through_c_abi():
    L = _lib.lib()
    rows, cols, pitch_in, pitch_out = 700, 900, 1024, 768   # items; both padded
    src = torch.randint(0, 2 ** 31 - 1, (rows, pitch_in), dtype=torch.int32, device="cuda")
    dst = torch.full((cols, pitch_out), -1, dtype=torch.int32, device="cuda")
    rc = L.b2k_transpose2d(src.data_ptr(), dst.data_ptr(), rows, cols, pitch_in * 4, 4, pitch_out * 4, 4, 4,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.b2k_last_error()
    assert torch.equal(dst[:, :rows], src[:, :cols].t())
    assert bool((dst[:, rows:] == -1).all())          # padding untouched
    assert no_timeouts()


def test_transposed_twice_is_identity_large():
    a = torch.randn(8192, 4096 + 64, device="cuda")
    d = cuda.as_cuda_array(a)
    back = transpose(transpose(d))
    assert torch.equal(torch.as_tensor(back, device="cuda"), a)


