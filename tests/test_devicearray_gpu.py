"""The device-array shim either side of the library kernels: the behaviours of
numba-cuda's DeviceNDArray / host API that callers of reduce, transpose and the
RNG rely on (numba/cuda/tests/cudadrv/test_cuda_ndarray.py, test_cuda_array_slicing.py,
numba/cuda/tests/cudapy/test_cuda_array_interface.py in outline)."""
import numpy as np
import pytest
import torch

import numba_cuda_b200 as cuda

pytestmark = pytest.mark.gpu


def test_round_trip_and_attributes():
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    d = cuda.to_device(a)
    assert d.shape == (4, 6) and d.strides == (24, 4) and d.dtype == np.float32
    assert d.size == 24 and d.ndim == 2 and d.nbytes == 96 and len(d) == 4
    np.testing.assert_array_equal(d.copy_to_host(), a)
    out = np.zeros_like(a)
    assert d.copy_to_host(out) is out
    np.testing.assert_array_equal(out, a)
    f = np.asfortranarray(a)
    df = cuda.to_device(f)
    assert df.strides == f.strides and df.is_f_contiguous()
    np.testing.assert_array_equal(df.copy_to_host(), f)


def test_non_contiguous_host_array_is_rejected():
    a = np.arange(100).reshape(10, 10)[::2, ::2]
    with pytest.raises(ValueError, match="non-contiguous"):
        cuda.to_device(a)


def test_device_array_and_like():
    d = cuda.device_array((3, 5), dtype=np.int16)
    assert d.shape == (3, 5) and d.strides == (10, 2)
    f = cuda.device_array((3, 5), dtype=np.int16, order="F")
    assert f.strides == (2, 6)
    like = cuda.device_array_like(f)
    assert like.strides == f.strides and like.dtype == f.dtype
    like_c = cuda.device_array_like(np.zeros((2, 7), dtype=np.float64))
    assert like_c.shape == (2, 7) and like_c.strides == (56, 8)
    one = cuda.device_array(10)
    assert one.shape == (10,) and one.dtype == np.float64


def test_indexing_views_and_scalars():
    a = np.arange(120, dtype=np.int64).reshape(10, 12)
    d = cuda.to_device(a)
    assert d[3, 4] == a[3, 4] and isinstance(d[3, 4], np.int64)
    np.testing.assert_array_equal(d[2].copy_to_host(), a[2])
    np.testing.assert_array_equal(d[2:5].copy_to_host(), a[2:5])
    np.testing.assert_array_equal(d[::2, ::3].copy_to_host(), a[::2, ::3])
    np.testing.assert_array_equal(d[1:, 5].copy_to_host(), a[1:, 5])
    np.testing.assert_array_equal(d[..., -1].copy_to_host(), a[..., -1])
    assert d[::2, ::2].strides == a[::2, ::2].strides
    assert d[5:2].size == 0 and d[5:2].copy_to_host().shape == (0, 12)
    with pytest.raises(IndexError):
        d[10]
    with pytest.raises(IndexError):
        d[0, 0, 0]


def test_setitem_and_copy_to_device():
    a = np.zeros((4, 6), dtype=np.float32)
    d = cuda.to_device(a)
    d[1] = 7
    d[2, 3] = 9
    d[:, 0] = np.arange(4, dtype=np.float32)
    want = a.copy()
    want[1] = 7
    want[2, 3] = 9
    want[:, 0] = np.arange(4)
    np.testing.assert_array_equal(d.copy_to_host(), want)
    e = cuda.device_array((4, 6), dtype=np.float32)
    e.copy_to_device(d)
    np.testing.assert_array_equal(e.copy_to_host(), want)
    with pytest.raises(TypeError, match="incompatible dtype"):
        e.copy_to_device(np.zeros((4, 6), dtype=np.float64))
    with pytest.raises(ValueError, match="incompatible shape"):
        e.copy_to_device(np.zeros((4, 5), dtype=np.float32))


def test_reshape_ravel_view_split_squeeze():
    a = np.arange(24, dtype=np.int32)
    d = cuda.to_device(a)
    np.testing.assert_array_equal(d.reshape(4, 6).copy_to_host(), a.reshape(4, 6))
    np.testing.assert_array_equal(d.reshape((2, -1)).copy_to_host(), a.reshape(2, 12))
    np.testing.assert_array_equal(d.reshape(4, 6).ravel().copy_to_host(), a)
    np.testing.assert_array_equal(d.view(np.int16).copy_to_host(), a.view(np.int16))
    np.testing.assert_array_equal(d.view(np.float32).copy_to_host(), a.view(np.float32))
    parts = list(d.split(10))
    assert [p.size for p in parts] == [10, 10, 4]
    np.testing.assert_array_equal(parts[2].copy_to_host(), a[20:])
    s = cuda.to_device(np.zeros((1, 5, 1))).squeeze()
    assert s.shape == (5,)
    with pytest.raises(ValueError):
        d.reshape(5, 5)
    with pytest.raises(NotImplementedError):
        d.reshape(4, 6)[:, ::2].reshape(12)


def test_cuda_array_interface_both_ways():
    t = torch.arange(12, dtype=torch.float32, device="cuda").reshape(3, 4)
    d = cuda.as_cuda_array(t)
    assert d.shape == (3, 4) and d.dtype == np.float32
    np.testing.assert_array_equal(d.copy_to_host(), t.cpu().numpy())
    d[0, 0] = 5
    assert t[0, 0].item() == 5                                   # zero copy
    back = torch.as_tensor(cuda.to_device(np.arange(6, dtype=np.int32)), device="cuda")
    assert back.tolist() == [0, 1, 2, 3, 4, 5]
    iface = d[:, ::2].__cuda_array_interface__
    assert iface["strides"] == (16, 8) and iface["version"] == 3 and iface["shape"] == (3, 2)
    assert cuda.is_cuda_array(t) and not cuda.is_cuda_array(np.zeros(3))
    with pytest.raises(TypeError):
        cuda.as_cuda_array(np.zeros(3))


def test_structured_and_bfloat16_dtypes():
    rec = np.dtype([("i", np.int32), ("j", np.float32, (3, 2))], align=True)
    a = np.zeros(7, dtype=rec)
    a["i"] = np.arange(7)
    d = cuda.to_device(a)
    assert d.dtype == rec and d.copy_to_host().tobytes() == a.tobytes()
    bf = cuda.bf16.bfloat16_dtype()
    x = np.arange(8, dtype=np.float32).astype(bf)
    assert cuda.to_device(x).copy_to_host().tobytes() == x.tobytes()


def test_streams_and_pinned():
    s = cuda.stream()
    h = cuda.pinned_array(1000, dtype=np.float64)
    h[:] = np.arange(1000)
    d = cuda.to_device(h, stream=s)
    s.synchronize()
    np.testing.assert_array_equal(d.copy_to_host(stream=s), h)
    assert d.stream is s and d.bind(0).stream == 0
    with s.auto_synchronize():
        pass
    assert cuda.is_bfloat16_supported() and cuda.is_fp8_supported()


def test_device_array_like_of_views_and_transposes():
    # test_array.py:176-263
    for order in ("C", "F"):
        for shape, key in (((10,), (slice(None, None, 2),)), ((10, 12), (slice(None, None, 2), slice(None, None, 2)))):
            view = np.zeros(shape, order=order)[key]
            d_view = cuda.device_array(shape, order=order)[key]
            like = cuda.device_array_like(d_view)
            want = np.zeros_like(view)
            assert like.shape == want.shape and like.dtype == want.dtype and like.strides == want.strides
            assert like.flags["C_CONTIGUOUS"] == want.flags["C_CONTIGUOUS"]
            assert like.flags["F_CONTIGUOUS"] == want.flags["F_CONTIGUOUS"]
            pinned = cuda.pinned_array_like(d_view)
            assert pinned.shape == want.shape and pinned.strides == want.strides
    # the transpose of a device view is a new dense allocation (test_array.py:221-237)
    d_t = cuda.device_array((10, 12))[::2, ::2].T
    like = cuda.device_array_like(d_t)
    assert like.shape == d_t.shape and like.strides == (40, 8)
    assert like.flags["C_CONTIGUOUS"] and not like.flags["F_CONTIGUOUS"]


def test_events_time_a_library_call():
    start, end = cuda.event(), cuda.event()
    x = cuda.to_device(np.ones(1 << 22, dtype=np.float32))
    s = cuda.stream()
    start.record(s)
    total = cuda.reduce(lambda a, b: a + b)(x, stream=s)
    end.record(s)
    end.synchronize()
    assert total == np.float32(1 << 22) and end.query()
    ms = cuda.event_elapsed_time(start, end)
    assert 0.0 < ms < 1000.0 and ms == start.elapsed_time(end)
    end.wait(s)                                  # enqueue-only; must not raise
