"""Device-side broadcasting assignment and N-D axis permutation (b2k_assign)
against NumPy, which is what the reference's own array tests compare with
(numba/cuda/tests/cudadrv/test_cuda_ndarray.py and test_cuda_array_slicing.py:
``assert_array_equal`` after ``d_arr[key] = value``)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

import numba_cuda_b200 as cuda  # noqa: E402
from numba_cuda_b200 import _lib  # noqa: E402
from numba_cuda_b200.kernels.transpose import permute  # noqa: E402

REC = np.dtype([("i", np.int32), ("j", np.float32, (3, 2))], align=True)   # 28 bytes


def _filled(shape, dtype, seed=0):
    rng = np.random.default_rng(seed)
    dtype = np.dtype(dtype)
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    raw = rng.integers(0, 256, size=n * dtype.itemsize, dtype=np.uint8)
    return raw.view(dtype).reshape(shape).copy()


SETITEM_CASES = [
    # (shape, key, value shape or None for a scalar)
    ((10,), slice(None), None),
    ((10,), 3, None),
    ((10,), slice(2, 9, 3), (3,)),
    ((10,), slice(None, None, -1), (10,)),
    ((6, 7), (slice(None), 2), (6,)),
    ((6, 7), (1, slice(None)), (7,)),
    ((6, 7), (slice(1, 5), slice(None, None, 2)), (4, 4)),
    ((6, 7), (slice(1, 5), slice(None, None, 2)), (1, 4)),
    ((6, 7), (slice(1, 5), slice(None, None, 2)), (4, 1)),
    ((6, 7), (slice(1, 5), slice(None, None, 2)), (4,)),
    ((6, 7), (slice(None, None, -2), slice(None, None, -1)), (3, 7)),
    ((4, 5, 6), (slice(None), 2), (4, 6)),
    ((4, 5, 6), (Ellipsis, 0), (4, 5)),
    ((4, 5, 6), (slice(None), slice(None), slice(None)), (5, 6)),
    ((4, 5, 6), (2, 3, 4), None),
    ((3, 4, 5, 6, 2), (slice(None), slice(1, 3), Ellipsis, slice(None, None, 2), 1), (3, 2, 5, 3)),
    ((257, 130), (slice(None), slice(None)), (257, 130)),
    ((257, 130), (slice(3, 250, 5), slice(1, 129)), (1, 128)),
    # one row / plane repeated over a long slower axis (the read-once, store-many kernel)
    ((100, 40, 64), (slice(None), slice(None), slice(None)), (40, 64)),
    ((100, 40, 64), (slice(None), slice(None), slice(None)), (100, 1, 64)),
    ((100, 40, 64), (slice(1, 99), slice(None), slice(0, 60)), (1, 1, 60)),
    ((1000, 36), (slice(None), slice(None)), (36,)),
    ((1000, 36), (slice(None, None, -1), slice(2, 34)), (32,)),
]


@pytest.mark.parametrize("dtype", [np.uint8, np.int16, np.float32, np.float64, np.complex128, REC])
@pytest.mark.parametrize("shape,key,vshape", SETITEM_CASES)
def test_setitem_matches_numpy(dtype, shape, key, vshape):
    host = _filled(shape, dtype, 1)
    value = _filled(() if vshape is None else vshape, dtype, 2)
    if vshape is None:
        value = value[()]
    dev = cuda.to_device(host)
    dev[key] = value
    host[key] = value
    assert dev.copy_to_host().tobytes() == host.tobytes()


def test_setitem_from_device_arrays_and_views():
    host = _filled((64, 96), np.float32, 3)
    other = _filled((64, 96), np.float32, 4)
    dev, dother = cuda.to_device(host), cuda.to_device(other)
    dev[::2, 1:90] = dother[1::2, 5:94]          # both sides strided views
    host[::2, 1:90] = other[1::2, 5:94]
    assert dev.copy_to_host().tobytes() == host.tobytes()
    dev[:, 0] = dother[7, :64]                    # a row into a column
    host[:, 0] = other[7, :64]
    assert dev.copy_to_host().tobytes() == host.tobytes()
    import torch
    t = torch.arange(96, dtype=torch.float32, device="cuda")
    dev[5] = t                                     # any CUDA-array-interface exporter
    host[5] = np.arange(96, dtype=np.float32)
    assert dev.copy_to_host().tobytes() == host.tobytes()


def test_setitem_converts_values_like_numpy():
    host = np.zeros((4, 5), dtype=np.int32)
    dev = cuda.to_device(host)
    dev[1] = 7.9                       # Python float into int32
    host[1] = 7.9
    dev[:, 2] = np.arange(4, dtype=np.int64) * 1000
    host[:, 2] = np.arange(4, dtype=np.int64) * 1000
    dev[3] = cuda.to_device(np.arange(5, dtype=np.float64))
    host[3] = np.arange(5, dtype=np.float64)
    assert (dev.copy_to_host() == host).all()


def test_setitem_errors_follow_the_reference():
    dev = cuda.to_device(np.zeros((4, 5), dtype=np.float32))
    with pytest.raises(ValueError, match="Can't assign 3-D array to 2-D self"):
        dev[:, :] = np.zeros((1, 4, 5), dtype=np.float32)
    with pytest.raises(ValueError, match="Can't copy sequence with size 3 to array axis 1 with dimension 5"):
        dev[:, :] = np.zeros((4, 3), dtype=np.float32)
    with pytest.raises(IndexError):
        dev[4, 0] = 1.0


def test_fill_entry_point_every_item_size_and_alignment():
    # b2k_fill: the item travels in the kernel parameters; dense, strided and byte-offset targets
    import torch
    L = _lib.lib()
    for item in (1, 2, 3, 4, 8, 12, 16):
        value = np.random.default_rng(item).integers(0, 256, size=item, dtype=np.uint8)
        for offset in (0, 1, 4, 16):
            buf = torch.zeros(offset + 7 * 48 * item + 64, dtype=torch.uint8, device="cuda")
            arr2 = ctypes.c_int64 * 2
            # 7 rows of 40 items inside rows of 48 items
            rc = L.b2k_fill(buf.data_ptr() + offset, 2, arr2(7, 40), arr2(48 * item, item), value.tobytes(), item, None)
            assert rc == 0, L.b2k_last_error()
            host = buf.cpu().numpy()
            want = np.zeros_like(host)
            view = want[offset:offset + 7 * 48 * item].reshape(7, 48, item)
            view[:, :40, :] = value
            assert host.tobytes() == want.tobytes(), (item, offset)


def test_setitem_with_stream():
    s = cuda.stream()
    host = _filled((33, 65), np.float64, 5)
    dev = cuda.to_device(host, stream=s)
    dev.setitem((slice(None), slice(0, 64, 2)), 1.5, stream=s)
    s.synchronize()
    host[:, 0:64:2] = 1.5
    assert dev.copy_to_host().tobytes() == host.tobytes()


PERMUTE_CASES = [
    ((5, 6), None), ((5, 6), (0, 1)), ((3, 4, 5), None), ((3, 4, 5), (0, 2, 1)), ((3, 4, 5), (1, 0, 2)),
    ((3, 4, 5), (2, 0, 1)), ((3, 4, 5), (1, 2, 0)), ((2, 3, 4, 5), (3, 1, 0, 2)), ((2, 3, 4, 5), (0, 1, 3, 2)),
    ((7, 1, 9), (2, 1, 0)), ((2, 3, 2, 3, 2, 3), (5, 3, 1, 4, 2, 0)), ((40, 50, 60), (2, 1, 0)),
    ((40, 50, 60), (1, 0, 2)), ((33, 70, 130), (0, 2, 1)), ((16, 8, 64, 64), (0, 2, 1, 3)),
    ((0, 4, 5), (2, 0, 1)), ((), ()), ((9,), (0,)),
]


@pytest.mark.parametrize("dtype", [np.uint8, np.uint16, np.float32, np.float64, np.complex128, REC])
@pytest.mark.parametrize("shape,axes", PERMUTE_CASES)
def test_permute_matches_numpy(dtype, shape, axes):
    host = _filled(shape, dtype, 6)
    got = permute(cuda.to_device(host), axes)
    want = host.transpose(axes).copy(order="C")
    assert got.shape == want.shape and got.is_c_contiguous()
    assert got.copy_to_host().tobytes() == want.tobytes()


def test_permute_of_a_strided_view_into_a_given_array_and_errors():
    host = _filled((20, 30, 40), np.float32, 7)
    dev = cuda.to_device(host)
    view = dev[2:18:3, ::-1, 4:36]
    out = cuda.device_array((32, 6, 30), dtype=np.float32)
    assert permute(view, (2, 0, 1), out) is out
    want = np.ascontiguousarray(host[2:18:3, ::-1, 4:36].transpose(2, 0, 1))
    assert out.copy_to_host().tobytes() == want.tobytes()
    with pytest.raises(ValueError, match="invalid axes list"):
        permute(dev, (0, 0, 1))
    with pytest.raises(ValueError, match="incompatible shape"):
        permute(dev, (2, 0, 1), cuda.device_array((40, 30, 20), dtype=np.float32))
    with pytest.raises(TypeError, match="incompatible dtype"):
        permute(dev, (2, 0, 1), cuda.device_array((40, 20, 30), dtype=np.int32))


@pytest.mark.parametrize("dtype", [np.uint8, np.int16, np.float32, np.float64, REC])
def test_copies_between_differently_aligned_runs(dtype):
    # a[i:] = b[j:] for every pair of small offsets: the two sides of each run are aligned differently
    n = 5000
    src = _filled((n,), dtype, 13)
    dsrc = cuda.to_device(src)
    for i in (0, 1, 2, 3, 5, 15, 16, 17):
        for j in (0, 1, 4, 7, 16, 33):
            length = n - 40 - max(i, j)
            host = _filled((n,), dtype, 14)
            dev = cuda.to_device(host)
            dev[i:i + length] = dsrc[j:j + length]
            host[i:i + length] = src[j:j + length]
            assert dev.copy_to_host().tobytes() == host.tobytes(), (i, j)
    # rows of an odd pitch into rows of another odd pitch, short and long rows
    for rows, cols in ((37, 1001), (300, 129), (5, 4097)):
        a, b = _filled((rows, cols + 3), dtype, 15), _filled((rows, cols + 6), dtype, 16)
        da, db = cuda.to_device(a), cuda.to_device(b)
        db[:, 5:5 + cols] = da[:, 2:2 + cols]
        b[:, 5:5 + cols] = a[:, 2:2 + cols]
        assert db.copy_to_host().tobytes() == b.tobytes()
        db[::-1, 1:1 + cols] = da[:, 0:cols]
        b[::-1, 1:1 + cols] = a[:, 0:cols]
        assert db.copy_to_host().tobytes() == b.tobytes()


def test_byte_permutations_on_unaligned_views():
    # 1-byte items: views that start at every byte offset and run with odd pitches, reversed rows
    host = _filled((300, 523), np.uint8, 9)
    dev = cuda.to_device(host)
    for r0, c0, rows, cols in ((0, 0, 300, 523), (1, 1, 255, 401), (3, 2, 129, 130), (2, 3, 64, 33), (5, 7, 290, 500)):
        view, dview = host[r0:r0 + rows, c0:c0 + cols], dev[r0:r0 + rows, c0:c0 + cols]
        assert permute(dview, (1, 0)).copy_to_host().tobytes() == view.T.copy().tobytes()
        out = cuda.device_array((cols + 3, rows + 5), dtype=np.uint8)          # odd destination pitch too
        out[:] = 0
        permute(dview, (1, 0), out[1:cols + 1, 2:rows + 2])
        want = np.zeros((cols + 3, rows + 5), dtype=np.uint8)
        want[1:cols + 1, 2:rows + 2] = view.T
        assert out.copy_to_host().tobytes() == want.tobytes()
    flipped = dev[::-1, 5:205]
    assert permute(flipped, (1, 0)).copy_to_host().tobytes() == host[::-1, 5:205].T.copy().tobytes()
    cube = _filled((7, 131, 197), np.int8, 10)
    assert permute(cuda.to_device(cube), (0, 2, 1)).copy_to_host().tobytes() == cube.transpose(0, 2, 1).copy().tobytes()
    assert permute(cuda.to_device(cube), (2, 1, 0)).copy_to_host().tobytes() == cube.transpose(2, 1, 0).copy().tobytes()


def test_large_permutations_through_both_kernels():
    # (batch, rows, cols) -> (batch, cols, rows): tiles; (a, b, c) -> (b, a, c): direct, wide units
    host = _filled((8, 1000, 1100), np.float32, 8)
    dev = cuda.to_device(host)
    assert permute(dev, (0, 2, 1)).copy_to_host().tobytes() == np.ascontiguousarray(host.transpose(0, 2, 1)).tobytes()
    assert permute(dev, (1, 0, 2)).copy_to_host().tobytes() == np.ascontiguousarray(host.transpose(1, 0, 2)).tobytes()
    assert permute(dev, (2, 1, 0)).copy_to_host().tobytes() == np.ascontiguousarray(host.transpose(2, 1, 0)).tobytes()


def test_c_abi_argument_checks():
    L = _lib.lib()
    arr3 = ctypes.c_int64 * 3
    assert L.b2k_assign(None, None, 3, arr3(2, 0, 4), arr3(32, 16, 4), arr3(32, 16, 4), 4, None) == 0   # empty
    assert L.b2k_assign(None, None, 3, arr3(2, 2, 4), arr3(32, 16, 4), arr3(32, 16, 4), 4, None) < 0    # null
    assert L.b2k_assign(None, None, 40, None, None, None, 4, None) < 0
    assert L.b2k_assign(None, None, 1, arr3(2, 0, 0), arr3(4, 0, 0), arr3(4, 0, 0), 0, None) < 0
    assert b"itemsize" in L.b2k_last_error()
    import torch
    buf = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rc = L.b2k_assign(buf.data_ptr(), buf.data_ptr() + 32, 1, arr3(4, 0, 0), arr3(0, 0, 0), arr3(4, 0, 0), 4, None)
    assert rc < 0 and b"destination stride 0" in L.b2k_last_error()


def test_randomised_assignments_and_permutations_match_numpy():
    # seeded differential test over every kernel the dispatcher can pick: random ranks,
    # shapes, slices (steps of either sign), broadcasts, item sizes and byte offsets
    rng = np.random.default_rng(2024)
    dtypes = [np.uint8, np.int16, np.float32, np.float64, np.complex128, REC]

    def random_view_key(shape):
        key = []
        for n in shape:
            kind = rng.integers(0, 4)
            if kind == 0 or n < 4:
                key.append(slice(None))
            else:
                start = int(rng.integers(0, n // 2))
                stop = int(rng.integers(start + 1, n + 1))
                step = int(rng.choice([1, 1, 2, 3, -1, -2]))
                key.append(slice(start, stop, step) if step > 0 else slice(stop - 1, start - 1 if start > 0 else None, step))
        return tuple(key)

    for case in range(160):
        dtype = dtypes[int(rng.integers(0, len(dtypes)))]
        nd = int(rng.integers(1, 5))
        big = rng.integers(0, 3) == 0
        shape = tuple(int(x) for x in rng.integers(1, 70 if big else 14, size=nd))
        if big and nd >= 2:
            shape = shape[:-2] + (int(rng.integers(33, 300)), int(rng.integers(33, 300)))
        host = _filled(shape, dtype, 1000 + case)
        dev = cuda.to_device(host)
        key = random_view_key(shape)
        target_shape = host[key].shape
        mode = int(rng.integers(0, 4))
        if mode == 0:      # scalar
            value = _filled((), dtype, 2000 + case)[()]
            dev[key] = value
            host[key] = value
        elif mode == 1:    # broadcast of trailing axes, some of length 1
            vshape = tuple(n if rng.integers(0, 3) else 1 for n in target_shape[int(rng.integers(0, len(target_shape) + 1)):])
            value = _filled(vshape, dtype, 3000 + case)
            dev[key] = value
            host[key] = value
        elif mode == 2:    # from a strided device view of another array
            other = _filled(tuple(2 * n + 3 for n in target_shape), dtype, 4000 + case)
            okey = tuple(slice(int(rng.integers(0, 3)), None, 2) for _ in target_shape)
            okey = tuple(slice(k.start, k.start + 2 * n, 2) for k, n in zip(okey, target_shape))
            dev[key] = cuda.to_device(other)[okey]
            host[key] = other[okey]
        else:              # permutation of a view into a fresh array
            axes = tuple(int(x) for x in rng.permutation(nd))
            got = permute(dev[key], axes).copy_to_host()
            assert got.tobytes() == host[key].transpose(axes).copy().tobytes(), (case, shape, key, axes)
            continue
        assert dev.copy_to_host().tobytes() == host.tobytes(), (case, shape, key, mode, np.dtype(dtype))
