"""cuda.reduce on the GPU against the CPU oracle.  The cases restate
numba/cuda/tests/cudapy/test_reduction.py and add every dtype/op, ragged sizes,
unaligned bases and the two benchmark configurations."""
import math
import os

import numpy as np
import pytest
import torch

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib

pytestmark = pytest.mark.gpu

sum_reduce = cuda.Reduce(lambda a, b: a + b)


@pytest.mark.parametrize("n", [1, 15, 16, 17, 127, 128, 129, 1023, 1024, 1025, 1536, 1048576, 1049600,
                               1049728, 34567])
def test_sum_reduce(n):
    # test_reduction.py:21-48: integer-valued float64, so the sum is exact
    A = np.arange(n, dtype=np.float64) + 1
    assert A.sum() == sum_reduce(A)


def test_empty_array_host():
    A = np.arange(0, dtype=np.float64) + 1
    assert sum_reduce(A) == 0.0


def test_empty_array_device():
    A = cuda.to_device(np.arange(0, dtype=np.float64) + 1)
    assert sum_reduce(A) == 0.0


def test_prod_reduce():
    prod = cuda.reduce(lambda a, b: a * b)
    A = np.arange(64, dtype=np.float64) + 1
    np.testing.assert_allclose(A.prod(), prod(A, init=1))


def test_max_reduce():
    mx = cuda.Reduce(lambda a, b: max(a, b))
    A = np.random.default_rng(5).random(3717)
    assert A.max() == mx(A, init=0)
    B = -A                                   # all negative: the default init (0) wins
    assert mx(B) == 0.0 and mx(B, init=-10.0) == B.max()


def test_non_identity_init():
    A = np.arange(10, dtype=np.float64) + 1
    assert A.sum() + 3 == sum_reduce(A, init=3)


def test_result_on_device():
    A = np.arange(10, dtype=np.float64) + 1
    got = cuda.to_device(np.zeros(1, dtype=np.float64))
    assert sum_reduce(A, res=got) is None
    assert got.copy_to_host()[0] == A.sum()
    assert got[0] == A.sum()


def test_result_dtype_and_res_mismatch():
    A = np.arange(10, dtype=np.int32)
    out = sum_reduce(A)
    assert out.dtype == np.int32 and out == 45
    with pytest.raises(TypeError, match="incompatible dtype"):
        sum_reduce(A, res=cuda.to_device(np.zeros(1, dtype=np.float64)))


def test_golden_simulator_values(golden_dir):
    g = np.load(os.path.join(golden_dir, "reduce_reference.npz"))
    x = np.random.default_rng(0).random(1 << 20)
    got = sum_reduce(x)                                          # configuration 1
    assert abs(got - g["c1_sum"]) <= 1e-12 * abs(g["c1_sum"])
    assert abs(got - math.fsum(x)) <= 1e-12 * math.fsum(x)
    y = np.random.default_rng(1).integers(-2 ** 31, 2 ** 31, size=int(g["c2_prefix_len"]), dtype=np.int32)
    assert cuda.reduce(lambda a, b: max(a, b))(y) == g["c2_prefix_max"]
    assert sum_reduce(np.arange(34567, dtype=np.float64) + 1) == g["sum_arange_34567"]
    assert cuda.reduce(lambda a, b: max(a, b))(g["max_input"], init=0) == g["max_3717_init0"]
    assert sum_reduce(np.arange(10, dtype=np.float64) + 1, init=3) == g["sum_10_init3"]


def test_every_small_length_int32():
    rng = np.random.default_rng(9)
    x = rng.integers(-2 ** 31, 2 ** 31, size=1200, dtype=np.int32)
    d = cuda.to_device(x)
    mx = cuda.reduce(lambda a, b: max(a, b))
    for n in range(0, 1101):
        assert sum_reduce(d, size=n) == oracle.fold(x[:n], "add", 0), n
        if n % 37 == 0:
            assert mx(d, size=n, init=-2 ** 31) == oracle.fold(x[:n], "max", -2 ** 31), n


OPS = {"add": lambda a, b: a + b, "mul": lambda a, b: a * b, "max": lambda a, b: max(a, b),
       "min": lambda a, b: min(a, b), "and": lambda a, b: a & b, "or": lambda a, b: a | b,
       "xor": lambda a, b: a ^ b}


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32,
                                   np.uint64, np.float32, np.float64])
@pytest.mark.parametrize("op", list(OPS))
def test_all_ops_all_dtypes(dtype, op):
    dt = np.dtype(dtype)
    if dt.kind == "f" and op in ("and", "or", "xor"):
        pytest.skip("bitwise ops are integer only")
    rng = np.random.default_rng(hash((dt.str, op)) % 2 ** 32)
    for n in (1, 31, 4099, 1 << 20):
        if dt.kind == "f":
            x = (rng.random(n) + 0.5).astype(dt) if op == "mul" else rng.standard_normal(n).astype(dt)
            if op == "mul":
                x = x[: min(n, 200)]
        else:
            info = np.iinfo(dt)
            x = rng.integers(info.min, info.max, size=n, dtype=dt, endpoint=True)
        init = {"mul": 1, "and": -1 if dt.kind == "i" else np.iinfo(dt).max if dt.kind == "u" else 0}.get(op, 0)
        if op == "min":
            init = x.max()
        got = cuda.reduce(OPS[op])(x, init=init)
        want = oracle.fold(x, op, init)
        assert got.dtype == dt
        if dt.kind == "f" and op in ("add", "mul"):
            tol = 1e-12 if dt == np.float64 else 1e-5
            scale = max(abs(float(want)), float(np.abs(x).sum()) if op == "add" else abs(float(want)))
            assert abs(float(got) - float(want)) <= tol * scale, (n, got, want)
        else:
            assert got == want, (n, got, want)


@pytest.mark.parametrize("dtype", [np.int8, np.int32, np.float64])
def test_unaligned_base_pointers(dtype):
    x = (np.random.default_rng(2).integers(-100, 100, size=5000)).astype(dtype)
    d = cuda.to_device(x)
    for off in range(0, 20):
        for n in (0, 1, 3, 16, 17, 1000, 5000 - off):
            assert sum_reduce(d[off:off + n]) == oracle.fold(x[off:off + n], "add", 0), (off, n)


def test_strided_view_input():
    x = np.arange(1000, dtype=np.int64)
    d = cuda.to_device(x)
    assert sum_reduce(d[::2]) == x[::2].sum()
    assert sum_reduce(d[5::7]) == x[5::7].sum()


def test_float32_sum_tolerance_and_determinism():
    x = np.random.default_rng(8).random(1 << 24, dtype=np.float32)
    d = cuda.to_device(x)
    a, b = sum_reduce(d), sum_reduce(d)
    assert a.tobytes() == b.tobytes()
    exact = math.fsum(x.astype(np.float64))
    assert abs(float(a) - exact) <= 1e-5 * exact


def test_config2_full_size_int32_max():
    n = 1 << 28
    x = np.random.default_rng(1).integers(-2 ** 31, 2 ** 31, size=n, dtype=np.int32)
    d = cuda.to_device(x)
    mx = cuda.reduce(lambda a, b: max(a, b))
    assert mx(d) == max(int(x.max()), 0)
    assert mx(d, init=-2 ** 31) == x.max()
    assert cuda.reduce(lambda a, b: min(a, b))(d, init=2 ** 31 - 1) == x.min()
    assert sum_reduce(d) == np.add.reduce(x, dtype=np.int32)
    # sharded view of the same array: per-shard results combine to the whole
    parts = [mx(d[lo:hi], init=-2 ** 31) for lo, hi in
             (cuda.sharded.shard_bounds(n, 8, r) for r in range(8))]
    assert max(parts) == x.max()


def test_stream_argument_and_raw_c_abi():
    s = cuda.stream()
    x = np.arange(100000, dtype=np.float64)
    assert sum_reduce(cuda.to_device(x, stream=s), stream=s) == x.sum()
    # straight through the C ABI with torch-owned buffers
    L = _lib.lib()
    t = torch.arange(1, 1001, dtype=torch.int64, device="cuda")
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    init = np.array([7], dtype=np.int64)
    before = L.b2k_launch_count()
    for _ in range(3):  # the scratch is left reusable
        rc = L.b2k_reduce(_lib.ADD, _lib.I64, t.data_ptr(), t.numel(), init.ctypes.data, out.data_ptr(),
                          scratch.data_ptr(), scratch.numel(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, L.b2k_last_error()
        assert out.item() == 500500 + 7
    assert L.b2k_launch_count() == before + 3
    assert int(scratch[:4].view(torch.int32).item()) == 0


def test_untraceable_functor_raises():
    import math
    with pytest.raises(NotImplementedError):
        cuda.reduce(lambda a, b: math.sqrt(a) + b)(np.arange(10.0))
    with pytest.raises(NotImplementedError):
        cuda.reduce(lambda a, b: a + b)(np.arange(10.0).astype(np.complex128))


def test_two_host_threads_reducing_on_one_stream_get_their_own_results():
    """Modelled on tests/cudapy/test_multithreads.py:40-68 of the reference: host threads
    share the device and the default stream; every call must return ITS result."""
    import threading
    reducers = {"add": cuda.reduce(lambda a, b: a + b), "max": cuda.reduce(lambda a, b: max(a, b))}
    arrays = [cuda.to_device(np.random.default_rng(50 + t).integers(-1000, 1000, size=20000 + 7 * t, dtype=np.int64))
              for t in range(4)]
    hosts = [a.copy_to_host() for a in arrays]
    errors = []

    def work(t):
        try:
            torch.cuda.set_device(0)
            for k in range(300):
                name = "add" if (k + t) % 2 else "max"
                got = reducers[name](arrays[t], init=t)
                want = hosts[t].sum() + t if name == "add" else max(hosts[t].max(), t)
                if got != want:
                    errors.append((t, k, name, int(got), int(want)))
                    return
        except Exception as exc:     # noqa: BLE001
            errors.append((t, repr(exc)))

    threads = [threading.Thread(target=work, args=(t,)) for t in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors[:3]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_in_the_same_process():
    """Function attributes (the dynamic shared-memory limit of the TMA transposes and of
    state creation) belong to a device: everything must also run on device 1 after
    device 0 has been used."""
    from numba_cuda_b200.kernels.transpose import permute, transpose
    from numba_cuda_b200.random import create_xoroshiro128p_states
    a = np.random.default_rng(3).standard_normal((1024, 2048)).astype(np.float32)
    cube = np.arange(32 * 64 * 128, dtype=np.float32).reshape(32, 64, 128)
    want_states = oracle.init_states(1 << 18, 9, 0)
    try:
        for dev in (0, 1):
            torch.cuda.set_device(dev)
            assert transpose(cuda.to_device(a)).copy_to_host().tobytes() == np.ascontiguousarray(a.T).tobytes()
            assert permute(cuda.to_device(cube), (0, 2, 1)).copy_to_host().tobytes() == \
                np.ascontiguousarray(cube.transpose(0, 2, 1)).tobytes()
            st = create_xoroshiro128p_states(1 << 18, seed=9)
            assert st.copy_to_host().tobytes() == want_states.tobytes()
            assert cuda.reduce(lambda x, y: x + y)(np.arange(100000, dtype=np.int64)) == 100000 * 99999 // 2
    finally:
        torch.cuda.set_device(0)


def test_a_run_of_reductions_with_input_ready_overlaps_and_keeps_every_result():
    """Reductions over arrays that were complete before the run started may overlap
    (programmatic dependent launch); results, scratch and order stay those of the stream.
    Also through the C ABI with both flag values, on sizes that use one CTA and a full grid."""
    rng = np.random.default_rng(21)
    arrays = [rng.integers(-2 ** 31, 2 ** 31, size=n, dtype=np.int64).astype(np.int32)
              for n in (5, 4096, 100003, (1 << 22) + 7, 3, (1 << 21) + 1, 777, 1 << 20)]
    dev = [cuda.to_device(a) for a in arrays]
    res = [cuda.device_array(1, np.int32) for _ in arrays]
    cuda.synchronize()
    fold = cuda.reduce(lambda a, b: max(a, b))
    for _ in range(3):                       # the same scratch serves every launch of the run
        for d, r in zip(dev, res):
            assert fold(d, res=r, init=-2 ** 31, input_ready=True) is None
    for a, r in zip(arrays, res):
        assert r.copy_to_host()[0] == a.max()
    total = cuda.reduce(lambda a, b: a + b)
    sums = [cuda.device_array(1, np.int32) for _ in arrays]
    for d, r in zip(dev, sums):
        total(d, res=r, input_ready=True)
    for a, r in zip(arrays, sums):
        assert r.copy_to_host()[0] == a.sum(dtype=np.int32)
    # a host array is staged by the call itself: the promise is dropped, the result is the same
    assert fold(arrays[3], init=-2 ** 31, input_ready=True) == arrays[3].max()
    # a strided view is gathered first: same
    assert fold(dev[3][::2], init=-2 ** 31, input_ready=True) == arrays[3][::2].max()
