"""User CUDA C++ kernels written against include/b2k_xoroshiro128p.cuh consume
the same stream as the reference's device functions: the documentation
example's 3-D strided fill (numba/cuda/tests/doc_examples/test_random.py:13-62)
and a per-thread normals kernel, both checked against the CPU oracle and the
GPU-generated reference fixture."""
import ctypes
import os

import numpy as np
import pytest

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _build
from numba_cuda_b200.random import create_xoroshiro128p_states

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def examples():
    path = _build.EXAMPLES_LIB
    if not os.path.exists(path):
        pytest.fail("libb2k_examples.so is not built (python -m numba_cuda_b200._build)")
    L = ctypes.CDLL(path)
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    L.b2k_example_random_3d.argtypes = [vp, i64, i64, i64, vp, i32, i32, i32, i32, i32, i32, vp]
    L.b2k_example_normals_per_thread.argtypes = [vp, i64, vp, i32, vp]
    return L


def test_doc_example_3d_grid(examples):
    # test_random.py:38-62, full size: statistics only, as the reference asserts
    X, Y, Z = 701, 900, 719
    bx, by, bz, gx, gy, gz = 8, 8, 8, 16, 16, 16
    nthreads = bx * by * bz * gx * gy * gz
    rng_states = create_xoroshiro128p_states(nthreads, seed=1)
    arr = cuda.device_array((X, Y, Z), dtype=np.float32)
    assert examples.b2k_example_random_3d(arr._ptr, X, Y, Z, rng_states._ptr, gx, gy, gz, bx, by, bz, None) == 0
    host = arr.copy_to_host()
    assert 0.49 < host.mean() < 0.51
    assert (host <= 1.0).all() and (host >= 0.0).all()


def test_3d_fill_is_bit_exact_on_a_small_grid(examples):
    X, Y, Z = 5, 7, 9                       # arr.shape; arr[i, j, k] with k fastest
    bx, by, bz, gx, gy, gz = 2, 2, 1, 2, 1, 2
    sx, sy, sz = bx * gx, by * gy, bz * gz
    nthreads = sx * sy * sz
    states = create_xoroshiro128p_states(nthreads, seed=9)
    arr = cuda.device_array((X, Y, Z), dtype=np.float32)
    assert examples.b2k_example_random_3d(arr._ptr, X, Y, Z, states._ptr, gx, gy, gz, bx, by, bz, None) == 0
    got = arr.copy_to_host()
    host = oracle.init_states(nthreads, 9, 0)
    want = np.zeros((X, Y, Z), dtype=np.float32)
    for z in range(sz):
        for y in range(sy):
            for x in range(sx):
                tid = z * sy * sx + y * sx + x
                cells = [(i, j, k) for i in range(z, X, sz) for j in range(y, Y, sy) for k in range(x, Z, sx)]
                draws = oracle.fill(host[tid:tid + 1], "uniform", np.float32, len(cells))[0] if cells else []
                for (i, j, k), v in zip(cells, draws):
                    want[i, j, k] = v
    assert got.tobytes() == want.tobytes()
    assert states.copy_to_host().tobytes() == host.tobytes()


def test_register_resident_normals_match_gpu_reference(examples, golden_dir):
    g = np.load(os.path.join(golden_dir, "gpu_normals_reference.npz"))
    n = g["states0"].shape[0]
    states = create_xoroshiro128p_states(n, 42, 0)
    out = cuda.device_array((n, 32), dtype=np.float64)
    assert examples.b2k_example_normals_per_thread(states._ptr, n, out._ptr, 32, None) == 0
    assert out.copy_to_host().tobytes() == g["normal_f64"].tobytes()
