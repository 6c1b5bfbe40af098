#!/usr/bin/env python
"""Generate ``gpu_normals_reference.npz``: Box-Muller normals produced ON A GPU by
the reference's own kernel source.

The normals depend on libdevice's logf / cosf / cos, which only run on a
device.  The reference package itself cannot drive a GPU in this image (its
``cuda-core`` dependency is absent), but upstream numba's bundled ``numba.cuda``
ships the same ``random.py`` (identical source apart from imports/formatting)
and compiles it through the same NVVM + libdevice.  Run this on a machine with a
GPU; it writes next to itself or to ``$1``::

    python tests/golden/make_gpu_golden.py [output.npz]

Writes ``output.npz`` (256 generators, every value) and ``output_checksums.npz`` (2^20
generators, block checksums of the bit patterns).

Also prints timings of the stock kernels (cuda.reduce, transpose, RNG) for context.
"""
import json
import os
import sys
import time

import numpy as np

from numba import cuda
from numba.cuda.random import (create_xoroshiro128p_states, xoroshiro128p_normal_float32,
                               xoroshiro128p_normal_float64, xoroshiro128p_uniform_float32,
                               xoroshiro128p_uniform_float64)


@cuda.jit
def c4_kernel(states, u, z, nu, nz):
    t = cuda.grid(1)
    if t < states.shape[0]:
        for i in range(nu):
            u[t * nu + i] = xoroshiro128p_uniform_float32(states, t)
        for i in range(nz):
            z[t * nz + i] = xoroshiro128p_normal_float64(states, t)


@cuda.jit
def normal32_kernel(states, out, count):
    t = cuda.grid(1)
    if t < states.shape[0]:
        for i in range(count):
            out[t * count + i] = xoroshiro128p_normal_float32(states, t)


@cuda.jit
def normal64_kernel(states, out, count):
    t = cuda.grid(1)
    if t < states.shape[0]:
        for i in range(count):
            out[t * count + i] = xoroshiro128p_normal_float64(states, t)


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else "gpu_normals_reference.npz"
    info = {"device": cuda.get_current_device().name.decode() if isinstance(cuda.get_current_device().name, bytes)
            else str(cuda.get_current_device().name), "cc": list(cuda.get_current_device().compute_capability)}
    n = 256
    res = {}
    st = create_xoroshiro128p_states(n, seed=42)
    res["states0"] = np.stack([st.copy_to_host()["s0"], st.copy_to_host()["s1"]], axis=1)
    u = cuda.device_array(n * 64, dtype=np.float32)
    z = cuda.device_array(n * 16, dtype=np.float64)
    c4_kernel[(n + 127) // 128, 128](st, u, z, 64, 16)
    res["c4_u"] = u.copy_to_host().reshape(n, 64)
    res["c4_z"] = z.copy_to_host().reshape(n, 16)
    e = st.copy_to_host()
    res["c4_end"] = np.stack([e["s0"], e["s1"]], axis=1)
    st = create_xoroshiro128p_states(n, seed=42)
    o = cuda.device_array(n * 32, dtype=np.float32)
    normal32_kernel[(n + 127) // 128, 128](st, o, 32)
    res["normal_f32"] = o.copy_to_host().reshape(n, 32)
    st = create_xoroshiro128p_states(n, seed=42)
    o = cuda.device_array(n * 32, dtype=np.float64)
    normal64_kernel[(n + 127) // 128, 128](st, o, 32)
    res["normal_f64"] = o.copy_to_host().reshape(n, 32)
    np.savez_compressed(out_path, **res)

    # The same three kernels over 2^20 generators, kept as block checksums of the bit
    # patterns (tests/config_inputs.py:block_checksums): a bit-level pin of 2^26 uniforms
    # and 2^24 + 2 * 2^25 normals in a few kilobytes.
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
    from config_inputs import block_checksums
    big = 1 << 20
    sums = {"generators": np.int64(big), "rows_per_block": np.int64(4096)}
    st = create_xoroshiro128p_states(big, seed=42)
    u = cuda.device_array(big * 64, dtype=np.float32)
    z = cuda.device_array(big * 16, dtype=np.float64)
    c4_kernel[(big + 127) // 128, 128](st, u, z, 64, 16)
    sums["c4_u"] = block_checksums(u.copy_to_host().reshape(big, 64))
    sums["c4_z"] = block_checksums(z.copy_to_host().reshape(big, 16))
    e = st.copy_to_host()
    sums["c4_end"] = block_checksums(np.stack([e["s0"], e["s1"]], axis=1).view(np.float64))
    del u, z
    st = create_xoroshiro128p_states(big, seed=42)
    o = cuda.device_array(big * 32, dtype=np.float32)
    normal32_kernel[(big + 127) // 128, 128](st, o, 32)
    sums["normal_f32"] = block_checksums(o.copy_to_host().reshape(big, 32))
    st = create_xoroshiro128p_states(big, seed=42)
    o = cuda.device_array(big * 32, dtype=np.float64)
    normal64_kernel[(big + 127) // 128, 128](st, o, 32)
    sums["normal_f64"] = block_checksums(o.copy_to_host().reshape(big, 32))
    del o
    np.savez_compressed(out_path.replace(".npz", "_checksums.npz"), **sums)

    # context timings of the stock kernels on this GPU (not fixtures)
    def timeit(fn, reps=5):
        fn()
        cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        cuda.synchronize()
        return (time.perf_counter() - t0) / reps

    try:
        x = cuda.to_device(np.random.default_rng(1).integers(-2 ** 31, 2 ** 31, size=1 << 28, dtype=np.int32))
        mx = cuda.reduce(lambda a, b: max(a, b))
        res0 = cuda.device_array(1, dtype=np.int32)
        info["reduce_max_int32_2p28_s"] = timeit(lambda: mx(x, res=res0))
        del x
        a = cuda.to_device(np.zeros((8192, 8192), dtype=np.float32))
        info["transpose_f32_8192_s_incl_jit"] = timeit(lambda: a.T, reps=2)
        del a
        n2 = 1 << 20
        t0 = time.perf_counter()
        st = create_xoroshiro128p_states(n2, seed=42)
        cuda.synchronize()
        info["create_states_2p20_s"] = time.perf_counter() - t0
        u = cuda.device_array(n2 * 64, dtype=np.float32)
        z = cuda.device_array(n2 * 16, dtype=np.float64)
        info["c4_kernel_2p20_states_s"] = timeit(lambda: c4_kernel[(n2 + 127) // 128, 128](st, u, z, 64, 16))
    except Exception as exc:  # context only
        info["timing_error"] = repr(exc)
    print(json.dumps(info))


if __name__ == "__main__":
    main()
