#!/usr/bin/env python
"""Generate the golden fixtures in this folder by EXECUTING THE REFERENCE.

Run only in a container that has the reference tree mounted (``--reference``);
the fixtures it writes are committed so that the tests need no reference at
run time.  Usage::

    python tests/golden/make_golden.py [--reference <numba-cuda checkout>]

Recipe (the reference is read-only and its C extensions are not built, and the
``cuda-core`` dependency is not installed):

1. copy the reference tree to a temporary directory and run
   ``python setup.py build_ext --inplace`` there;
2. put an import-only placeholder for ``cuda.core`` on PYTHONPATH;
3. ``import _numba_cuda_redirector`` so that ``numba.cuda`` resolves to the
   reference's ``numba_cuda/numba/cuda``;
4. run two children: one with ``NUMBA_ENABLE_CUDASIM=0`` (the RNG functions are
   CPU ``@jit`` functions and run natively on host arrays) and one with
   ``NUMBA_ENABLE_CUDASIM=1`` (``cuda.reduce`` and simulated kernels);
5. evaluate the vendored ``cuda_fp8.hpp`` / ``cuda_bf16.hpp`` host paths through
   ``oracle/_ref/libb2k_ref_headers.so`` (built by ``oracle/Makefile``).

Outputs: ``rng_reference.npz``, ``reduce_reference.npz``, ``cast_reference.npz``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile
import textwrap

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

STUB_INIT = '''
"""Import-only placeholder for the absent cuda-core package."""
__version__ = "0.5.1"
class _P:
    def __init__(self, *a, **k): pass
    def __call__(self, *a, **k): return _P()
    def __getattr__(self, n): return _P()
for _n in ("Buffer","Device","Stream","Event","Program","ProgramOptions","LaunchConfig",
           "GraphBuilder","Linker","LinkerOptions","ObjectCode","Kernel"):
    globals()[_n] = type(_n, (_P,), {})
def launch(*a, **k): raise RuntimeError("cuda.core placeholder")
def __getattr__(name): return type(name, (_P,), {})
'''
STUB_UTILS = '''
class StridedMemoryView:
    def __init__(self, *a, **k): pass
def __getattr__(name): return type(name, (), {})
'''

CHILD_JIT = r'''
import sys, numpy as np
import _numba_cuda_redirector  # noqa
from numba import cuda
assert "numba_cuda" in cuda.__file__, cuda.__file__
from numba.cuda import random as R
out = {}
def states(n, seed, start):
    st = np.empty(n, dtype=R.xoroshiro128p_dtype)
    R.init_xoroshiro128p_states_cpu(st, seed, start)
    return st
def as2(st):
    return np.stack([st["s0"], st["s1"]], axis=1)
out["states_seed42_n64"] = as2(states(64, 42, 0))
out["states_seed1_n4"] = as2(states(4, 1, 0))
out["states_seed1_start2_n8"] = as2(states(8, 1, 2))
out["states_seed7_start1000_n4"] = as2(states(4, 7, 1000))
big = states(1 << 20, 42, 0)
idx = np.array([0, 1, 2, 3, 31, 32, 255, 256, 257, 4095, 4096, 65535, 65536, 65537,
                (1 << 19) - 1, 1 << 19, (1 << 20) - 1], dtype=np.int64)
out["big_idx"] = idx
out["big_states_seed42"] = as2(big[idx])
# every 4099th state as a stride check of the whole chain
out["big_stride"] = np.int64(4099)
out["big_states_seed42_strided"] = as2(big[::4099])
# draws: 4 generators, seed 42
def draws(fn, dtype, count, n=4, seed=42):
    st = states(n, seed, 0)
    o = np.empty((n, count), dtype=dtype)
    for t in range(n):
        for i in range(count):
            o[t, i] = fn(st, t)
    return o, as2(st)
out["uniform_f32"], out["uniform_f32_end"] = draws(R.xoroshiro128p_uniform_float32, np.float32, 64)
out["uniform_f64"], out["uniform_f64_end"] = draws(R.xoroshiro128p_uniform_float64, np.float64, 64)
# normals on the CPU-jitted path use the host libm (NOT the GPU's libdevice)
out["normal_f32_hostlibm"], out["normal_f32_end"] = draws(R.xoroshiro128p_normal_float32, np.float32, 32)
out["normal_f64_hostlibm"], out["normal_f64_end"] = draws(R.xoroshiro128p_normal_float64, np.float64, 32)
# the config-4 sequence: 64 uniform f32 then 16 normal f64 per generator
st = states(8, 42, 0)
u = np.empty((8, 64), np.float32); z = np.empty((8, 16), np.float64)
for t in range(8):
    for i in range(64): u[t, i] = R.xoroshiro128p_uniform_float32(st, t)
    for i in range(16): z[t, i] = R.xoroshiro128p_normal_float64(st, t)
out["c4_u"], out["c4_z_hostlibm"], out["c4_end"] = u, z, as2(st)
np.savez_compressed(sys.argv[1], **out)
'''

CHILD_SIM = r'''
import sys, numpy as np
import _numba_cuda_redirector  # noqa
from numba import cuda
from numba.cuda import config
assert config.ENABLE_CUDASIM and "numba_cuda" in cuda.__file__
out = {}
x = np.random.default_rng(0).random(1 << 20)
out["c1_sum"] = np.float64(cuda.reduce(lambda a, b: a + b)(x))
y = np.random.default_rng(1).integers(-2**31, 2**31, size=1 << 18, dtype=np.int32)
out["c2_prefix_len"] = np.int64(y.size)
out["c2_prefix_max"] = np.int32(cuda.reduce(lambda a, b: max(a, b))(y))
# the reference test cases (tests/cudapy/test_reduction.py)
A = np.arange(34567, dtype=np.float64) + 1
out["sum_arange_34567"] = np.float64(cuda.reduce(lambda a, b: a + b)(A))
B = np.arange(64, dtype=np.float64) + 1
out["prod_64_init1"] = np.float64(cuda.reduce(lambda a, b: a * b)(B, init=1))
C = np.random.default_rng(5).integers(-1000, 1000, size=3717).astype(np.float64)
out["max_input"] = C
out["max_3717_init0"] = np.float64(cuda.reduce(lambda a, b: max(a, b))(C, init=0))
out["sum_10_init3"] = np.float64(cuda.reduce(lambda a, b: a + b)(np.arange(10, dtype=np.float64) + 1, init=3))
# the simulator running the RNG device functions inside a simulated kernel
from numba.cuda.random import create_xoroshiro128p_states, xoroshiro128p_uniform_float32
@cuda.jit
def k(states, o, count):
    t = cuda.grid(1)
    for i in range(count):
        o[t * count + i] = xoroshiro128p_uniform_float32(states, t)
st = create_xoroshiro128p_states(8, seed=42)
o = np.zeros(8 * 4, dtype=np.float32)
k[1, 8](st, o, 4)
out["sim_uniform_f32_8x4"] = o.reshape(8, 4)
np.savez_compressed(sys.argv[1], **out)
'''


def f32_probe_inputs() -> np.ndarray:
    """float32 bit patterns that straddle every fp8 / bf16 rounding decision."""
    top12 = np.arange(4096, dtype=np.uint32) << 20          # sign, exponent, 3 mantissa bits
    low20 = np.array([0x00000, 0x00001, 0x7FFFF, 0x80000, 0x80001, 0xFFFFF], dtype=np.uint32)
    a = (top12[:, None] | low20[None, :]).ravel()
    sign = np.arange(2, dtype=np.uint32) << 31
    expo = np.arange(256, dtype=np.uint32) << 23
    m7 = np.array([0, 1, 2, 0x3F, 0x40, 0x7E, 0x7F], dtype=np.uint32) << 16
    low16 = np.array([0x0000, 0x0001, 0x7FFF, 0x8000, 0x8001, 0xFFFF], dtype=np.uint32)
    b = (sign[:, None, None, None] | expo[None, :, None, None] | m7[None, None, :, None]
         | low16[None, None, None, :]).ravel()
    extra = np.array([1e20, -1e20, 1e6, -1e6, 448.0, 464.0, 465.0, 57344.0, 61440.0, 61441.0,
                      2.0 ** -10, 2.0 ** -9, 2.0 ** -17, 2.0 ** -16, 0.017, 1.0, 2.0, 4.0, 1.5, 3.14],
                     dtype=np.float32).view(np.uint32)
    return np.unique(np.concatenate([a, b, extra]))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a numba-cuda source tree")
    args = ap.parse_args()
    if not os.path.isdir(args.reference):
        sys.exit("reference tree not found: fixtures can only be regenerated where it is mounted")

    with tempfile.TemporaryDirectory() as tmp:
        ref = os.path.join(tmp, "ref")
        shutil.copytree(args.reference, ref)
        subprocess.run([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=ref, check=True,
                       capture_output=True)
        stub = os.path.join(tmp, "stub", "cuda", "core")
        os.makedirs(stub)
        open(os.path.join(stub, "__init__.py"), "w").write(textwrap.dedent(STUB_INIT))
        open(os.path.join(stub, "utils.py"), "w").write(textwrap.dedent(STUB_UTILS))
        env = dict(os.environ)
        env["PYTHONPATH"] = os.pathsep.join([ref, os.path.join(ref, "site-packages"),
                                             os.path.join(tmp, "stub")])
        for name, code, sim in (("rng_reference.npz", CHILD_JIT, "0"),
                                ("reduce_reference.npz", CHILD_SIM, "1")):
            script = os.path.join(tmp, name + ".py")
            open(script, "w").write(code)
            env["NUMBA_ENABLE_CUDASIM"] = sim
            subprocess.run([sys.executable, script, os.path.join(HERE, name)], env=env, check=True)
            print("wrote", name)

    # fp8 / bf16: the reference's vendored headers, host path
    sys.path.insert(0, ROOT)
    import oracle
    oracle.build()
    R = oracle.ref_headers()
    bits = f32_probe_inputs()
    x = bits.view(np.float32)
    out = {"f32_bits": bits}
    for name, dst in (("e4m3", oracle.E4M3), ("e5m2", oracle.E5M2)):
        out[f"{name}_satfinite"] = oracle.ref_cast(x, oracle.F32, dst, sat=1)
        out[f"{name}_nosat"] = oracle.ref_cast(x, oracle.F32, dst, sat=0)
        codes = np.arange(256, dtype=np.uint8)
        out[f"{name}_decode_f32_bits"] = oracle.ref_cast(codes, dst, oracle.F32).view(np.uint32)
        out[f"{name}_decode_half_bits"] = np.array(
            [R.ref_cvt_fp8_to_halfraw(int(c), dst - 2) for c in codes], dtype=np.uint16)
        out[f"{name}_ctor"] = np.array(
            [R.ref_fp8_from_float(float(v), dst - 2) for v in (1.0, 2.0, 4.0, 1e20, -1e20)], dtype=np.uint8)
    out["bf16_rn"] = oracle.ref_cast(x, oracle.F32, oracle.BF16)
    # directed rounding, f64 -> bf16 and the E8M0 scale type (vendored headers, host path)
    for mode, tag in ((1, "rz"), (2, "ru"), (3, "rd")):
        out[f"bf16_{tag}"] = np.array([R.ref_float2bfloat16_mode(float(v), mode) for v in x], dtype=np.uint16)
    for sat, stag in ((0, "nosat"), (1, "satfinite")):
        for mode, mtag in ((1, "rz"), (2, "rp")):
            out[f"e8m0_from_f32_{stag}_{mtag}"] = np.array(
                [R.ref_cvt_float_to_e8m0(float(v), sat, mode) for v in x], dtype=np.uint8)
            out[f"e8m0_from_bf16_{stag}_{mtag}"] = np.array(
                [R.ref_cvt_bfloat16raw_to_e8m0(h, sat, mode) for h in range(65536)], dtype=np.uint8)
    out["e8m0_to_bf16"] = np.array([R.ref_cvt_e8m0_to_bf16raw(e) for e in range(256)], dtype=np.uint16)
    rng = np.random.default_rng(12)
    d = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-42, 40, size=4000),
                        x[::11].astype(np.float64) * (1 + 2.0 ** -30),
                        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e300, -1e300, 1e-300, 1.00390625,
                                  1.0039062500000002, 1.0039062499999998])])
    out["f64_inputs"] = d
    out["bf16_from_f64"] = np.array([R.ref_double2bfloat16(float(v)) for v in d], dtype=np.uint16)
    np.savez_compressed(os.path.join(HERE, "cast_reference.npz"), **out)
    print("wrote cast_reference.npz", bits.size, "probe inputs")


if __name__ == "__main__":
    main()
