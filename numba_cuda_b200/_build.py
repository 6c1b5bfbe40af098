"""Builds ``libb2k.so`` in-tree with nvcc for sm_100a.

``python -m numba_cuda_b200._build [--force] [--verbose]`` or :func:`build`.
nvcc cross-compiles without a GPU; the built library sits next to the sources
(``csrc/libb2k.so``) so it travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libb2k.so")

SOURCES = [
    "b2k_api.cu",
    "b2k_reduce.cu",
    "b2k_reduce_user.cu",
    "b2k_reduce_axis.cu",
    "b2k_cast.cu",
    "b2k_xoroshiro.cu",
    "b2k_transpose.cu",
    "b2k_transpose_tma.cu",
    "b2k_assign.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libb2k.so cannot be built")


def _deps(src: str) -> list[str]:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "b2k.h"))
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "b2k_xoroshiro128p.cuh"))
    return [src] + hdrs


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link ``libb2k.so``; returns its path."""
    nvcc = _nvcc()
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for name in SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(objdir, name[:-3] + ".o")
        if force or _stale(obj, _deps(src)):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((name, cmd))

    def run(job):
        name, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return name, p.returncode, p.stdout + p.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for name, rc, log in pool.map(run, jobs):
            if verbose or rc != 0:
                sys.stderr.write(f"--- {name}\n{log}\n")
            if rc != 0:
                raise RuntimeError(f"nvcc failed on {name}")
    objs = [os.path.join(objdir, n[:-3] + ".o") for n in SOURCES]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC", "-cudart", "static", "-ldl"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("linking libb2k.so failed")
    return LIB


EXAMPLES_LIB = os.path.join(CSRC, "examples", "libb2k_examples.so")


def build_examples(force: bool = False) -> str:
    """Compile the example user kernels (``csrc/examples``) that are written
    against ``include/b2k_xoroshiro128p.cuh``; the tests load the result."""
    src = os.path.join(CSRC, "examples", "rng_user_kernels.cu")
    hdr = os.path.join(os.path.dirname(HERE), "include", "b2k_xoroshiro128p.cuh")
    if force or _stale(EXAMPLES_LIB, [src, hdr]):
        cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", EXAMPLES_LIB, src, "-cudart", "static"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("building libb2k_examples.so failed")
    return EXAMPLES_LIB


if __name__ == "__main__":
    build_examples(force="--force" in sys.argv)
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
