"""B200-native drop-in for numba-cuda's built-in library kernels.

``import numba_cuda_b200 as cuda`` gives the names a user of ``numba.cuda``
reaches for on this path::

    cuda.reduce / cuda.Reduce          (numba/cuda/kernels/reduction.py)
    cuda.to_device, cuda.device_array, cuda.as_cuda_array, d_arr.T ...
    cuda.kernels.transpose.transpose   (numba/cuda/kernels/transpose.py)
    cuda.random.*                      (numba/cuda/random.py)
    cuda.bf16.*, cuda.fp8.*            (conversion intrinsics, bulk and scalar)
    cuda.sharded.*                     (contiguous-shard multi-GPU wrappers; new)

Host code is Python; all device work is hand-written sm_100a CUDA in
``csrc/libb2k.so`` behind the C ABI of ``include/b2k.h``.  There is no CPU
fallback: without the library or without a GPU the calls raise.
"""
from . import _lib, bf16, casts, fp8, kernels, random, sharded  # noqa: F401
from .api import (as_cuda_array, auto_device, default_stream, device_array, device_array_like,  # noqa: F401
                  event, event_elapsed_time, external_stream, is_available, is_bfloat16_supported, is_cuda_array,
                  is_fp8_supported, pinned_array, pinned_array_like, stream, synchronize, to_device)
from .devicearray import DeviceNDArray, Event, Stream  # noqa: F401
from .kernels import reduction as _reduction, transpose as _transpose  # noqa: F401
from .kernels.reduction import Reduce

reduce = Reduce


def stats() -> dict:
    """Counters of this process: kernels launched by the library so far, and whether
    the C-ABI calls are wrapped in NVTX ranges (``B2K_NVTX=1``)."""
    import os
    return {"kernel_launches": _lib.launch_count(), "nvtx_ranges": os.environ.get("B2K_NVTX", "") not in ("", "0"),
            "library": _lib.LIB_PATH}

__version__ = "0.1.0"
