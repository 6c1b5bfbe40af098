"""ctypes binding of ``libb2k.so`` (the C ABI declared in ``include/b2k.h``).

There is no CPU fallback: if the library is missing or does not load, every
entry point raises.  Build it with ``python -m numba_cuda_b200._build``.
"""
from __future__ import annotations

import ctypes
import functools
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
#: B2K_LIBRARY names another build of the library (comparing two builds side by side)
LIB_PATH = os.environ.get("B2K_LIBRARY") or os.path.join(_HERE, "csrc", "libb2k.so")

# enums of include/b2k.h
I8, I16, I32, I64, U8, U16, U32, U64, F32, F64 = range(10)
ADD, MUL, MAX, MIN, AND, OR, XOR = range(7)
FMT_F32, FMT_BF16, FMT_E4M3, FMT_E5M2, FMT_F64, FMT_F16, FMT_E8M0 = range(7)
FMT_I8, FMT_I16, FMT_I32, FMT_I64, FMT_U8, FMT_U16, FMT_U32, FMT_U64, FMT_BOOL = range(7, 16)
ROUND_NEAREST, ROUND_ZERO, ROUND_POS_INF, ROUND_MIN_INF = range(4)
UNIFORM_F32, UNIFORM_F64, NORMAL_F32, NORMAL_F64 = range(4)

REDUCE_INPUT_READY = 1

ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_SCRATCH, ERR_TOO_LARGE = -1, -2, -3, -4, -5

#: every symbol include/b2k.h declares, with (restype, argtypes)
_vp, _i64, _u64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_int
SIGNATURES = {
    "b2k_version": (_i32, []),
    "b2k_last_error": (ctypes.c_char_p, []),
    "b2k_launch_count": (_i64, []),
    "b2k_reduce_scratch_bytes": (_i64, []),
    "b2k_reduce": (_i32, [_i32, _i32, _vp, _i64, _vp, _vp, _vp, _i64, _vp]),
    "b2k_reduce_ex": (_i32, [_i32, _i32, _vp, _i64, _vp, _vp, _vp, _i64, ctypes.c_uint, _vp]),
    "b2k_reduce_expr": (_i32, [ctypes.c_char_p, _i32, _vp, _i64, _vp, _vp, _vp, _i64, _vp]),
    "b2k_reduce_noalloc_max_elements": (_i64, []),
    "b2k_reduce_noalloc": (_i32, [_i32, _i32, _vp, _i64, _vp, _vp, _vp]),
    "b2k_peer_mailbox_bytes": (_i64, []),
    "b2k_peer_handle_bytes": (_i64, []),
    "b2k_peer_max_world": (_i32, []),
    "b2k_peer_mailbox_create": (_i32, [ctypes.POINTER(_vp)]),
    "b2k_peer_mailbox_destroy": (_i32, [_vp]),
    "b2k_peer_mailbox_export": (_i32, [_vp, _vp]),
    "b2k_peer_mailbox_open": (_i32, [_vp, ctypes.POINTER(_vp)]),
    "b2k_peer_mailbox_close": (_i32, [_vp]),
    "b2k_reduce_peer": (_i32, [_i32, _i32, _vp, _i64, _vp, _vp, _vp, _i64, ctypes.POINTER(_vp), _i32, _i32,
                               _u64, _u64, _vp, ctypes.c_uint, _vp]),
    "b2k_transpose2d": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "b2k_transpose_wait_timeouts": (_i32, [ctypes.POINTER(ctypes.c_uint)]),
    "b2k_reduce_axis_scratch_bytes": (_i64, [_i64, _i64, _i32, _i32]),
    "b2k_reduce_axis": (_i32, [_i32, _i32, _vp, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _i64, _vp]),
    "b2k_reduce_cols_batched_scratch_bytes": (_i64, [_i64, _i64, _i64, _i32]),
    "b2k_reduce_cols_batched": (_i32, [_i32, _i32, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "b2k_assign": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _i64, _vp]),
    "b2k_fill": (_i32, [_vp, _i32, _vp, _vp, _vp, _i64, _vp]),
    "b2k_xoroshiro128p_tables_bytes": (_i64, []),
    "b2k_xoroshiro128p_build_tables": (_i32, [_vp, _i64, _vp]),
    "b2k_xoroshiro128p_init": (_i32, [_vp, _i64, _u64, _u64, _vp, _i64, _vp]),
    "b2k_xoroshiro128p_fill": (_i32, [_vp, _i64, _i32, _vp, _i64, _i32, _vp, _i64, _vp]),
    "b2k_cast": (_i32, [_i32, _i32, _i32, _vp, _vp, _i64, _vp]),
    "b2k_cast_ex": (_i32, [_i32, _i32, _i32, _i32, _vp, _vp, _i64, _vp]),
}
class B2KError(RuntimeError):
    """A libb2k call failed; ``status`` is the ABI status (negative = argument
    error found on the host, positive = a cudaError_t)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libb2k status {status}: {message}")
        self.status = status


@functools.lru_cache(maxsize=None)
def lib() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: numba_cuda_b200 has no CPU fallback. "
            "Build it with `python -m numba_cuda_b200._build` (needs nvcc).")
    L = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def check(status: int) -> None:
    """Raise for a non-zero ABI status."""
    if status == 0:
        return
    msg = lib().b2k_last_error().decode("utf-8", "replace")
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    if status in (ERR_INVALID_ARG, ERR_ALIGNMENT, ERR_SCRATCH, ERR_TOO_LARGE):
        raise ValueError(msg)
    raise B2KError(status, msg)


def launch_count() -> int:
    return int(lib().b2k_launch_count())
