"""Contiguous-shard multi-GPU wrappers (one process per GPU, torch.distributed).

The reference has no distributed layer; this module is the new part of the
drop-in.  Reduce, RNG and casts partition by contiguous index range:

* reduce: every rank folds its shard with the single-launch kernel, then ONE
  collective on a one-element buffer combines the partials -- ``all_reduce``
  (sum / product / max / min) where the backend carries the dtype, else an
  ``all_gather`` of the G partials folded locally.  ``init`` is folded in once,
  after the collective;
* RNG: rank k creates states ``[lo_k, hi_k)`` with
  ``subsequence_start + lo_k``, so the concatenation over ranks equals the
  single-GPU array, and fills only its rows -- no exchange;
* casts: contiguous ranges aligned to 16 elements -- no exchange.

The host logic (bounds, identities, the combine) runs on any backend, so it is
tested with ``gloo`` on CPU tensors.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from .kernels.reduction import OP_NAMES, Reduce, classify_functor


# ------------------------------------------------------------------ partitioning
def shard_bounds(n: int, world_size: int, rank: int, align: int = 1):
    """Half-open item range of ``rank``'s contiguous shard of ``n`` items.
    Every shard but the last holds ``floor(n / world_size)`` items rounded down
    to a multiple of ``align``; the last shard takes the remainder."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    base = (n // world_size) // align * align
    lo = rank * base
    hi = n if rank == world_size - 1 else lo + base
    return lo, hi


def _world(group=None):
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return None, 1, 0
    return dist, dist.get_world_size(group), dist.get_rank(group)


# ------------------------------------------------------------------ reduce
def op_identity(op: int, dtype):
    """The value that leaves ``op`` unchanged, as a NumPy scalar of ``dtype``."""
    dtype = np.dtype(dtype)
    t = dtype.type
    if op in (_lib.ADD, _lib.OR, _lib.XOR):
        return t(0)
    if op == _lib.MUL:
        return t(1)
    if op == _lib.AND:
        return t(np.iinfo(dtype).max) if dtype.kind == "u" else t(-1)
    if op == _lib.MAX:
        return t(-np.inf) if dtype.kind == "f" else t(np.iinfo(dtype).min)
    if op == _lib.MIN:
        return t(np.inf) if dtype.kind == "f" else t(np.iinfo(dtype).max)
    raise ValueError(f"unknown op {op}")


def host_fold(op: int, values: np.ndarray, init):
    """Fold a short host array with a table op (wrap-around for integers)."""
    dtype = values.dtype
    acc = dtype.type(init)
    with np.errstate(over="ignore"):
        for v in values:
            if op == _lib.ADD:
                acc = dtype.type(acc + v)
            elif op == _lib.MUL:
                acc = dtype.type(acc * v)
            elif op == _lib.MAX:
                acc = v if v > acc else acc
            elif op == _lib.MIN:
                acc = v if v < acc else acc
            elif op == _lib.AND:
                acc = dtype.type(acc & v)
            elif op == _lib.OR:
                acc = dtype.type(acc | v)
            else:
                acc = dtype.type(acc ^ v)
    return acc


_NATIVE_ALLREDUCE_DTYPES = {np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
                            np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64,
                            np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8}


def combine_partials(partial: torch.Tensor, op: int, dtype, group=None) -> torch.Tensor:
    """Combine one-element per-rank partials (raw ``uint8`` bytes of ``dtype``,
    on whatever device the process group works with) into the same buffer on
    every rank.  One collective call."""
    dist, world, _ = _world(group)
    dtype = np.dtype(dtype)
    if world == 1:
        return partial
    if op in (_lib.ADD, _lib.MUL, _lib.MAX, _lib.MIN) and dtype in _NATIVE_ALLREDUCE_DTYPES:
        typed = partial.view(_NATIVE_ALLREDUCE_DTYPES[dtype])
        red = {_lib.ADD: dist.ReduceOp.SUM, _lib.MUL: dist.ReduceOp.PRODUCT,
               _lib.MAX: dist.ReduceOp.MAX, _lib.MIN: dist.ReduceOp.MIN}[op]
        dist.all_reduce(typed, op=red, group=group)
        return partial
    gathered = torch.empty(world * partial.numel(), dtype=torch.uint8, device=partial.device)
    dist.all_gather_into_tensor(gathered, partial, group=group) if partial.is_cuda else \
        dist.all_gather(list(gathered.view(world, -1).unbind(0)), partial, group=group)
    host = gathered.cpu().numpy().view(dtype)
    folded = host_fold(op, host, op_identity(op, dtype))
    partial.copy_(torch.from_numpy(np.array([folded], dtype=dtype).view(np.uint8)))
    return partial


class ShardedReduce:
    """``cuda.reduce`` over an array that is sharded by contiguous range across
    the ranks of a process group.  Call on every rank with the local shard; the
    full result (with ``init`` folded in once) is returned on every rank."""

    def __init__(self, functor):
        self._functor = functor
        self._local = Reduce(functor)

    def __call__(self, local_arr, init=0, stream=0, group=None):
        from .api import device_array
        dtype = np.dtype(local_arr.dtype)
        op = classify_functor(self._functor, dtype) if local_arr.size else self._local._compile(dtype)
        ident = op_identity(op, dtype)
        slot = device_array(1, dtype=dtype, stream=stream)
        if local_arr.size:
            self._local(local_arr, res=slot, init=ident, stream=stream)
        else:
            slot.copy_to_device(np.array([ident], dtype=dtype), stream=stream)
        combined = combine_partials(slot._bytes_view(), op, dtype, group=group)
        host = combined.cpu().numpy().view(dtype)
        return host_fold(op, host, dtype.type(init))


def op_name(op: int) -> str:
    return OP_NAMES[op]


# ------------------------------------------------------------------ RNG
def create_sharded_xoroshiro128p_states(n_total, seed, subsequence_start=0, stream=0, group=None,
                                        world_size=None, rank=None):
    """This rank's slice of ``create_xoroshiro128p_states(n_total, seed,
    subsequence_start)``; returns ``(states, lo, hi)``."""
    from .random import create_xoroshiro128p_states
    if world_size is None or rank is None:
        _, world_size, rank = _world(group)
    lo, hi = shard_bounds(int(n_total), world_size, rank)
    states = create_xoroshiro128p_states(hi - lo, seed, subsequence_start=int(subsequence_start) + lo,
                                         stream=stream)
    return states, lo, hi


# ------------------------------------------------------------------ casts
def sharded_cast(src_local, src_format, dst_format, out=None, saturate=1, stream=0):
    """Cast this rank's contiguous shard (no communication)."""
    from .casts import cast
    return cast(src_local, src_format, dst_format, out=out, saturate=saturate, stream=stream)


__all__ = ["shard_bounds", "op_identity", "host_fold", "combine_partials", "ShardedReduce",
           "create_sharded_xoroshiro128p_states", "sharded_cast", "op_name"]
