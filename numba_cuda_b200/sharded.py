"""Contiguous-shard multi-GPU wrappers (one process per GPU, torch.distributed).

The reference has no distributed layer; this module is the new part of the
drop-in.  Reduce, RNG and casts partition by contiguous index range:

* reduce: every rank folds its shard with the single-launch kernel; the partials
  are combined either inside that kernel over NVLink peer memory
  (``PeerMailboxes``) or by ONE collective on a one-element buffer --
  ``all_reduce`` (sum / product / max / min) where the backend carries the dtype,
  else an ``all_gather`` of the G partials folded locally; for a traced user
  function the gathered partials are folded on the device by the same run-time
  compiled kernel.  ``init`` is folded in once, after the combine;
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


def _on_stream(tensor: torch.Tensor, stream):
    """Context in which torch orders work on ``tensor`` behind ``stream``: the
    collectives and copies of this module must follow the kernel that was launched
    on the caller's stream, and torch orders them against ITS current stream."""
    import contextlib
    if not tensor.is_cuda:
        return contextlib.nullcontext()
    from .devicearray import _torch_stream
    return torch.cuda.stream(_torch_stream(stream))


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


def combine_partials(partial: torch.Tensor, op: int, dtype, group=None, stream=0) -> torch.Tensor:
    """Combine one-element per-rank partials (raw ``uint8`` bytes of ``dtype``,
    on whatever device the process group works with) into the same buffer on
    every rank.  One collective call, ordered behind ``stream``."""
    dist, world, _ = _world(group)
    dtype = np.dtype(dtype)
    if world == 1:
        return partial
    with _on_stream(partial, stream):
        if op in (_lib.ADD, _lib.MUL, _lib.MAX, _lib.MIN) and dtype in _NATIVE_ALLREDUCE_DTYPES:
            typed = partial.view(_NATIVE_ALLREDUCE_DTYPES[dtype])
            red = {_lib.ADD: dist.ReduceOp.SUM, _lib.MUL: dist.ReduceOp.PRODUCT,
                   _lib.MAX: dist.ReduceOp.MAX, _lib.MIN: dist.ReduceOp.MIN}[op]
            dist.all_reduce(typed, op=red, group=group)
            return partial
        gathered = gather_partial_rows(partial, group=group, stream=stream)
        host = gathered.cpu().numpy().reshape(-1).view(dtype)
        folded = host_fold(op, host, op_identity(op, dtype))
        partial.copy_(torch.from_numpy(np.array([folded], dtype=dtype).view(np.uint8)))
    return partial


class PeerMailboxes:
    """The mailboxes of one communicator for the in-kernel cross-GPU combine
    (``b2k_reduce_peer``): this rank's own mailbox plus a mapping of every
    peer's, exchanged as IPC handles over the process group at construction.
    All ranks of the group must construct it together and must then call
    ``reduce`` in the same order (the call counter is the epoch the kernels
    match on).  Single node, at most ``b2k_peer_max_world()`` ranks.

    A rank whose wait runs out (``timeout_s``; a peer delayed by a long copy, by
    first-call module loading, or gone) writes only ``init`` and reports it through
    ``check``, while ranks whose waits succeeded hold the real result: after a
    timeout the ranks DISAGREE.  ``check(agree=True)`` makes the decision common
    (one small all-reduce of the status over the process group)."""

    def __init__(self, group=None, world_size=None, rank=None, timeout_s: float = 2.0):
        import ctypes
        L = _lib.lib()
        dist, world, my_rank = _world(group)
        if world_size is not None:
            world, my_rank = int(world_size), int(rank)
        if world > L.b2k_peer_max_world():
            raise ValueError(f"at most {L.b2k_peer_max_world()} ranks")
        self.world, self.rank, self.group = world, my_rank, group
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        own = ctypes.c_void_p()
        _lib.check(L.b2k_peer_mailbox_create(ctypes.byref(own)))
        self._own = own.value
        self._opened = []
        ptrs = [None] * world
        ptrs[my_rank] = self._own
        if world > 1 and dist is not None:
            handle = ctypes.create_string_buffer(int(L.b2k_peer_handle_bytes()))
            _lib.check(L.b2k_peer_mailbox_export(self._own, handle))
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r, h in enumerate(handles):
                if r == my_rank:
                    continue
                peer = ctypes.c_void_p()
                _lib.check(L.b2k_peer_mailbox_open(ctypes.create_string_buffer(h, len(h)), ctypes.byref(peer)))
                ptrs[r] = peer.value
                self._opened.append(peer.value)
            dist.barrier(group=group)
        self._ptrs = (ctypes.c_void_p * world)(*ptrs)
        # [0] timed-out flag, [1] local fold done (ns), [2] all peers seen (ns)
        self._status = torch.zeros(3, dtype=torch.int64, device="cuda")
        # ONE scratch buffer per communicator: its two ticket/partial sets alternate with the
        # call counter, so up to two calls may be in flight (on one stream or on several)
        self._scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
        torch.cuda.current_stream().synchronize()          # zero-filled before any stream uses it
        self._launch = L.b2k_reduce_peer
        self._scratch_ptr, self._scratch_bytes = self._scratch.data_ptr(), self._scratch.numel()
        self._status_ptr = self._status.data_ptr()

    def reduce(self, op, dtype_code, x_ptr, n, init_host, out_ptr, stream=0, input_ready=False):
        """One collective call: launches the fused kernel on this rank.  The epoch
        advances only when the launch was accepted, so an argument error on one rank
        does not put it out of step with the others.  ``init_host`` is a one-element
        NumPy array or the address of one; ``stream`` a stream object or its handle
        (plain integers keep the per-call cost of a tight loop of launches down)."""
        if not isinstance(stream, int):
            from .devicearray import stream_ptr
            stream = stream_ptr(stream)
        init_ptr = init_host if isinstance(init_host, int) else init_host.ctypes.data
        epoch = self.epoch + 1
        rc = self._launch(op, dtype_code, x_ptr, n, init_ptr, out_ptr, self._scratch_ptr, self._scratch_bytes,
                          self._ptrs, self.world, self.rank, epoch, self.timeout_ns, self._status_ptr,
                          _lib.REDUCE_INPUT_READY if input_ready else 0, stream)
        if rc:
            _lib.check(rc)
        self.epoch = epoch

    def exchange_ns(self) -> int:
        """What the exchange of the most recent call cost this rank, from the GPU's
        nanosecond timer: local fold complete -> last peer value seen (launch skew
        between the ranks included).  Synchronises."""
        s = self._status.cpu()
        return int(s[2] - s[1])

    def check(self, agree: bool = False):
        """Raise if any earlier call on this rank gave up waiting for a peer
        (synchronises).  With ``agree=True`` the ranks first take the maximum of
        their flags over the process group, so that either all raise or none."""
        flag = self._status[:1].clone()
        if agree and self.world > 1:
            dist, _, _ = _world(self.group)
            if dist is not None:
                dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if int(flag.item()) != 0:
            self._status[:1].zero_()
            raise RuntimeError("a peer's partial result did not arrive within the time limit; "
                               "the ranks may hold different results for that call")

    def close(self):
        L = _lib.lib()
        for p in self._opened:
            L.b2k_peer_mailbox_close(p)
        self._opened = []
        if self._own:
            L.b2k_peer_mailbox_destroy(self._own)
            self._own = None


class ShardedReduce:
    """``cuda.reduce`` over an array that is sharded by contiguous range across
    the ranks of a process group.  Call on every rank with the local shard; the
    full result (with ``init`` folded in once) is returned on every rank.

    With ``peer=PeerMailboxes(...)`` the combine happens inside the reduce kernel
    over NVLink peer memory (one launch per rank, no library collective);
    without it, one NCCL collective on a one-element buffer follows the kernel.
    A user function outside the precompiled table (a traced expression) always
    takes the collective route: one all-gather of the partials, which the same
    run-time compiled kernel then folds on the device."""

    def __init__(self, functor, peer: "PeerMailboxes | None" = None):
        self._functor = functor
        self._local = Reduce(functor)
        self._peer = peer

    def __call__(self, local_arr, init=0, stream=0, group=None, res=None, input_ready=False):
        """The reduction of the whole array, on every rank.  With ``res`` (a device array
        of the shard's dtype; fused combine only) the call only launches: the result lands
        in ``res[0]`` in stream order, nothing is copied back and ``None`` is returned --
        call ``peer.check()`` once the stream has been synchronised.  ``input_ready`` as
        in ``Reduce.__call__``: a run of such launches over resident shards overlaps."""
        from .api import auto_device, device_array
        from .kernels.reduction import _DTYPE_CODES
        dtype = np.dtype(local_arr.dtype)
        op = self._local._compile(dtype)
        if res is not None and (isinstance(op, str) or self._peer is None):
            raise NotImplementedError("res= needs a table op and the fused combine (peer=PeerMailboxes())")
        if isinstance(op, str):
            return self._traced(local_arr, dtype, init, stream, group)
        if self._peer is not None:
            darr, staged = auto_device(local_arr, stream=stream)
            if darr.ndim != 1 or (darr.size and darr.strides[0] != dtype.itemsize):
                raise ValueError("the shard must be a contiguous 1-D array")
            init_host = np.array([init], dtype=dtype)
            if res is not None:
                dres, _ = auto_device(res, stream=stream)
                if dres.dtype != dtype or dres.size < 1:
                    raise TypeError("res must hold one item of the shard's dtype")
                self._peer.reduce(op, _DTYPE_CODES[dtype], darr._ptr, darr.size, init_host, dres._ptr, stream,
                                  input_ready=bool(input_ready) and not staged)
                return None
            slot = device_array(1, dtype=dtype, stream=stream)
            self._peer.reduce(op, _DTYPE_CODES[dtype], darr._ptr, darr.size, init_host, slot._ptr, stream)
            result = slot.copy_to_host()[0]
            self._peer.check()
            return result
        ident = op_identity(op, dtype)
        slot = device_array(1, dtype=dtype, stream=stream)
        if local_arr.size:
            self._local(local_arr, res=slot, init=ident, stream=stream)
        else:
            slot.copy_to_device(np.array([ident], dtype=dtype), stream=stream)
        combined = combine_partials(slot._bytes_view(), op, dtype, group=group, stream=stream)
        with _on_stream(combined, stream):
            host = combined.cpu().numpy().view(dtype)
        return host_fold(op, host, dtype.type(init))

    def _traced(self, local_arr, dtype, init, stream, group):
        """A user function with no identity element: every rank with a non-empty shard
        contributes its partial (no ``init`` in it) plus a presence mark; after one
        all-gather the partials that are there are folded, with ``init``, by the same
        kernel that folded the shards."""
        from .api import device_array
        record = device_array(16, dtype=np.uint8, stream=stream)          # [value | present]
        mark = np.zeros(16, dtype=np.uint8)
        if local_arr.size:
            mark[8] = 1
            record.copy_to_device(mark, stream=stream)
            self._local(local_arr, res=record.view(dtype)[:1], stream=stream, _fold_init=False)
        else:
            record.copy_to_device(mark, stream=stream)
        rows = gather_partial_rows(record._bytes_view(), group=group, stream=stream)
        return fold_gathered(rows, dtype, init, lambda values: self._local(values, init=init, stream=stream),
                             stream=stream)


def fold_gathered(rows: torch.Tensor, dtype, init, fold, stream=0):
    """``rows`` is the ``[world, 16]`` stack of per-rank records ``[value | present]``.
    The values that are present go, in rank order, to ``fold`` (a callable that
    reduces a 1-D array of ``dtype`` with the user's function and ``init``); with
    none present the result is ``init``."""
    from .devicearray import DeviceNDArray
    dtype = np.dtype(dtype)
    with _on_stream(rows, stream):
        present = rows[:, 8].cpu().numpy() != 0
        if not present.any():
            return dtype.type(init)
        keep = torch.from_numpy(np.flatnonzero(present)).to(rows.device)
        values = rows[:, :dtype.itemsize].index_select(0, keep).contiguous().reshape(-1)
    if values.is_cuda:
        count = int(present.sum())
        values = DeviceNDArray((count,), (dtype.itemsize,), dtype, stream=stream, gpu_data=(values, 0))
    else:
        values = values.numpy().view(dtype)
    return fold(values)


def gather_partial_rows(partial: torch.Tensor, group=None, stream=0) -> torch.Tensor:
    """All ranks' partial result rows (raw ``uint8`` bytes, same length on every
    rank) stacked into a ``[world, nbytes]`` tensor on every rank: ONE collective,
    ordered behind ``stream``."""
    dist, world, _ = _world(group)
    if world == 1:
        return partial.reshape(1, -1)
    with _on_stream(partial, stream):
        stacked = torch.empty(world * partial.numel(), dtype=torch.uint8, device=partial.device)
        if partial.is_cuda:
            dist.all_gather_into_tensor(stacked, partial.contiguous(), group=group)
        else:
            dist.all_gather(list(stacked.view(world, -1).unbind(0)), partial.contiguous(), group=group)
    return stacked.view(world, -1)


class ShardedReduceAxis:
    """``Reduce(fn).along_axis`` over a matrix whose ROWS are sharded by contiguous
    range across the ranks of a process group.  Axis 1 (one result per row) needs
    no exchange: every rank returns the results of its own rows.  Axis 0 (one result
    per column): every rank reduces its rows, one all-gather stacks the partial rows
    and the stack is reduced along axis 0 by the same kernel, which also folds
    ``init`` in once; the full result is returned on every rank."""

    def __init__(self, functor):
        self._local = Reduce(functor)

    def __call__(self, local_rows, axis, init=0, stream=0, group=None):
        from .api import auto_device
        from .devicearray import DeviceNDArray, _c_strides
        dtype = np.dtype(local_rows.dtype)
        op = self._local._compile(dtype)
        if isinstance(op, str):
            raise NotImplementedError("sharded axis-wise reduction supports the precompiled table ops only")
        if axis % 2 == 1:
            return self._local.along_axis(local_rows, 1, init=init, stream=stream)
        darr, _ = auto_device(local_rows, stream=stream)
        partial = self._local.along_axis(darr, 0, init=op_identity(op, dtype), stream=stream)
        stacked = gather_partial_rows(partial._bytes_view(), group=group, stream=stream)
        world, cols = stacked.shape[0], partial.shape[0]
        rows = DeviceNDArray((world, cols), _c_strides((world, cols), dtype.itemsize), dtype, stream=stream,
                             gpu_data=(stacked.view(-1), 0))
        return self._local.along_axis(rows, 0, init=init, stream=stream)


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
def sharded_cast(src_local, src_format, dst_format, out=None, saturate=1, stream=0, rounding=0):
    """Cast this rank's contiguous shard (no communication); ``rounding`` as in
    ``casts.cast`` (the directed modes, the integer sides)."""
    from .casts import cast
    return cast(src_local, src_format, dst_format, out=out, saturate=saturate, stream=stream, rounding=rounding)


__all__ = ["PeerMailboxes", "ShardedReduceAxis", "gather_partial_rows", "fold_gathered", "shard_bounds", "op_identity", "host_fold", "combine_partials", "ShardedReduce",
           "create_sharded_xoroshiro128p_states", "sharded_cast", "op_name"]
