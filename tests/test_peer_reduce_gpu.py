"""The reduce kernel's in-kernel cross-GPU combine (``b2k_reduce_peer``).

On one GPU the exchange is exercised without ever making a kernel wait for
another launch: a peer's mailbox is a second local buffer and the peer's value
is written into this rank's mailbox *before* the kernel starts.  The give-up path
is checked by letting a short wait run out on a word that nothing writes (the
kernel records a status and returns; the context stays usable).  A value travels
as 64-bit words {low 32 bits of the epoch | 32 bits of payload}.  With two or
more GPUs, real ranks in separate processes run the fused path end to end."""
import ctypes
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch

import oracle
import numba_cuda_b200 as cuda
from numba_cuda_b200 import _lib, sharded
from numba_cuda_b200.devicearray import _ForeignBuffer

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Mailbox:
    def __init__(self):
        L = _lib.lib()
        p = ctypes.c_void_p()
        _lib.check(L.b2k_peer_mailbox_create(ctypes.byref(p)))
        self.ptr = p.value
        self.words = _ForeignBuffer(self.ptr, int(L.b2k_peer_mailbox_bytes()), self).tensor.view(torch.int64)

    def slot(self, epoch, writer):
        return 2 * ((epoch & 1) * _lib.lib().b2k_peer_max_world() + writer)

    def close(self):
        _lib.lib().b2k_peer_mailbox_destroy(self.ptr)


def new_status():
    return torch.zeros(3, dtype=torch.int64, device="cuda")


def deliver(box, epoch, writer, bits):
    """What rank `writer`'s kernel stores into `box` for call `epoch`."""
    s = box.slot(epoch, writer)
    tag = ((epoch % 0xFFFFFFFF) + 1) << 32
    for k, part in enumerate((bits & 0xFFFFFFFF, (bits >> 32) & 0xFFFFFFFF)):
        word = tag | part
        box.words[s + k] = word - (1 << 64) if word >= (1 << 63) else word


def delivered(box, epoch, writer, itemsize):
    s = box.slot(epoch, writer)
    w0 = int(box.words[s].item()) & (2 ** 64 - 1)
    assert w0 >> 32 == (epoch % 0xFFFFFFFF) + 1
    bits = w0 & 0xFFFFFFFF
    if itemsize > 4:
        w1 = int(box.words[s + 1].item()) & (2 ** 64 - 1)
        assert w1 >> 32 == (epoch % 0xFFFFFFFF) + 1
        bits |= (w1 & 0xFFFFFFFF) << 32
    return bits


def call_peer(op, code, x, init, boxes, world, rank, epoch, timeout_ns, status, scratch, out, flags=0):
    L = _lib.lib()
    ptrs = (ctypes.c_void_p * world)(*[b.ptr for b in boxes])
    rc = L.b2k_reduce_peer(op, code, x.data_ptr(), x.numel(), init.ctypes.data, out.data_ptr(), scratch.data_ptr(),
                           scratch.numel(), ptrs, world, rank, epoch, timeout_ns, status.data_ptr(), flags,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.b2k_last_error()


def test_world_of_one_equals_plain_reduce():
    L = _lib.lib()
    box = Mailbox()
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    status = new_status()
    x = torch.randint(-2 ** 31, 2 ** 31 - 1, (1 << 20,), dtype=torch.int32, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    init = np.array([-5], dtype=np.int32)
    for epoch in (1, 2, 3, 4, 5):
        for flags in (0, _lib.REDUCE_INPUT_READY):
            call_peer(_lib.MAX, _lib.I32, x, init, [box], 1, 0, epoch, 0, status, scratch, out, flags)
            assert out.item() == max(int(x.max().item()), -5) and status[0].item() == 0
            assert 0 <= (status[2] - status[1]).item() < 1_000_000     # both stamps written, microseconds apart
    box.close()


@pytest.mark.parametrize("op,code,tdt,name", [(_lib.MAX, _lib.I32, torch.int32, "max"),
                                              (_lib.ADD, _lib.F64, torch.float64, "add"),
                                              (_lib.ADD, _lib.I8, torch.int8, "add"),
                                              (_lib.MIN, _lib.F32, torch.float32, "min")])
def test_fold_with_a_value_that_already_arrived(op, code, tdt, name):
    L = _lib.lib()
    mine, theirs = Mailbox(), Mailbox()         # rank 0's mailbox, and a stand-in for rank 1's memory
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    status = new_status()
    ndt = np.dtype(str(tdt).replace("torch.", ""))
    if tdt.is_floating_point:
        x = torch.rand(100003, dtype=tdt, device="cuda")
    else:
        info = torch.iinfo(tdt)
        x = torch.randint(info.min, info.max, (100003,), dtype=tdt, device="cuda")
    out = torch.zeros(1, dtype=tdt, device="cuda")
    init = np.array([3], dtype=ndt)
    peer_value = np.array([7], dtype=ndt)
    for epoch in (1, 2, 3, 4):                  # both parities, reuse without any reset
        bits = np.zeros(1, dtype=np.uint64)
        bits.view(np.uint8)[: ndt.itemsize] = peer_value.view(np.uint8)
        deliver(mine, epoch, 1, int(bits[0]))
        torch.cuda.synchronize()
        call_peer(op, code, x, init, [mine, theirs], 2, 0, epoch, 0, status, scratch, out)
        local = oracle.fold(x.cpu().numpy(), name, sharded.op_identity(op, ndt))
        want = sharded.host_fold(op, np.array([local, peer_value[0]], dtype=ndt), init[0])
        got = out.cpu().numpy()[0]
        if ndt.kind == "f" and name == "add":
            assert abs(got - want) <= (1e-12 if ndt == np.float64 else 1e-5) * abs(want)
        else:
            assert got == want
        assert status[0].item() == 0
        # this rank published its own value, under the epoch, into the peer's mailbox
        raw = np.array([delivered(theirs, epoch, 0, ndt.itemsize)], dtype=np.uint64)
        pub = raw.view(np.uint8)[: ndt.itemsize].view(ndt)[0]
        assert pub == local or (ndt.kind == "f" and abs(pub - local) <= 1e-5 * abs(local))
    mine.close(); theirs.close()


def test_wait_that_runs_out_sets_status_and_returns():
    L = _lib.lib()
    mine, theirs = Mailbox(), Mailbox()
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    status = new_status()
    x = torch.ones(1000, dtype=torch.int32, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    init = np.array([0], dtype=np.int32)
    # nothing ever writes rank 1's word: the wait gives up after 2 ms
    call_peer(_lib.ADD, _lib.I32, x, init, [mine, theirs], 2, 0, 1, 2_000_000, status, scratch, out)
    torch.cuda.synchronize()
    assert status[0].item() == 1
    assert (status[2] - status[1]).item() >= 2_000_000
    # a word of another epoch (a call two steps on, same slot) does not count either
    deliver(mine, 4, 1, 99)
    torch.cuda.synchronize()
    status.zero_()
    call_peer(_lib.ADD, _lib.I32, x, init, [mine, theirs], 2, 0, 2, 2_000_000, status, scratch, out)
    torch.cuda.synchronize()
    assert status[0].item() == 1
    # a call whose scratch set was never released by the call two epochs back (epoch 5 after
    # 1 and 2: nothing ran as 3) gives up on that too, and says which wait it was
    deliver(mine, 5, 1, 7)
    torch.cuda.synchronize()
    status.zero_()
    call_peer(_lib.ADD, _lib.I32, x, init, [mine, theirs], 2, 0, 5, 2_000_000, status, scratch, out)
    torch.cuda.synchronize()
    assert status[0].item() == 2 and out.item() == 1007      # the fold itself still completed
    # the context is intact and the scratch reusable
    status.zero_()
    plain = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert L.b2k_reduce(_lib.ADD, _lib.I32, x.data_ptr(), x.numel(), init.ctypes.data, plain.data_ptr(),
                        scratch.data_ptr(), scratch.numel(), torch.cuda.current_stream().cuda_stream) == 0
    assert plain.item() == 1000
    mine.close(); theirs.close()


def test_epochs_across_the_tag_wrap():
    """The 32-bit tag of an epoch is (epoch mod (2^32 - 1)) + 1; a communicator that has made
    four billion calls runs through the wrap.  The scratch is prepared as those calls would
    have left it (the markers of the two sets name the two preceding epochs)."""
    L = _lib.lib()
    mine, theirs = Mailbox(), Mailbox()
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    markers = scratch[64:80].view(torch.int64)
    first = (1 << 32) - 4
    markers[(first - 2) & 1] = first - 2
    markers[(first - 1) & 1] = first - 1
    status = new_status()
    x = torch.arange(1, 5001, dtype=torch.int64, device="cuda")
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    init = np.array([0], dtype=np.int64)
    for epoch in range(first, first + 8):
        deliver(mine, epoch, 1, 1_000_000_000_000 + epoch)          # an 8-byte value: two words
        torch.cuda.synchronize()
        call_peer(_lib.ADD, _lib.I64, x, init, [mine, theirs], 2, 0, epoch, 0, status, scratch, out,
                  _lib.REDUCE_INPUT_READY)
        assert out.item() == 5000 * 5001 // 2 + 1_000_000_000_000 + epoch and status[0].item() == 0
        assert delivered(theirs, epoch, 0, 8) == 5000 * 5001 // 2
    mine.close(); theirs.close()


def test_row_sharded_axis_reduce_in_a_world_of_one():
    full = np.random.default_rng(9).integers(-2 ** 31, 2 ** 31, size=(1000, 70), dtype=np.int32)
    red = sharded.ShardedReduceAxis(lambda a, b: a + b)
    with np.errstate(over="ignore"):
        assert red(full, 0, init=5).copy_to_host().tobytes() == (np.add.reduce(full, axis=0, dtype=np.int32)
                                                                 + np.int32(5)).tobytes()
        assert red(full, 1).copy_to_host().tobytes() == np.add.reduce(full, axis=1, dtype=np.int32).tobytes()


def test_argument_checks():
    L = _lib.lib()
    init = np.zeros(1, dtype=np.int32)
    ptrs = (ctypes.c_void_p * 1)(4096)
    assert L.b2k_reduce_peer(_lib.ADD, _lib.I32, 4096, 4, init.ctypes.data, 8192, 256, 1 << 20, ptrs, 0, 0, 1, 0,
                             4096, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_peer(_lib.ADD, _lib.I32, 4096, 4, init.ctypes.data, 8192, 256, 1 << 20, ptrs, 1, 0, 0, 0,
                             4096, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_peer(_lib.ADD, _lib.I32, 4096, 4, init.ctypes.data, 8192, 256, 40000, ptrs, 1, 0, 1, 0,
                             4096, 0, None) == _lib.ERR_SCRATCH              # needs both halves of the scratch
    assert L.b2k_reduce_peer(_lib.ADD, _lib.I32, 4096, 4, init.ctypes.data, 8192, 256, 1 << 20, ptrs, 17, 0, 1, 0,
                             4096, 0, None) == _lib.ERR_INVALID_ARG
    assert L.b2k_reduce_peer(_lib.ADD, _lib.I32, 4096, 4, init.ctypes.data, 8192, 256, 1 << 20, ptrs, 1, 0, 1, 0,
                             4096, 2, None) == _lib.ERR_INVALID_ARG          # unknown flag
    assert L.b2k_reduce_peer(_lib.ADD, _lib.I32, 4096, 4, init.ctypes.data, 8192, 256, 1 << 20, ptrs, 1, 0, 1, 0,
                             4100, 0, None) == _lib.ERR_ALIGNMENT            # status not 8-byte aligned


# ---- real ranks on separate GPUs ---------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, errors):
    try:
        sys.path.insert(0, ROOT)
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        boxes = sharded.PeerMailboxes()
        cases = [("max", lambda a, b: max(a, b), np.int32, 0), ("add", lambda a, b: a + b, np.float64, 2.5),
                 ("add", lambda a, b: a + b, np.int64, -7), ("min", lambda a, b: min(a, b), np.float32, 1e30),
                 ("xor", lambda a, b: a ^ b, np.uint16, 0)]
        for round_no in range(3):
            for name, fn, dt, init in cases:
                n = 1 << 20
                rng = np.random.default_rng(100 + round_no)
                if np.dtype(dt).kind == "f":
                    whole = rng.standard_normal(n).astype(dt)
                else:
                    info = np.iinfo(dt)
                    whole = rng.integers(info.min, info.max, size=n, dtype=dt, endpoint=True)
                lo, hi = sharded.shard_bounds(n, world, rank)
                fused = sharded.ShardedReduce(fn, peer=boxes)(whole[lo:hi], init=init)
                nccl = sharded.ShardedReduce(fn)(whole[lo:hi], init=init)
                want = oracle.fold(whole, name, init)
                if np.dtype(dt).kind == "f" and name == "add":
                    assert abs(fused - want) <= 1e-12 * np.abs(whole).sum(), (name, dt, fused, want)
                    assert abs(nccl - want) <= 1e-12 * np.abs(whole).sum()
                else:
                    assert fused == want == nccl, (name, dt, fused, nccl, want)
        # a user function outside the op table: partials gathered once, folded on the device
        fn = lambda a, b: (a + b) % 1000003       # noqa: E731
        whole = np.random.default_rng(77).integers(0, 1000003, size=300001, dtype=np.int64)
        lo, hi = sharded.shard_bounds(whole.size, world, rank)
        import functools
        want = functools.reduce(lambda a, b: (a + b) % 1000003, [int(v) for v in whole[::1]], 5)
        for peer in (None, boxes):
            assert sharded.ShardedReduce(fn, peer=peer)(whole[lo:hi], init=5) == want
        empty_here = whole[:0] if rank == world - 1 else whole[lo:hi]      # one rank has nothing
        want = functools.reduce(lambda a, b: (a + b) % 1000003, [int(v) for v in whole[:sharded.shard_bounds(
            whole.size, world, world - 1)[0]]], 5)
        assert sharded.ShardedReduce(fn)(empty_here, init=5) == want
        # a non-default stream: collectives and copies must follow the kernel on it
        side = cuda.stream()
        x = np.random.default_rng(5).integers(-2 ** 31, 2 ** 31, size=1 << 22, dtype=np.int32)
        lo, hi = sharded.shard_bounds(x.size, world, rank)
        for peer in (None, boxes):
            for _ in range(5):
                assert sharded.ShardedReduce(lambda a, b: max(a, b), peer=peer)(x[lo:hi], init=0, stream=side) == \
                    max(int(x.max()), 0)
        with np.errstate(over="ignore"):
            m = x[: (x.size // 512) * 512].reshape(-1, 512)
            lo, hi = sharded.shard_bounds(m.shape[0], world, rank)
            got = sharded.ShardedReduceAxis(lambda a, b: a + b)(m[lo:hi], 0, stream=side).copy_to_host(stream=side)
            side.synchronize()
            assert got.tobytes() == np.add.reduce(m, axis=0, dtype=np.int32).tobytes()
        # a pipeline of fused reductions whose inputs are all complete beforehand:
        # each reads its shard while the one before finishes its exchange
        from numba_cuda_b200.kernels.reduction import _DTYPE_CODES
        shards = [cuda.to_device(np.random.default_rng(200 + k).integers(-2 ** 31, 2 ** 31, size=1 << 22,
                                                                          dtype=np.int32)[
            slice(*sharded.shard_bounds(1 << 22, world, rank))]) for k in range(8)]
        outs = cuda.device_array(8, dtype=np.int32)
        ident = np.array([-2 ** 31], dtype=np.int32)
        torch.cuda.synchronize()
        dist.barrier()
        for k, sh in enumerate(shards):
            boxes.reduce(_lib.MAX, _DTYPE_CODES[np.dtype(np.int32)], sh._ptr, sh.size, ident, outs[k:k + 1]._ptr,
                         0, input_ready=True)
        got = outs.copy_to_host()
        boxes.check(agree=True)
        want = [int(np.random.default_rng(200 + k).integers(-2 ** 31, 2 ** 31, size=1 << 22, dtype=np.int32).max())
                for k in range(8)]
        assert got.tolist() == want
        assert 0 <= boxes.exchange_ns() < 50_000_000
        # the same pipeline through the Python wrapper: launches only, results stay on the device
        fused = sharded.ShardedReduce(lambda a, b: max(a, b), peer=boxes)
        outs2 = cuda.device_array(8, dtype=np.int32)
        for k, sh in enumerate(shards):
            assert fused(sh, init=-2 ** 31, res=outs2[k:k + 1], input_ready=True) is None
        got2 = outs2.copy_to_host()
        boxes.check(agree=True)
        assert got2.tolist() == want
        with pytest.raises(NotImplementedError):
            sharded.ShardedReduce(lambda a, b: max(a, b))(shards[0], res=outs2[:1])
        # a row-sharded matrix reduced along both axes
        full = np.random.default_rng(9).integers(-2 ** 31, 2 ** 31, size=(4099, 260), dtype=np.int32)
        lo, hi = sharded.shard_bounds(full.shape[0], world, rank)
        for fn, ufunc in ((lambda a, b: a + b, np.add), (lambda a, b: max(a, b), np.maximum)):
            red = sharded.ShardedReduceAxis(fn)
            cols = red(full[lo:hi], 0, init=3).copy_to_host()
            with np.errstate(over="ignore"):
                want = ufunc(ufunc.reduce(full, axis=0, dtype=np.int32), np.int32(3), dtype=np.int32)
                want_rows = ufunc(ufunc.reduce(full[lo:hi], axis=1, dtype=np.int32), np.int32(3), dtype=np.int32)
            assert cols.tobytes() == want.tobytes()
            assert red(full[lo:hi], 1, init=3).copy_to_host().tobytes() == want_rows.tobytes()
        dist.barrier()
        boxes.close()
        dist.destroy_process_group()
    except Exception:
        errors.put((rank, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_combine_across_real_ranks():
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
    if not errors.empty():
        rank, tb = errors.get()
        pytest.fail(f"rank {rank} failed:\n{tb}")
    assert all(p.exitcode == 0 for p in procs)
