"""Multi-rank host logic on CPU: two `gloo` ranks exercise the partition
bounds, the one-collective combine of reduce partials and the RNG / cast
sharding rules.  The per-shard arithmetic is done by the CPU oracle here (the
CUDA kernels are checked against the same oracle in the gpu tests)."""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, errors):
    try:
        import datetime
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
        if fn_name.startswith("_fail_"):
            globals()[fn_name](rank, world)
            return
        globals()[fn_name](rank, world)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errors.put((rank, traceback.format_exc()))


def _run(fn_name, world=2):
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        if p.is_alive():
            p.kill()
            pytest.fail("rank did not finish")
    if not errors.empty():
        rank, tb = errors.get()
        pytest.fail(f"rank {rank} failed:\n{tb}")
    assert all(p.exitcode == 0 for p in procs)


# ---- bodies run inside each rank ------------------------------------------------
def _body_reduce(rank, world):
    import oracle
    from numba_cuda_b200 import _lib, sharded
    cases = [("max", _lib.MAX, np.int32), ("add", _lib.ADD, np.float64), ("add", _lib.ADD, np.int16),
             ("min", _lib.MIN, np.uint64), ("mul", _lib.MUL, np.float32), ("xor", _lib.XOR, np.uint32),
             ("and", _lib.AND, np.int8), ("or", _lib.OR, np.uint16), ("max", _lib.MAX, np.uint64)]
    for name, op, dt in cases:
        rng = np.random.default_rng(1)
        n = 10007
        if np.dtype(dt).kind == "f":
            x = (rng.random(n) + 0.5).astype(dt) if name == "mul" else rng.standard_normal(n).astype(dt)
            if name == "mul":
                x = x[:64]
                n = 64
        else:
            info = np.iinfo(dt)
            x = rng.integers(info.min, info.max, size=n, dtype=dt, endpoint=True)
        lo, hi = sharded.shard_bounds(n, world, rank)
        ident = sharded.op_identity(op, dt)
        partial = oracle.fold(x[lo:hi], name, ident)       # stands in for the device kernel
        buf = torch.from_numpy(np.array([partial], dtype=dt).view(np.uint8).copy())
        sharded.combine_partials(buf, op, dt)
        init = np.dtype(dt).type(3)
        got = sharded.host_fold(op, buf.numpy().view(dt), init)
        want = oracle.fold(x, name, init)
        if np.dtype(dt).kind == "f":
            assert abs(got - want) <= 1e-5 * abs(want) + 1e-12, (name, dt, got, want)
        else:
            assert got == want, (name, dt, got, want)


def _body_rng(rank, world):
    import oracle
    from numba_cuda_b200 import sharded
    n, seed, start = 1000, 42, 5
    whole = oracle.init_states(n, seed, start)
    lo, hi = sharded.shard_bounds(n, world, rank)
    mine = oracle.init_states(hi - lo, seed, start + lo)    # the rule create_sharded_* applies
    assert mine.tobytes() == whole[lo:hi].tobytes()
    # gather the shards and compare the concatenation with the single-rank array
    pieces = [None] * world
    dist.all_gather_object(pieces, (lo, hi, mine.tobytes()))
    cat = b"".join(p[2] for p in sorted(pieces))
    assert cat == whole.tobytes()
    u_whole = oracle.fill(whole.copy(), "uniform", np.float32, 8)
    u_mine = oracle.fill(mine, "uniform", np.float32, 8)
    assert u_mine.tobytes() == u_whole[lo:hi].tobytes()


def _body_cast(rank, world):
    import oracle
    from numba_cuda_b200 import sharded
    n = 100003
    x = (4 * np.random.default_rng(3).standard_normal(n)).astype(np.float32)
    lo, hi = sharded.shard_bounds(n, world, rank, align=16)
    assert lo % 16 == 0
    whole = oracle.cast(x, oracle.F32, oracle.E4M3)
    assert oracle.cast(x[lo:hi], oracle.F32, oracle.E4M3).tobytes() == whole[lo:hi].tobytes()
    sizes = [None] * world
    dist.all_gather_object(sizes, hi - lo)
    assert sum(sizes) == n


def _body_axis_rows(rank, world):
    # rows sharded by contiguous range; the stacked partial rows folded along axis 0
    # must give the column results of the whole matrix (NumPy stands in for the kernel)
    from numba_cuda_b200 import _lib, sharded
    rng = np.random.default_rng(5)
    full = rng.integers(-2 ** 31, 2 ** 31, size=(1001, 37), dtype=np.int32)
    lo, hi = sharded.shard_bounds(full.shape[0], world, rank)
    for ufunc, op in ((np.add, _lib.ADD), (np.maximum, _lib.MAX), (np.bitwise_xor, _lib.XOR)):
        ident = sharded.op_identity(op, np.int32)
        with np.errstate(over="ignore"):
            partial = ufunc(ufunc.reduce(full[lo:hi], axis=0, dtype=np.int32), ident, dtype=np.int32)
        stacked = sharded.gather_partial_rows(torch.from_numpy(partial.view(np.uint8).copy()))
        assert tuple(stacked.shape) == (world, 37 * 4)
        rows = stacked.numpy().view(np.int32)
        with np.errstate(over="ignore"):
            got = ufunc.reduce(rows, axis=0, dtype=np.int32)
            want = ufunc.reduce(full, axis=0, dtype=np.int32)
        assert got.tobytes() == want.tobytes()
        # rank order is preserved: row r of the stack is rank r's partial
        assert rows[rank].tobytes() == partial.tobytes()


def _body_traced_combine(rank, world):
    """A user function outside the op table: per-rank records [value | present] are
    gathered once and the values that are there are folded in rank order with init
    (functools.reduce stands in for the run-time compiled kernel).  Rank 1's shard is
    empty in the second case, every shard in the third."""
    import functools
    from numba_cuda_b200 import sharded
    fn = lambda a, b: (a * 31 + b) % 1000003 if a > b else (b * 31 + a) % 1000003     # noqa: E731  (commutative)
    whole = np.random.default_rng(8).integers(0, 1 << 20, size=1000, dtype=np.int64)
    for case, bounds in (("all", sharded.shard_bounds(1000, world, rank)),
                         ("one empty", (0, 1000) if rank == 0 else (1000, 1000)),
                         ("all empty", (0, 0))):
        lo, hi = bounds
        record = np.zeros(16, dtype=np.uint8)
        if hi > lo:
            record[:8] = np.array([functools.reduce(fn, whole[lo:hi].tolist())], dtype=np.int64).view(np.uint8)
            record[8] = 1
        rows = sharded.gather_partial_rows(torch.from_numpy(record))
        assert tuple(rows.shape) == (world, 16)
        seen = []

        def fold(values):
            seen.append(np.array(values))
            return np.int64(functools.reduce(fn, values.tolist(), 7))
        got = sharded.fold_gathered(rows, np.int64, 7, fold)
        if case == "all empty":
            assert got == 7 and not seen
        else:
            parts = [functools.reduce(fn, whole[a:b].tolist())
                     for a, b in ([sharded.shard_bounds(1000, world, r) for r in range(world)]
                                  if case == "all" else [(0, 1000)])]
            assert seen[0].tolist() == parts                      # rank order, absent ranks dropped
            assert got == functools.reduce(fn, parts, 7)


def _body_world_mismatch(rank, world):
    from numba_cuda_b200 import sharded
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, world, world)


# ---- failures made on the host (no GPU involved) -----------------------------------
def _fail_rank_leaves_before_the_combine(rank, world):
    """Rank 1 raises before the collective; rank 0 must get an error from the
    combine instead of waiting for ever."""
    from numba_cuda_b200 import _lib, sharded
    if rank == 1:
        os._exit(0)          # leaves between steps, nothing in flight
    buf = torch.from_numpy(np.array([5], dtype=np.int32).view(np.uint8).copy())
    try:
        sharded.combine_partials(buf, _lib.MAX, np.int32)
    except Exception:
        return               # the expected outcome
    raise AssertionError("combine returned although a rank was missing")


def _fail_ranks_disagree_on_partition(rank, world):
    """A rank configured with a different world size computes bounds that do not
    tile the array; the mismatch is detected by exchanging the bounds."""
    from numba_cuda_b200 import sharded
    n = 1000
    claimed_world = world if rank == 0 else world + 1
    lo, hi = sharded.shard_bounds(n, claimed_world, rank)
    all_bounds = [None] * world
    dist.all_gather_object(all_bounds, (lo, hi))
    covered = sorted(all_bounds)
    contiguous = covered[0][0] == 0 and covered[-1][1] == n and all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    assert not contiguous
    dist.barrier()


# ---- tests ------------------------------------------------------------------------
def test_combine_partials_two_ranks():
    _run("_body_reduce")


def test_rng_shards_concatenate_to_single_stream():
    _run("_body_rng")


def test_cast_shards_are_aligned_and_complete():
    _run("_body_cast")


def test_row_sharded_axis_reduce_combines_with_one_gather():
    _run("_body_axis_rows")


def test_traced_function_partials_are_gathered_and_folded_in_rank_order():
    _run("_body_traced_combine")


def test_bad_rank_is_rejected():
    _run("_body_world_mismatch")


def test_missing_rank_fails_the_combine_instead_of_hanging():
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, "_fail_rank_leaves_before_the_combine", errors))
             for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        if p.is_alive():
            p.kill()
            pytest.fail("a rank hung")
    assert errors.empty(), errors.get()


def test_partition_mismatch_is_detectable():
    _run("_fail_ranks_disagree_on_partition")


def test_single_process_is_world_of_one():
    from numba_cuda_b200 import _lib, sharded
    buf = torch.from_numpy(np.array([5], dtype=np.int32).view(np.uint8).copy())
    assert sharded.combine_partials(buf, _lib.MAX, np.int32) is buf
