#!/usr/bin/env python
"""Benchmark of the B200-native library kernels on the reference's configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline line (one JSON object on stdout, printed by rank 0):

* workload = configuration 2: ``cuda.reduce(max)`` over 2^28 int32 IN TOTAL
  (``default_rng(1).integers`` over the full int32 range).  With N > 1 rank k reduces
  the contiguous shard ``x[k*n/N:(k+1)*n/N]`` and the partials are combined once per
  step (strong scaling: the job is the same 1 GiB at every N).  The default combine
  runs inside the reduce kernel over NVLink peer memory (``b2k_reduce_peer``), and
  consecutive steps are pipelined with programmatic dependent launch (a step reads
  its shard while the previous step's exchange completes; results stay in stream
  order).  ``paths`` also carries the same step without pipelining, the step with
  one NCCL all-reduce(max) of one int32 after the kernel, and the weak-scaling
  figure (2^28 per rank);
* every rank keeps N copies of its shard at different addresses and the steps
  rotate over them, so a step always streams 1 GiB per GPU's worth of distinct
  lines through the 126 MB L2 before a line is read again;
* ``value``  : GB/s of input consumed by the whole job, inputs resident in HBM,
  CUDA-event time, max over ranks;
* ``e2e``    : the same metric through the public Python API with the shard in
  pinned HOST memory: H2D copy of the shard + kernel (+ combine) + D2H of the scalar
  are all inside the timed region;
* ``roofline``: the reduce kernel alone against the measured HBM copy rate;
* ``cpu_baseline``: the reference's CPU path for cuda.reduce (the simulator's
  sequential functools.reduce) timed on a bounded prefix on the host;
* ``paths``  : the other configurations (reduce f64 2^20, transposes, RNG, casts),
  each with its own value and roofline fraction; ``paths_reference_gpu``: the
  reference's own GPU kernels (upstream numba's identical kernel source) on the
  same GPU, for context.

``--impl reference`` times only the reference's CPU path (rank 0; other ranks
exit at once) and prints a line of the same shape.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_C2 = 1 << 28
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the reduce kernel over
# 2^28 int32, from an ncu capture of this kernel (traffic grows with the bytes read, so
# a shard's launch is charged its share)
REDUCE_TRAFFIC_BYTES_2P28 = 1077902920
# executed thread-instructions per sample of the RNG fill kernels, from ncu
# (smsp__thread_inst_executed.sum / samples) on 2^21 generators
RNG_INSTR_PER_SAMPLE = {"c4_rng_generate_64u32_16n64": 48.0, "rng_uniform_f32_only_64": 22.0}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def config_dict(n_gpus):
    """The workload both arms are run on (identical for ours and the reference arm)."""
    return {"workload": "C2: cuda.reduce(max) over 2^28 int32 in total, uniform over the full int32 range "
                        "(default_rng(seed=1).integers), default init=0",
            "elements_total": N_C2, "bytes_total": N_C2 * 4,
            "elements_per_gpu": N_C2 // n_gpus, "bytes_per_gpu": N_C2 * 4 // n_gpus,
            "sharding": ("single GPU" if n_gpus == 1 else
                         f"contiguous shard x[k*n/{n_gpus}:(k+1)*n/{n_gpus}] per rank, partials combined once per step"),
            "l2": ("input (1 GiB) is larger than L2 (126 MB); no flush between steps" if n_gpus == 1 else
                   f"each rank rotates over {n_gpus} copies of its shard at different addresses (1 GiB per GPU in "
                   "rotation, larger than the 126 MB L2); no flush between steps")}


def c2_array_chunks(chunk=1 << 24):
    """Configuration 2's input, chunk by chunk (one generator, drawn in order)."""
    rng = np.random.default_rng(1)
    for lo in range(0, N_C2, chunk):
        yield lo, rng.integers(-2 ** 31, 2 ** 31, size=chunk, dtype=np.int32)


# --------------------------------------------------------------------------- reference arm
def reference_arm(args, rank):
    """The reference's CPU path for cuda.reduce is the simulator's Reduce:
    functools.reduce(functor, seq, init) (numba/cuda/simulator/reduction.py:7-16),
    single-threaded Python by construction.  Each step folds a bounded prefix of
    configuration 2's array."""
    if rank != 0:
        return
    import oracle
    sample_n = 1 << 22
    x = np.random.default_rng(1).integers(-2 ** 31, 2 ** 31, size=sample_n, dtype=np.int32)
    fn = lambda a, b: max(a, b)  # noqa: E731
    for _ in range(args.warmup):
        oracle.py_fold(fn, x[: 1 << 18], 0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        got = oracle.py_fold(fn, x, 0)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    assert got == max(int(x.max()), 0)
    gbs = sample_n * 4 / dt / 1e9
    line = {
        "impl": "reference", "metric": "reduce_max_int32_GBps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int32",
        "data": "synthetic", "config": config_dict(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": f"each step folds the first 2^22 of the 2^28 int32 with functools.reduce(max), as "
                                   f"the simulator's Reduce does; host has {os.cpu_count()} cores, the path is "
                                   "single-threaded by construction; GB/s is per element rate, size-independent"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-paths", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--only", default=None,
                    help="run a single path (profiling aid): c1,user,c2,c3a,c3b,c4,c5,n2,refgpu")
    ap.add_argument("--scale", type=int, default=0, help="shrink the --only workload by 2^scale (profiling aid)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.only == "refgpu":
        reference_gpu_kernels()
        return

    import torch
    import torch.distributed as dist
    import numba_cuda_b200 as cuda
    from numba_cuda_b200 import _lib, sharded

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    L = _lib.lib()
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if not distributed:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    by_rank = {}

    def timed(fn, steps, warmup, label=None):
        """CUDA-event time per step on the launching stream, max over ranks (ms)."""
        for _ in range(max(warmup, 3)):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = L.b2k_launch_count()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        launches = L.b2k_launch_count() - before
        mine = e0.elapsed_time(e1) / steps
        if label and distributed:
            every = torch.empty(world, dtype=torch.float64, device="cuda")
            dist.all_gather_into_tensor(every, torch.tensor([mine], dtype=torch.float64, device="cuda"))
            by_rank[label] = [round(v * 1e3, 2) for v in every.cpu().tolist()]
        return max_over_ranks(mine), launches

    peak, peak_kind = measured_peak()

    if args.only:
        run_single_path(args, cuda, L, torch, timed, peak, peak_kind, sptr)
        if distributed:
            dist.destroy_process_group()
        return

    # ---------------- headline: configuration 2, strong scaling ------------------
    lo, hi = sharded.shard_bounds(N_C2, world, rank, align=8)
    n_shard = hi - lo
    host = cuda.pinned_array(n_shard, dtype=np.int32)
    expect = -2 ** 31
    for base, piece in c2_array_chunks():
        expect = max(expect, int(piece.max()))
        a, b = max(lo, base), min(hi, base + piece.size)
        if a < b:
            host[a - lo:b - lo] = piece[a - base:b - base]
    copies = [cuda.to_device(host) for _ in range(world)]     # 1 GiB per GPU in rotation
    torch.cuda.synchronize()

    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    ident = np.array([-2 ** 31], dtype=np.int32)
    ident_ptr, out_ptr = ident.ctypes.data, out.data_ptr()
    copy_ptrs = [c._ptr for c in copies]
    turn = [0]

    def next_copy():
        turn[0] = (turn[0] + 1) % len(copy_ptrs)
        return copy_ptrs[turn[0]]

    def check(rc):
        if rc:
            raise RuntimeError(L.b2k_last_error())

    def kernel_only():
        check(L.b2k_reduce(_lib.MAX, _lib.I32, next_copy(), n_shard, ident.ctypes.data, out.data_ptr(),
                           scratch.data_ptr(), scratch.numel(), sptr))

    boxes = None
    if distributed and os.environ.get("B2K_BENCH_NCCL", "0") != "1":
        try:
            boxes = sharded.PeerMailboxes()
        except Exception as exc:  # e.g. no peer access between the GPUs
            if rank == 0:
                print(f"peer mailboxes unavailable ({exc}); using NCCL", file=sys.stderr)
            boxes = None

    def step_pipelined():
        if boxes is not None:
            boxes.reduce(_lib.MAX, _lib.I32, next_copy(), n_shard, ident_ptr, out_ptr, sptr, input_ready=True)
        elif distributed:
            step_nccl()
        else:
            check(L.b2k_reduce_ex(_lib.MAX, _lib.I32, next_copy(), n_shard, ident.ctypes.data, out.data_ptr(),
                                  scratch.data_ptr(), scratch.numel(), _lib.REDUCE_INPUT_READY, sptr))

    def step_unpipelined():
        if boxes is not None:
            boxes.reduce(_lib.MAX, _lib.I32, next_copy(), n_shard, ident_ptr, out_ptr, sptr)
        else:
            kernel_only()

    def step_nccl():
        kernel_only()
        dist.all_reduce(out, op=dist.ReduceOp.MAX)

    def verify(what):
        got = int(out.item())
        assert got == expect, (what, got, expect)
        if boxes is not None:
            boxes.check(agree=True)

    # clocks are sampled from here to the end of the end-to-end leg (the headline region
    # alone lasts only a few milliseconds, less than one nvidia-smi sample)
    clocks = ClockSampler(local_rank)
    clocks.__enter__()
    ms_step, launches = timed(step_pipelined, args.steps, args.warmup, "step_us")
    verify("pipelined step")

    variants = {}
    ms_unpiped, _ = timed(step_unpipelined, args.steps, 3)
    if distributed:
        verify("unpipelined step")
    # the kernel alone (roofline): the same launches on this rank's shard, no combine
    ms_kernel, _ = timed(kernel_only, args.steps, 3, "kernel_us")
    shard_bytes = n_shard * 4
    total_bytes = N_C2 * 4

    def gbs(ms):
        return total_bytes / (ms * 1e-3) / 1e9

    variants["c2_step_unpipelined"] = {
        "GBps": gbs(ms_unpiped), "ms": ms_unpiped,
        "note": "the same step with every kernel waiting for the one before (no programmatic overlap)"}
    exchange = None
    if distributed:
        # every rank alone: the same pipelined launches without any exchange (what a kernel
        # boundary costs by itself on a shard of this size)
        def step_alone():
            check(L.b2k_reduce_ex(_lib.MAX, _lib.I32, next_copy(), n_shard, ident_ptr, out_ptr,
                                  scratch.data_ptr(), scratch.numel(), _lib.REDUCE_INPUT_READY, sptr))
        ms_alone, _ = timed(step_alone, args.steps, 3, "alone_us")
        variants["c2_pipelined_no_exchange"] = {
            "GBps": gbs(ms_alone), "ms": ms_alone,
            "note": "every rank reduces its shard with the same pipelined launches and no combine (not a valid "
                    "result for the job: shows what the exchange adds)"}
        ms_nccl, _ = timed(step_nccl, args.steps, 3)
        verify("nccl step")
        variants["c2_nccl"] = {"GBps": gbs(ms_nccl), "ms": ms_nccl,
                               "note": "reduce kernel + one NCCL all-reduce(max) of one int32 per step"}
        if boxes is not None:
            exchange = measure_exchange(boxes, step_unpipelined, barrier, dist, torch, world)
            exchange["step_minus_kernel_us_unpipelined"] = (ms_unpiped - ms_kernel) * 1e3
            exchange["step_minus_kernel_us_pipelined"] = (ms_step - ms_kernel) * 1e3
            exchange["step_minus_kernel_us_nccl"] = (ms_nccl - ms_kernel) * 1e3

    # end to end through the public API: host shard -> device -> kernel (+ combine) -> host scalar
    sharded_max = sharded.ShardedReduce(lambda a, b: max(a, b), peer=boxes)
    plain_max = cuda.reduce(lambda a, b: max(a, b))

    def e2e_step():
        got = sharded_max(host, init=0) if distributed else plain_max(host, init=0)
        assert got == max(expect, 0)

    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e, _ = timed(e2e_step, e2e_steps, 3)
    clocks.__exit__(None, None, None)
    clock_summary = clocks.summary()

    achieved = shard_bytes / (ms_kernel * 1e-3) / 1e9
    line = {
        "metric": "reduce_max_int32_GBps",
        "value": gbs(ms_step),
        "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int32", "data": "synthetic",
        "config": config_dict(world),
        "combine": (
            "single GPU; consecutive steps overlap through programmatic dependent launch" if not distributed else
            "inside the reduce kernel: peer-memory mailboxes over NVLink (b2k_reduce_peer), one launch per rank per "
            "step, steps pipelined with programmatic dependent launch" if boxes is not None
            else "reduce kernel + one NCCL all-reduce(max) of one int32"),
        "clocks": clock_summary,
        "e2e": {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": total_bytes, "d2h_bytes_per_step": 4 * world,
                "h2d_bytes_per_step_per_gpu": shard_bytes, "steps": e2e_steps, "ms_per_step": ms_e2e,
                "call": "ShardedReduce(max, peer=...)(pinned host shard, init=0)" if distributed
                        else "cuda.reduce(max)(pinned host array, init=0)"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak,
                     "traffic": int(REDUCE_TRAFFIC_BYTES_2P28 * (shard_bytes / (N_C2 * 4))), "peak_kind": peak_kind,
                     "kernel": "reduce_kernel<int, OpMax>", "us_per_launch": ms_kernel * 1e3,
                     "algorithmic_bytes_per_launch": shard_bytes,
                     "note": "per rank: this rank's shard / its kernel's time, no combine"},
    }
    if exchange is not None:
        line["exchange_us"] = exchange
    if by_rank:
        line["us_by_rank"] = by_rank

    if rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(host)
    del copies, host

    paths = dict(variants)
    if distributed:
        paths["c2_weak"] = weak_scaling_leg(cuda, L, _lib, torch, timed, boxes, world, rank, sptr)
    if not args.no_paths:
        paths.update(secondary_paths(cuda, L, torch, timed, peak, world, rank, sptr))
        if rank == 0 and world == 1:
            line["paths_cpu"] = secondary_cpu_baselines()
    line["paths"] = paths
    if rank == 0 and world == 1 and not args.no_paths:
        line["paths_reference_gpu"] = reference_gpu_subprocess()

    if rank == 0:
        print(json.dumps(line), flush=True)
    if boxes is not None:
        boxes.close()
    if distributed:
        dist.destroy_process_group()


def measure_exchange(boxes, step, barrier, dist, torch, world, rounds=40):
    """What the in-kernel exchange costs, from the GPUs' own nanosecond timers: per
    step and rank, (last peer value seen) - (local fold complete).  The rank that
    finishes last waits for nobody, so the minimum over ranks is the bare one-way
    delivery; the maximum adds how far the ranks' kernels were out of step."""
    waits = []
    for _ in range(rounds):
        barrier()
        step()
        torch.cuda.synchronize()
        waits.append(boxes.exchange_ns())
    mine = torch.tensor(waits, dtype=torch.float64, device="cuda")
    every = torch.empty(world * rounds, dtype=torch.float64, device="cuda")
    dist.all_gather_into_tensor(every, mine)
    table = every.view(world, rounds).cpu().numpy() / 1e3
    return {"min_over_ranks_median": float(np.median(table.min(axis=0))),
            "max_over_ranks_median": float(np.median(table.max(axis=0))),
            "rounds": rounds,
            "meaning": "device-timer microseconds from 'local fold done' to 'all peers seen' per step; min over "
                       "ranks = delivery latency, max over ranks = latency + launch skew between ranks "
                       "(ranks released from a host barrier each round)"}


def weak_scaling_leg(cuda, L, _lib, torch, timed, boxes, world, rank, sptr):
    """2^28 int32 per rank (the job grows with N), fused combine, pipelined."""
    x = torch.randint(-2 ** 31, 2 ** 31 - 1, (N_C2,), dtype=torch.int32, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    ident = np.array([-2 ** 31], dtype=np.int32)
    scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")

    def step():
        if boxes is not None:
            boxes.reduce(_lib.MAX, _lib.I32, x.data_ptr(), N_C2, ident, out.data_ptr(), sptr, input_ready=True)
        else:
            rc = L.b2k_reduce(_lib.MAX, _lib.I32, x.data_ptr(), N_C2, ident.ctypes.data, out.data_ptr(),
                              scratch.data_ptr(), scratch.numel(), sptr)
            assert rc == 0
            torch.distributed.all_reduce(out, op=torch.distributed.ReduceOp.MAX)
    ms, _ = timed(step, 20, 3)
    return {"GBps": N_C2 * 4 * world / (ms * 1e-3) / 1e9, "ms": ms,
            "note": "weak scaling: 2^28 int32 per rank (torch.randint), same fused step"}


def cpu_baseline(whole):
    """The reference's CPU path for this workload on a bounded prefix; NumPy's own
    ``max`` over the whole array beside it as the sane CPU line."""
    import oracle
    sample = 1 << 24
    x = np.array(whole[:sample])
    fn = lambda a, b: max(a, b)  # noqa: E731
    t0 = time.perf_counter()
    got = oracle.py_fold(fn, x, 0)
    dt = time.perf_counter() - t0
    assert got == max(int(x.max()), 0)
    t1 = time.perf_counter()
    np_max = int(whole.max())
    dt_np = time.perf_counter() - t1
    return {"value": sample * 4 / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": "first 2^24 of the 2^28 int32, functools.reduce(max, seq, 0) as the simulator's Reduce "
                      f"does (single Python thread; host has {os.cpu_count()} cores)",
            "seconds": dt,
            "numpy_max_GBps": whole.nbytes / dt_np / 1e9, "numpy_max_value": np_max,
            "numpy_note": "x.max() over all 2^28 int32 in host memory, one thread: the sane CPU line"}


def secondary_cpu_baselines():
    """The reference's CPU path for the other configurations, each on a bounded
    sample (a few seconds in total).  kind "reference" = the reference's own code
    (its vendored conversion headers compiled with g++); kind "port" = the oracle's
    restatement of the reference algorithm."""
    import oracle
    out = {"host_cores": os.cpu_count()}

    def clock(fn):
        t0 = time.perf_counter()
        r = fn()
        return time.perf_counter() - t0, r

    # C1: the simulator's Reduce is functools.reduce over the sequence
    x = np.random.default_rng(0).random(1 << 20)
    dt, got = clock(lambda: oracle.py_fold(lambda a, b: a + b, x, 0))
    out["c1_reduce_sum_f64_2p20"] = {"GBps": x.nbytes / dt / 1e9, "seconds": dt, "cores": 1, "kind": "port",
                                     "sample": "full 2^20 float64, functools.reduce as the simulator does"}
    # C3: the simulator's transpose is np.transpose; the copy is the honest cost
    a = np.random.default_rng(2).standard_normal((4096, 4096), dtype=np.float32)
    dt, _ = clock(lambda: np.ascontiguousarray(a.T))
    out["c3a_transpose_f32"] = {"GBps": 2 * a.nbytes / dt / 1e9, "seconds": dt, "cores": 1, "kind": "port",
                                "sample": "4096x4096 float32 block, np.ascontiguousarray(a.T)"}
    # assignment / permutation: the simulator's device array is a NumPy array underneath
    src = np.random.default_rng(4).standard_normal(1 << 24, dtype=np.float32)
    dst = np.empty_like(src)

    def copy():
        dst[:] = src
    dt, _ = clock(copy)
    out["n2_assign_copy_f32"] = {"GBps": 2 * src.nbytes / dt / 1e9, "seconds": dt, "cores": 1, "kind": "port",
                                 "sample": "2^24 of the 2^28 float32, NumPy slice assignment"}
    cube = src.reshape(64, 512, 512)
    dt_permute, _ = clock(lambda: np.ascontiguousarray(cube.transpose(0, 2, 1)))
    out["n4_permute_021_f32"] = {"GBps": 2 * src.nbytes / dt_permute / 1e9, "seconds": dt_permute, "cores": 1,
                                 "kind": "port",
                                 "sample": "64x512x512 float32, np.ascontiguousarray(a.transpose(0, 2, 1))"}
    mat = src[:1 << 22].reshape(2048, 2048)
    dt_axis, _ = clock(lambda: (mat.sum(axis=0), mat.sum(axis=1)))
    out["n4_reduce_sum_axis_f32"] = {"GBps": 2 * mat.nbytes / dt_axis / 1e9, "seconds": dt_axis, "cores": 1,
                                     "kind": "port",
                                     "sample": "2048x2048 float32, NumPy sum along axis 0 and along axis 1"}
    # C4: serial state chain (random.py:242-257) and the draw loop, C restatement
    n = 1 << 16
    dt, st = clock(lambda: oracle.init_states(n, 42, 0))
    out["c4_rng_init"] = {"Mstates_per_s": n / dt / 1e6, "seconds": dt, "cores": 1, "kind": "port",
                          "sample": "2^16 of the 2^24 states, serial jump chain in C"}

    def draws():
        oracle.fill(st, "uniform", np.float32, 64)
        oracle.fill(st, "normal", np.float64, 16)
    dt, _ = clock(draws)
    out["c4_rng_generate_64u32_16n64"] = {"Gsamples_per_s": n * 80 / dt / 1e9, "GBps": n * 416 / dt / 1e9,
                                          "seconds": dt, "cores": 1, "kind": "port",
                                          "sample": "2^16 generators x (64 uniform f32 + 16 normal f64), C restatement"}
    # C5: the reference's vendored cuda_fp8.hpp / cuda_bf16.hpp host paths on all cores
    m = 1 << 24
    v = (4 * np.random.default_rng(3).standard_normal(m)).astype(np.float32)
    if oracle.have_ref_headers():
        for label, src_f, dst_f, bpe in (("c5_cast_f32_to_e4m3", oracle.F32, oracle.E4M3, 5),
                                         ("c5_cast_f32_to_bf16", oracle.F32, oracle.BF16, 6)):
            dt, codes = clock(lambda: oracle.ref_cast(v, src_f, dst_f, 1, threads=0))
            out[label] = {"GBps": m * bpe / dt / 1e9, "seconds": dt, "cores": os.cpu_count(), "kind": "reference",
                          "sample": "2^24 of the 2^30 elements, vendored header host path, std::thread over all cores"}
        e = oracle.ref_cast(v, oracle.F32, oracle.E4M3, 1)
        dt, _ = clock(lambda: oracle.ref_cast(e, oracle.E4M3, oracle.F32, 1, threads=0))
        out["c5_cast_e4m3_to_f32"] = {"GBps": m * 5 / dt / 1e9, "seconds": dt, "cores": os.cpu_count(),
                                      "kind": "reference", "sample": "2^24 codes, vendored header host path"}
    else:
        dt, _ = clock(lambda: oracle.cast(v, oracle.F32, oracle.E4M3, 1))
        out["c5_cast_f32_to_e4m3"] = {"GBps": m * 5 / dt / 1e9, "seconds": dt, "cores": 1, "kind": "port",
                                      "sample": "2^24 of the 2^30 elements, C restatement"}
    return out


# --------------------------------------------------------------------------- the reference's own GPU kernels
def reference_gpu_subprocess():
    """Run ``bench.py --only refgpu`` in a process of its own (numba's driver layer and
    torch each keep their own view of the context) after this arm's timed regions."""
    try:
        p = subprocess.run([sys.executable, os.path.abspath(__file__), "--only", "refgpu"], capture_output=True,
                           text=True, timeout=240, cwd=ROOT)
        for raw in reversed(p.stdout.strip().splitlines()):
            if raw.startswith("{"):
                return json.loads(raw)
        return {"unavailable": (p.stderr or p.stdout).strip()[-300:] or f"exit code {p.returncode}"}
    except Exception as exc:  # context only, never a reason to fail the bench
        return {"unavailable": repr(exc)}


def reference_gpu_kernels():
    """The reference's GPU kernels for the same configurations, for context: upstream
    numba's bundled ``numba.cuda`` (same kernel source as the reference's
    kernels/reduction.py, kernels/transpose.py and random.py; the reference package
    itself needs ``cuda-core``, which this image lacks).  Wall-clock around
    synchronised calls, compile time excluded where the reference caches its kernel."""
    info = {"what": "upstream numba.cuda (identical kernel source) on this GPU; wall clock, synchronised"}
    try:
        import warnings
        warnings.filterwarnings("ignore")
        from numba import cuda as ncuda
        from numba.cuda.random import create_xoroshiro128p_states, xoroshiro128p_normal_float64, \
            xoroshiro128p_uniform_float32
    except Exception as exc:
        print(json.dumps({"unavailable": f"numba.cuda not importable: {exc!r}"}))
        return

    def timeit(fn, reps=5):
        fn()
        ncuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        ncuda.synchronize()
        return (time.perf_counter() - t0) / reps

    try:
        x = ncuda.to_device(np.random.default_rng(1).integers(-2 ** 31, 2 ** 31, size=N_C2, dtype=np.int32))
        mx = ncuda.reduce(lambda a, b: max(a, b))
        res0 = ncuda.device_array(1, dtype=np.int32)
        s = timeit(lambda: mx(x, res=res0))
        info["c2_reduce_max_int32_2p28"] = {"us": s * 1e6, "GBps": N_C2 * 4 / s / 1e9,
                                            "note": "three launches + partials allocation per call"}
        del x
        y = ncuda.to_device(np.random.default_rng(0).random(1 << 20))
        sm = ncuda.reduce(lambda a, b: a + b)
        res1 = ncuda.device_array(1, dtype=np.float64)
        s = timeit(lambda: sm(y, res=res1), reps=50)
        info["c1_reduce_sum_f64_2p20"] = {"us": s * 1e6}
        a = ncuda.to_device(np.zeros((8192, 8192), dtype=np.float32))
        s = timeit(lambda: a.T, reps=2)
        info["transpose_f32_8192x8192"] = {"us": s * 1e6, "GBps": 2 * 8192 * 8192 * 4 / s / 1e9,
                                           "note": "the kernel is re-compiled on every call, as the reference does"}
        del a
        n2 = 1 << 20
        t0 = time.perf_counter()
        st = create_xoroshiro128p_states(n2, seed=42)
        ncuda.synchronize()
        info["rng_create_states_2p20"] = {"us": (time.perf_counter() - t0) * 1e6,
                                          "note": "serial chain on the CPU + upload"}

        @ncuda.jit
        def c4_kernel(states, u, z, nu, nz):
            t = ncuda.grid(1)
            if t < states.shape[0]:
                for i in range(nu):
                    u[t * nu + i] = xoroshiro128p_uniform_float32(states, t)
                for i in range(nz):
                    z[t * nz + i] = xoroshiro128p_normal_float64(states, t)

        u = ncuda.device_array(n2 * 64, dtype=np.float32)
        z = ncuda.device_array(n2 * 16, dtype=np.float64)
        s = timeit(lambda: c4_kernel[(n2 + 127) // 128, 128](st, u, z, 64, 16))
        info["c4_generate_64u32_16n64_2p20_states"] = {"us": s * 1e6, "Gsamples_per_s": n2 * 80 / s / 1e9,
                                                       "GBps": n2 * 416 / s / 1e9}
    except Exception as exc:  # context only
        info["error"] = repr(exc)
    print(json.dumps(info), flush=True)


# --------------------------------------------------------------------------- other configurations
def _roof(bytes_per_launch, ms, peak):
    ach = bytes_per_launch / (ms * 1e-3) / 1e9
    return {"GBps": ach, "frac_of_measured_copy": ach / peak, "frac_of_8000": ach / 8000.0, "ms": ms}


def _issue_bound(res, samples_per_s, instr_per_sample, torch):
    """RNG kernels are bound by instruction issue, not by HBM: the fraction of the
    GPU's issue rate (SMs x 4 schedulers x 32 lanes x SM clock) the kernel uses."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    try:
        mhz = float(subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits", "-i",
                                    str(torch.cuda.current_device())], capture_output=True, text=True,
                                   timeout=10).stdout.split()[0])
    except Exception:
        mhz = 1965.0
    peak = sms * 128 * mhz * 1e6
    res.update(bound="issue", thread_instr_per_sample=instr_per_sample, sm_mhz_sampled=mhz,
               frac_of_issue_peak=samples_per_s * instr_per_sample / peak)


def secondary_paths(cuda, L, torch, timed, peak, world, rank, sptr, only=None, scale=0):
    """Configurations 1, 3a, 3b, 4, 5 and the adjacent paths: per-rank work is fixed
    (every rank runs the same case); times are CUDA-event, max over ranks; GB/s are
    per GPU.  Inputs: configuration 1 is the seeded NumPy array itself; the multi-GiB
    inputs of configurations 3-5 are drawn on the device with torch from the same
    distributions (normal(0,1); normal(0,4) with 1 % specials), because drawing them
    with NumPy costs minutes of host time -- the seeded NumPy inputs at full size are
    what the parity tests use."""
    from numba_cuda_b200 import _lib
    res = {}
    iters, warm = 10, 3

    def want(name):
        return only is None or only == name

    def check(rc):
        if rc:
            raise RuntimeError(L.b2k_last_error())

    if want("c1"):
        n = 1 << 20
        x = cuda.to_device(np.random.default_rng(0).random(n))
        scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
        out = torch.zeros(1, dtype=torch.float64, device="cuda")
        zero = np.zeros(1, dtype=np.float64)

        # the arguments are worked out once: the loop below measures the C-ABI call, not
        # Python attribute look-ups (ndarray.ctypes alone costs more than a microsecond)
        xp, zp, op_, sp_, sn = x._ptr, zero.ctypes.data, out.data_ptr(), scratch.data_ptr(), scratch.numel()
        reduce_fn, reduce_ex = L.b2k_reduce, L.b2k_reduce_ex

        def call():
            if reduce_fn(_lib.ADD, _lib.F64, xp, n, zp, op_, sp_, sn, sptr):
                raise RuntimeError(L.b2k_last_error())

        def call_ready():
            if reduce_ex(_lib.ADD, _lib.F64, xp, n, zp, op_, sp_, sn, _lib.REDUCE_INPUT_READY, sptr):
                raise RuntimeError(L.b2k_last_error())
        ms, _ = timed(call, 200, 10)
        entry = dict(_roof(n * 8, ms, peak), us_per_call=ms * 1e3,
                     note="8 MiB: launch-latency bound, L2 resident; us_per_call = back-to-back calls through "
                          "ctypes (CUDA events), kernel_us = the same launches replayed from a CUDA graph, "
                          "host_us_per_call = wall clock of the issuing loop alone; *_input_ready = the same with "
                          "B2K_REDUCE_INPUT_READY (the input is not produced by the previous kernel), which lets "
                          "a reduction read its input while the one before finishes")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(2000):
            call()
        entry["host_us_per_call"] = (time.perf_counter() - t0) / 2000 * 1e6
        torch.cuda.synchronize()
        ms_r, _ = timed(call_ready, 200, 10)
        entry["us_per_call_input_ready"] = ms_r * 1e3
        assert abs(float(out.item()) - float(np.random.default_rng(0).random(n).sum())) < 1e-6
        # the same call captured in a CUDA graph (20 launches per replay): what is left
        # of the 8 MiB case once the launch path is off the critical line
        for key, fn_ in (("kernel_us", reduce_fn), ("kernel_us_input_ready", reduce_ex)):
            try:
                side = torch.cuda.Stream()
                graph = torch.cuda.CUDAGraph()
                extra = () if fn_ is reduce_fn else (_lib.REDUCE_INPUT_READY,)
                with torch.cuda.stream(side):
                    check(fn_(_lib.ADD, _lib.F64, xp, n, zp, op_, sp_, sn, *extra, side.cuda_stream))
                side.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(20):
                        check(fn_(_lib.ADD, _lib.F64, xp, n, zp, op_, sp_, sn, *extra,
                                  torch.cuda.current_stream().cuda_stream))
                ms_g, _ = timed(graph.replay, 20, 5)
                entry[key] = ms_g * 1e3 / 20
                del graph
            except Exception as exc:  # graphs are an extra, never a reason to fail the bench
                entry[key + "_error"] = repr(exc)
        if "kernel_us" in entry:
            entry["us_per_call_in_cuda_graph"] = entry["kernel_us"]
        res["c1_reduce_sum_f64_2p20"] = entry
        n2 = 1 << (28 - scale)
        y = torch.rand(n2, dtype=torch.float64, device="cuda")
        ms, _ = timed(lambda: check(L.b2k_reduce(_lib.ADD, _lib.F64, y.data_ptr(), n2, zero.ctypes.data,
                                                 out.data_ptr(), scratch.data_ptr(), scratch.numel(), sptr)),
                      iters, warm)
        res["reduce_sum_f64_2p28"] = _roof(n2 * 8, ms, peak)
        del x, y

    if want("user"):
        # a user function outside the op table: traced, compiled at run time around the same reduce skeleton
        scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
        n3 = 1 << (28 - scale)
        w = torch.randint(0, 1000003, (n3,), dtype=torch.int32, device="cuda")
        out32 = torch.zeros(1, dtype=torch.int32, device="cuda")
        zero32 = np.zeros(1, dtype=np.int32)
        expr = cuda.Reduce(lambda a, b: (a + b) % 1000003)._compile(np.dtype(np.int32))
        assert isinstance(expr, str)
        ms, _ = timed(lambda: check(L.b2k_reduce_expr(expr.encode(), _lib.I32, w.data_ptr(), n3, zero32.ctypes.data,
                                                      out32.data_ptr(), scratch.data_ptr(), scratch.numel(), sptr)),
                      iters, warm)
        res["user_reduce_mod_add_int32_2p28"] = dict(
            _roof(n3 * 4, ms, peak), expression=expr,
            spot_check=bool(int(out32.item()) == int(w.sum(dtype=torch.int64).item()) % 1000003),
            note="numba's typing: the sum and the remainder are 64-bit operations")
        # a light user function (no division): the same skeleton is HBM-bound
        expr2 = cuda.Reduce(lambda a, b: max(abs(a), abs(b)))._compile(np.dtype(np.int32))
        assert isinstance(expr2, str)
        ms, _ = timed(lambda: check(L.b2k_reduce_expr(expr2.encode(), _lib.I32, w.data_ptr(), n3, zero32.ctypes.data,
                                                      out32.data_ptr(), scratch.data_ptr(), scratch.numel(), sptr)),
                      iters, warm)
        res["user_reduce_absmax_int32_2p28"] = dict(
            _roof(n3 * 4, ms, peak), expression=expr2,
            spot_check=bool(int(out32.item()) == int(w.abs().max().item())))
        del w

    for name, rows, cols, tdt, item in (("c3a_transpose_f32_32768x32768", 32768, 32768, torch.float32, 4),
                                        ("c3b_transpose_bf16_16384x65536", 16384, 65536, torch.bfloat16, 2)):
        key = name[:3]
        if not want(key):
            continue
        rows >>= scale
        a = torch.randn(rows, cols, device="cuda", dtype=torch.float32).to(tdt)
        b = torch.empty(cols, rows, device="cuda", dtype=tdt)
        ms, _ = timed(lambda: check(L.b2k_transpose2d(a.data_ptr(), b.data_ptr(), rows, cols, cols * item, item,
                                                      rows * item, item, item, sptr)), iters, warm)
        # spot check against NumPy .T on two corner blocks (the full-size comparison is a parity test)
        view = torch.int32 if item == 4 else torch.int16
        ok = True
        for r0, c0 in ((0, 0), (rows - 256, cols - 256)):
            got = b[c0:c0 + 256, r0:r0 + 256].contiguous().view(view).cpu().numpy()
            ok = ok and np.array_equal(got, a[r0:r0 + 256, c0:c0 + 256].contiguous().view(view).cpu().numpy().T)
        res[name] = dict(_roof(2 * rows * cols * item, ms, peak), spot_check=bool(ok),
                         scope="replicas" if world > 1 else "single GPU")
        del a, b

    if want("c4"):
        n = 1 << (24 - scale)
        states = cuda.device_array(n, dtype=cuda.random.xoroshiro128p_dtype)
        ms_init, _ = timed(lambda: cuda.random.init_xoroshiro128p_states(states, 42, rank * n), iters, warm)
        u = torch.empty(n, 64, dtype=torch.float32, device="cuda")
        z = torch.empty(n, 16, dtype=torch.float64, device="cuda")

        def fill(d0, p0, c0, d1=0, p1=None, c1=0):
            return lambda: check(L.b2k_xoroshiro128p_fill(states._ptr, n, d0, p0, c0, d1, p1, c1, sptr))
        ms, _ = timed(fill(_lib.UNIFORM_F32, u.data_ptr(), 64, _lib.NORMAL_F64, z.data_ptr(), 16), iters, warm)
        res["c4_rng_init_2p24_states"] = dict(_roof(n * 16, ms_init, peak), Mstates_per_s=n / ms_init / 1e3,
                                              bound="shared-memory bandwidth (16 table lookups of 16 bytes per state)")
        res["c4_rng_generate_64u32_16n64"] = dict(_roof(n * 416, ms, peak), Gsamples_per_s=n * 80 / ms / 1e6)
        _issue_bound(res["c4_rng_generate_64u32_16n64"], n * 80 / (ms * 1e-3),
                     RNG_INSTR_PER_SAMPLE["c4_rng_generate_64u32_16n64"], torch)
        ms_u, _ = timed(fill(_lib.UNIFORM_F32, u.data_ptr(), 64), iters, warm)
        res["rng_uniform_f32_only_64"] = dict(_roof(n * (32 + 256), ms_u, peak), Gsamples_per_s=n * 64 / ms_u / 1e6)
        _issue_bound(res["rng_uniform_f32_only_64"], n * 64 / (ms_u * 1e-3),
                     RNG_INSTR_PER_SAMPLE["rng_uniform_f32_only_64"], torch)
        # the other three draws of random.py:174-238, one kind per launch
        ms_d, _ = timed(fill(_lib.UNIFORM_F64, z.data_ptr(), 16), iters, warm)
        res["rng_uniform_f64_only_16"] = dict(_roof(n * (32 + 128), ms_d, peak), Gsamples_per_s=n * 16 / ms_d / 1e6)
        ms_d, _ = timed(fill(_lib.NORMAL_F32, u.data_ptr(), 64), iters, warm)
        res["rng_normal_f32_only_64"] = dict(_roof(n * (32 + 256), ms_d, peak), Gsamples_per_s=n * 64 / ms_d / 1e6,
                                             bound="issue")
        ms_d, _ = timed(fill(_lib.NORMAL_F64, z.data_ptr(), 16), iters, warm)
        res["rng_normal_f64_only_16"] = dict(_roof(n * (32 + 128), ms_d, peak), Gsamples_per_s=n * 16 / ms_d / 1e6,
                                             bound="issue")
        del u, z, states

    if want("n2"):
        # the callers either side of the path: device-side assignment (slice copies,
        # fills) and N-D axis permutations, all through b2k_assign
        import ctypes

        def assign(dst, src, shape, dstr, sstr, item):
            arr = ctypes.c_int64 * len(shape)
            check(L.b2k_assign(dst, src, len(shape), arr(*shape), arr(*dstr), arr(*sstr), item, sptr))

        def c_steps(shape, item):
            steps = [item] * len(shape)
            for k in range(len(shape) - 2, -1, -1):
                steps[k] = steps[k + 1] * shape[k + 1]
            return steps

        n = 1 << (28 - scale)
        a = torch.randn(n, device="cuda")
        b = torch.empty(n, device="cuda")
        ms, _ = timed(lambda: assign(b.data_ptr(), a.data_ptr(), [n], [4], [4], 4), iters, warm)
        res["n2_assign_copy_f32_2p28"] = dict(_roof(n * 8, ms, peak), spot_check=bool(torch.equal(a[:4096], b[:4096])))
        ms, _ = timed(lambda: assign(b.data_ptr(), a.data_ptr(), [n], [4], [0], 4), iters, warm)
        res["n2_assign_fill_scalar_f32_2p28"] = dict(_roof(n * 4, ms, peak), note="write-only: 4 B per item",
                                                     spot_check=bool((b[-4096:] == a[0]).all()))
        nbytes = n * 4 - 64
        ms, _ = timed(lambda: assign(b.data_ptr() + 1, a.data_ptr(), [nbytes], [1], [1], 1), iters, warm)
        res["n2_assign_copy_shifted_one_byte"] = dict(
            _roof(nbytes * 2, ms, peak), note="destination one byte off the source's alignment",
            spot_check=bool(torch.equal(b.view(torch.uint8)[1:4097], a.view(torch.uint8)[:4096])))
        rows = 16384 >> scale
        ms, _ = timed(lambda: assign(b.data_ptr(), a.data_ptr(), [rows // 2, 16384], [2 * 65536, 4], [2 * 65536, 4], 4),
                      iters, warm)
        res["n2_assign_every_other_row_f32"] = _roof(rows // 2 * 16384 * 8, ms, peak)
        ms, _ = timed(lambda: assign(b.data_ptr(), a.data_ptr(), [rows, 16384], [65536, 4], [0, 4], 4), iters, warm)
        res["n2_assign_row_to_every_row_f32"] = dict(_roof(rows * 16384 * 4, ms, peak), note="write-only: 4 B per item",
                                                     spot_check=bool(torch.equal(b[-16384:], a[:16384])))
        for label, shape, perm in (("n4_permute_021_f32_64x2048x2048", [64 >> scale, 2048, 2048], (0, 2, 1)),
                                   ("n4_permute_102_f32_2048x64x2048", [2048 >> scale, 64, 2048], (1, 0, 2)),
                                   ("n4_permute_210_f32_512x512x1024", [512 >> scale, 512, 1024], (2, 1, 0))):
            count = shape[0] * shape[1] * shape[2]
            src = a[:count].view(shape)
            in_steps = c_steps(shape, 4)
            out_shape = [shape[k] for k in perm]
            ms, _ = timed(lambda: assign(b.data_ptr(), src.data_ptr(), out_shape, c_steps(out_shape, 4),
                                         [in_steps[k] for k in perm], 4), iters, warm)
            got = b[:count].view(out_shape)
            res[label] = dict(_roof(count * 8, ms, peak),
                              spot_check=bool(torch.equal(got[:2, :64], src.permute(perm)[:2, :64])))
        rows = cols = 16384 >> (scale // 2)
        m = a[:rows * cols].view(rows, cols)
        zero32 = np.zeros(1, dtype=np.float32)
        for axis in (0, 1):
            need = int(L.b2k_reduce_axis_scratch_bytes(rows, cols, _lib.F32, axis))
            scr = torch.zeros(max(need, 256), dtype=torch.uint8, device="cuda")
            outv = torch.empty(cols if axis == 0 else rows, dtype=torch.float32, device="cuda")
            ms, _ = timed(lambda: check(L.b2k_reduce_axis(_lib.ADD, _lib.F32, m.data_ptr(), rows, cols, cols * 4, axis,
                                                          zero32.ctypes.data, outv.data_ptr(), scr.data_ptr(),
                                                          scr.numel(), sptr)), iters, warm)
            ref = m[:, :256].sum(dim=0) if axis == 0 else m[:256].sum(dim=1)
            res[f"n4_reduce_sum_axis{axis}_f32_16384x16384"] = dict(
                _roof(rows * cols * 4, ms, peak), spot_check=bool(torch.allclose(outv[:256], ref, rtol=1e-4, atol=1e-2)))
        # the middle axis of a batch of matrices: one launch over all slabs
        batch, length, inner = 256 >> scale, 1024, 1024
        need = int(L.b2k_reduce_cols_batched_scratch_bytes(batch, length, inner, _lib.F32))
        scr = torch.zeros(max(need, 256), dtype=torch.uint8, device="cuda")
        outv = torch.empty(batch * inner, dtype=torch.float32, device="cuda")
        ms, _ = timed(lambda: check(L.b2k_reduce_cols_batched(
            _lib.ADD, _lib.F32, a.data_ptr(), batch, length, inner, inner * 4, length * inner * 4, zero32.ctypes.data,
            outv.data_ptr(), scr.data_ptr(), scr.numel(), sptr)), iters, warm)
        ref = a[:length * inner].view(length, inner).sum(dim=0)
        res["n4_reduce_sum_middle_axis_f32_256x1024x1024"] = dict(
            _roof(batch * length * inner * 4, ms, peak),
            spot_check=bool(torch.allclose(outv[:inner], ref, rtol=1e-4, atol=1e-2)))
        del a, b

    if want("c5"):
        n = 1 << (30 - scale)
        x = torch.randn(n, device="cuda") * 4
        idx = torch.randint(0, n, (n // 100,), device="cuda")
        specials = torch.tensor([float("inf"), float("-inf"), float("nan"), 1e6, -1e6], device="cuda")
        x[idx] = specials[torch.arange(idx.numel(), device="cuda") % 5]
        del idx
        e = torch.empty(n, dtype=torch.uint8, device="cuda")
        h = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        back = torch.empty(n, dtype=torch.float32, device="cuda")
        for label, s, d, src, dst, bpe in (
                ("c5_cast_f32_to_e4m3", _lib.FMT_F32, _lib.FMT_E4M3, x, e, 5),
                ("c5_cast_e4m3_to_f32", _lib.FMT_E4M3, _lib.FMT_F32, e, back, 5),
                ("c5_cast_f32_to_e5m2", _lib.FMT_F32, _lib.FMT_E5M2, x, e, 5),
                ("c5_cast_f32_to_bf16", _lib.FMT_F32, _lib.FMT_BF16, x, h, 6),
                ("c5_cast_bf16_to_f32", _lib.FMT_BF16, _lib.FMT_F32, h, back, 6)):
            ms, _ = timed(lambda: check(L.b2k_cast(s, d, 1, src.data_ptr(), dst.data_ptr(), n, sptr)), iters, warm)
            res[label] = _roof(n * bpe, ms, peak)
        res["c5_cast_f32_to_bf16"]["matches_torch_on_finite"] = bool(
            torch.equal(h[:1 << 20].view(torch.int16)[torch.isfinite(x[:1 << 20])],
                        x[:1 << 20].to(torch.bfloat16).view(torch.int16)[torch.isfinite(x[:1 << 20])]))
        del back, h
        # float64 and bfloat16 sources of the fp8 encoder (cvt_double_to_fp8, cvt_bfloat16raw_to_fp8)
        nd = n // 2
        xd = x[:nd].double()
        ms, _ = timed(lambda: check(L.b2k_cast_ex(_lib.FMT_F64, _lib.FMT_E4M3, 1, 0, xd.data_ptr(), e.data_ptr(), nd,
                                                  sptr)), iters, warm)
        res["n1_cast_f64_to_e4m3"] = dict(_roof(nd * 9, ms, peak), elements=nd)
        del xd
        hb = x.to(torch.bfloat16)
        ms, _ = timed(lambda: check(L.b2k_cast_ex(_lib.FMT_BF16, _lib.FMT_E4M3, 1, 0, hb.data_ptr(), e.data_ptr(), n,
                                                  sptr)), iters, warm)
        res["n1_cast_bf16_to_e4m3"] = _roof(n * 3, ms, peak)
        del hb
        # integer sides: int32(fp8_e4m3) over the codes just written, fp8_e4m3(int32) and
        # int32_to_bfloat16_rn over the same integers
        ni = n // 2
        iv = torch.empty(ni, dtype=torch.int32, device="cuda")
        ms, _ = timed(lambda: check(L.b2k_cast_ex(_lib.FMT_E4M3, _lib.FMT_I32, 1, _lib.ROUND_ZERO, e.data_ptr(),
                                                  iv.data_ptr(), ni, sptr)), iters, warm)
        res["n1_cast_e4m3_to_int32"] = dict(_roof(ni * 5, ms, peak), elements=ni)
        ms, _ = timed(lambda: check(L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_E4M3, 1, 0, iv.data_ptr(), e.data_ptr(), ni,
                                                  sptr)), iters, warm)
        res["n1_cast_int32_to_e4m3"] = dict(_roof(ni * 5, ms, peak), elements=ni)
        hb = torch.empty(ni, dtype=torch.bfloat16, device="cuda")
        ms, _ = timed(lambda: check(L.b2k_cast_ex(_lib.FMT_I32, _lib.FMT_BF16, 1, 0, iv.data_ptr(), hb.data_ptr(), ni,
                                                  sptr)), iters, warm)
        res["n1_cast_int32_to_bf16"] = dict(_roof(ni * 6, ms, peak), elements=ni)
        del x, e, hb, iv
    torch.cuda.empty_cache()
    return res


def run_single_path(args, cuda, L, torch, timed, peak, peak_kind, sptr):
    """Profiling aid: run one configuration, optionally shrunk, and print its numbers."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.only == "c2":
        from numba_cuda_b200 import _lib
        n = N_C2 >> args.scale
        x = torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), dtype=torch.int32, device="cuda")
        scratch = torch.zeros(int(L.b2k_reduce_scratch_bytes()), dtype=torch.uint8, device="cuda")
        out = torch.zeros(1, dtype=torch.int32, device="cuda")
        ident = np.array([-2 ** 31], dtype=np.int32)

        def k():
            rc = L.b2k_reduce(_lib.MAX, _lib.I32, x.data_ptr(), n, ident.ctypes.data, out.data_ptr(),
                              scratch.data_ptr(), scratch.numel(), sptr)
            if rc:
                raise RuntimeError(L.b2k_last_error())
        ms, _ = timed(k, args.steps, args.warmup)
        assert int(out.item()) == int(x.max().item())
        res = {"c2_reduce_max_int32": _roof(n * 4, ms, peak)}
    else:
        res = secondary_paths(cuda, L, torch, timed, peak, world, rank, sptr, only=args.only, scale=args.scale)
    if rank == 0:
        print(json.dumps({"only": args.only, "scale": args.scale, "peak": peak, "peak_kind": peak_kind,
                          "paths": res}), flush=True)


if __name__ == "__main__":
    main()
