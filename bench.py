#!/usr/bin/env python
"""Benchmark of the fp64 MLP training hot path (benchmark config 4).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: MLP 784 -> 1024 -> 1024 -> 10, ReLU hidden layers, softmax
cross-entropy, global batch 65536 split by rows over N GPUs (one process per
GPU under torch.distributed.run), plain SGD lr 0.01; inputs uniform[0,1),
labels uniform 0..9, weights N(0, 1/sqrt(fan_in)), biases 0, all seeded and
synthetic.  One step = forward + backward + gradient all-reduce + SGD update on
one global batch.

Beside it the line carries the other configs of the benchmark: `c5` (inference of
the 784-128-64-10 MLP on 1,048,576 inputs sharded over the N ranks, with a
checksum of the class ids that must be the same at every N), `c1` (batch-32
train step, N=1) and `sweeps` (DGEMM TFLOP/s and elementwise GB/s, N=1).

Prints ONE JSON line on rank 0:
  value      samples/s with the batch already resident in HBM (device-timed with
             events on the library's compute stream, max over ranks)
  e2e        the same step through the public Tensor API with HOST batches: every
             step copies its shard of X and the labels from pinned host memory
             and reads the loss back
  roofline   the dominant kernel (FP64 tensor-core GEMM), timed alone on the
             layer-2 forward shape, against the FP64 MMA issue rate measured on
             this device and the nominal FP64 peak
  cpu_baseline  the reference's own compiled CPU code (one thread, as it is
             written) on a bounded sample; cpu_baseline_all_cores is the
             order-preserving CPU port on every host core

`--impl reference` times the reference's own CPU implementation (oracle/_ref,
single-threaded as the reference is) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import gc
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SIZES = [784, 1024, 1024, 10]
GLOBAL_BATCH = 65536
LR = 0.01
# Useful flop per sample: forward 2*(784*1024+1024*1024+1024*10), the same again for
# the weight gradients, and the input gradients of the two hidden layers.
FLOP_PER_SAMPLE = 9_564_160
NOMINAL_FP64_TFLOPS = 148 * 128 * 1.965e9 / 1e12  # 148 SMs x 128 flop/clk x 1.965 GHz = 37.2
METRIC = "fp64_mlp_train_samples_per_s"


def make_params(seed=1234):
    rng = np.random.default_rng(seed)
    return [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o))
            for i, o in zip(SIZES[:-1], SIZES[1:])]


def make_batch(rows, seed):
    rng = np.random.default_rng(seed)
    return rng.random((rows, SIZES[0])), rng.integers(0, 10, rows).astype(np.int32)


BATCH_BLOCK = 4096


def global_batch_rows(begin, end, seed=1000):
    """Rows [begin, end) of THE global batch.  Block b of 4096 rows is drawn from
    generator seed + b, so every rank — at any world size — sees the same rows of
    the same batch and only generates the blocks it owns."""
    xs, ys = [], []
    for b in range(begin // BATCH_BLOCK, (end + BATCH_BLOCK - 1) // BATCH_BLOCK):
        X, y = make_batch(BATCH_BLOCK, seed + b)
        lo, hi = max(begin, b * BATCH_BLOCK), min(end, (b + 1) * BATCH_BLOCK)
        xs.append(X[lo - b * BATCH_BLOCK:hi - b * BATCH_BLOCK])
        ys.append(y[lo - b * BATCH_BLOCK:hi - b * BATCH_BLOCK])
    if not xs:
        return np.zeros((0, SIZES[0])), np.zeros(0, dtype=np.int32)
    return np.ascontiguousarray(np.concatenate(xs)), np.ascontiguousarray(np.concatenate(ys))


def uniform01_host(seed, first, n):
    """Host twin of mg_fill_uniform01 (splitmix64, top 53 bits)."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + np.arange(first + 1, first + n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(11)).astype(np.float64) * 2.0 ** -53


def best_and_median(abi, fn, reps=10, warm=2, before=None, inner=1):
    """Device time (ms) per launch of fn() over `reps` repeats, each repeat a run of
    `inner` back-to-back launches bracketed by one event pair on the library's
    compute stream (an event pair costs several microseconds, which `inner` > 1
    spreads over short kernels); `before` runs untimed ahead of every repeat (an
    L2 flush).  Returns (best, median)."""
    for _ in range(warm):
        fn()
    times = []
    for _ in range(reps):
        if before:
            before()
        times.append(abi.timed_ms(fn, inner) / inner)
    return min(times), float(np.median(times))


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, power and throttle reasons while a region runs.

    Uses NVML in-process (a light query every 100 ms from a thread); falls back to
    an `nvidia-smi -lms` child process when the NVML binding is unavailable.
    MG_BENCH_SAMPLER=smi|nvml|none overrides the choice."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.rows, self.proc, self.thread = index, [], None, None
        self.mode = os.environ.get("MG_BENCH_SAMPLER", "nvml")
        self._stop = threading.Event()

    def start(self):
        if self.mode == "none":
            return
        if self.mode == "nvml":
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nvml = pynvml
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
                self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
                self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
                self.thread.start()
                return
            except Exception:
                self.mode = "smi"
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _poll_nvml(self):
        nv = self._nvml
        bits = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                "sw_power_cap": 0x4}
        while not self._stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                pw = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                flags = ["Active" if mask & bits[n] else "Not Active" for n in self.NAMES]
                self.rows.append([str(sm), str(self._max), str(pw)] + flags)
            except Exception:
                pass
            self._stop.wait(0.1)

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.mode == "none" or (self.proc is None and self.thread is None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["sampler unavailable"]}
        time.sleep(0.15)
        self._stop.set()
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread:
            self.thread.join(timeout=2)
        ok = lambda v: v.replace(".", "").isdigit()
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and ok(r[0])]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and ok(r[1])]
        pw = [float(r[2]) for r in self.rows if len(r) >= 7 and ok(r[2])]
        reasons = [n for i, n in enumerate(self.NAMES)
                   if any(len(r) >= 7 and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None,
                "samples": len(sm), "sampler": self.mode, "reasons": reasons}


# --------------------------------------------------------------------------- product arm
def build_model(api, params):
    layers = []
    for W, b in params:
        lin = api.Linear(W.shape[0], W.shape[1])
        lin.weights().set_data(W)
        lin.bias().set_data(b)
        layers.append(lin)
    opt = api.SGD([t for lin in layers for t in (lin.weights(), lin.bias())], LR)
    opt.enable_allreduce()
    return layers, opt


def train_step(api, layers, opt, x, labels, denom):
    h = layers[0].forward_relu(x)
    h = layers[1].forward_relu(h)
    loss = api.softmax_cross_entropy(layers[2].forward(h), labels, denom)
    opt.zero_grad()
    loss.backward()
    opt.step()
    return loss


def run_product(args):
    import torch
    import torch.distributed as dist

    import micrograd_b200
    from micrograd_b200 import cabi as K
    from micrograd_b200.dist import (bind_near_gpu, env_rank_world, init_comm, max_over_ranks,
                                     shard_rows)

    rank, world, local_rank = env_rank_world()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    # Before any pinned allocation: stay on the CPUs next to this rank's GPU (only
    # in multi-rank jobs; a single rank keeps every core for the CPU baselines).
    placement = bind_near_gpu(local_rank) if world > 1 else {"bound": False, "cpus": os.cpu_count()}
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    abi = micrograd_b200.load_abi()
    abi.mg_init(local_rank)
    api = micrograd_b200.load_api()
    if world > 1:
        init_comm(api)

    def barrier():
        abi.mg_sync()
        if world > 1:
            dist.barrier()
        abi.mg_sync()

    def sum_over_ranks(value, dtype=None):
        if world == 1:
            return value
        t = torch.tensor([value], dtype=dtype or torch.float64, device="cuda")
        dist.all_reduce(t)
        return t.item()

    def min_over_ranks(value):
        return -max_over_ranks(-float(value))

    batch = args.batch
    b0, b1 = shard_rows(batch, rank, world)
    rows = b1 - b0
    layers, opt = build_model(api, make_params())
    X, y = global_batch_rows(b0, b1)          # this rank's rows of the one global batch

    # ---- value: inputs resident in HBM ----
    x_dev = api.Tensor([rows, SIZES[0]], X)
    x_dev.set_requires_grad(False)
    y_dev = api.Tensor([rows], y.astype(np.float64))
    # The clock sampler is started before the warm-up: the first NVML query of a
    # new nvidia-smi process stalls kernel launches for tens of milliseconds, which
    # must not land inside the timed region.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(1.0)
    # Warm-up with the timed loop's object lifetimes: `loss` keeps the previous step's
    # graph alive while the next one is built, so the memory pool reaches its steady
    # size here and not (by a slow driver allocation) inside the timed region.
    # The losses of the first three steps are kept: they start from the seeded
    # parameters on the one global batch, so they are the same numbers at every
    # world size (up to the order in which the ranks' partial sums are added).
    loss = None
    first_losses = []
    for i in range(args.warmup):
        loss = train_step(api, layers, opt, x_dev, y_dev, batch)
        if i < 3:
            first_losses.append(sum_over_ranks(float(loss.data()[0])))
    barrier()
    if rank == 0:
        sampler.rows.clear()          # keep only samples taken under the timed load
    launches0 = abi.mg_launch_count()
    if world > 1:
        abi.mg_comm_trace(1)
    # one event per step boundary: the total is first-to-last, the per-step
    # spread shows whether a slow run was slow throughout
    marks = []
    for _ in range(args.steps + 1):
        ev = C.c_int()
        abi.mg_event_create(C.byref(ev))
        marks.append(ev.value)
    abi.mg_event_record(marks[0])
    for i in range(args.steps):
        loss = train_step(api, layers, opt, x_dev, y_dev, batch)
        if args.sync_each_step:
            abi.mg_sync()
        abi.mg_event_record(marks[i + 1])
    ms = C.c_float()
    abi.mg_event_elapsed_ms(marks[0], marks[-1], C.byref(ms))
    per_step = []
    for i in range(args.steps):
        t = C.c_float()
        abi.mg_event_elapsed_ms(marks[i], marks[i + 1], C.byref(t))
        per_step.append(float(t.value))
    for ev in marks:
        abi.mg_event_destroy(ev)
    barrier()
    launches = abi.mg_launch_count() - launches0
    exchange_timing = None
    if world > 1:
        ex_ms, ex_n, wait_ms, wait_n = C.c_double(), C.c_int(), C.c_double(), C.c_int()
        abi.mg_comm_trace_summary(C.byref(ex_ms), C.byref(ex_n), C.byref(wait_ms), C.byref(wait_n))
        abi.mg_comm_trace(0)
        # slowest rank for both: the all-reduce kernels' own duration (they overlap the
        # backward GEMMs) and the time the compute stream stood waiting for them
        exchange_timing = {
            "allreduce_ms_per_step": max_over_ranks(ex_ms.value / args.steps),
            "allreduces_per_step": ex_n.value / args.steps,
            "exposed_wait_ms_per_step": max_over_ranks(wait_ms.value / args.steps),
            "what": "event pairs on the communication stream around each all-reduce, and on the compute "
                    "stream around each wait for it; max over ranks"}
    clocks = sampler.stop() if rank == 0 else None
    total_ms = max_over_ranks(float(ms.value))
    step_spread = {"min": min(per_step), "median": float(np.median(per_step)), "max": max(per_step)}
    # each rank's loss is its share of the global mean (divisor = global batch)
    final_loss = sum_over_ranks(float(loss.data()[0]))
    abi.mg_check_kernel_status()
    del x_dev, y_dev, loss

    if args.value_only:
        if world > 1:
            api.comm_shutdown()
            dist.destroy_process_group()
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": batch * args.steps / (total_ms * 1e-3),
                              "unit": "samples/s", "n_gpus": world, "steps": args.steps,
                              "ms_per_step": total_ms / args.steps, "ms_per_step_spread": step_spread,
                              "gpu_launches": int(launches), "clocks": clocks,
                              "first_losses": first_losses, "final_loss": final_loss,
                              "config": {"global_batch": batch, "value_only": True}}), flush=True)
        return

    # ---- e2e: host batches through the public API ----
    nbytes = rows * SIZES[0] * 8
    # Two pinned staging buffers: while step i computes, the batch of step i+1 is
    # copied on the library's copy stream (Tensor::prefetch_from_host), so each timed step
    # contains one full host->device batch copy and one device->host loss read.
    pinned = [C.c_void_p(), C.c_void_p()]
    for pbuf in pinned:
        abi.mg_host_alloc(nbytes, C.byref(pbuf))
        host_x = np.ctypeslib.as_array(C.cast(pbuf.value, C.POINTER(C.c_double)),
                                       shape=(rows, SIZES[0]))
        host_x[...] = X
    e2e_steps = max(3, min(args.steps, 20))

    # Two input tensors, created once and refreshed in turn (Tensor::prefetch_from_host):
    # no batch tensor is allocated or freed inside the loop.
    inputs = [api.from_host([rows, SIZES[0]], pbuf.value) for pbuf in pinned]
    for x in inputs:
        x.set_requires_grad(False)

    uploads = [0]

    def upload():
        i = uploads[0] % 2                               # the buffer the previous step did not use
        uploads[0] += 1
        inputs[i].prefetch_from_host(pinned[i].value)
        return inputs[i]

    def e2e_loop(n, x_next):
        # Software-pipelined, as a training loop that logs its loss would be: the batch of
        # step i+1 is uploading and the loss of step i-1 is read back while step i runs,
        # so the device never waits for the host.  Every step's loss is read.
        pending = None
        for i in range(n):
            x_cur, x_next = x_next, upload()            # prefetch the next batch
            out = train_step(api, layers, opt, x_cur, y, batch)
            if pending is not None:
                float(pending.data()[0])                 # device -> host read of a loss
                e2e_marks.append(time.perf_counter())
            pending = out
        float(pending.data()[0])
        e2e_marks.append(time.perf_counter())
        return x_next

    e2e_marks = []
    x_next = e2e_loop(3, upload())
    # As timeit does: no garbage-collector pass inside the host-timed region (the
    # loop makes a few hundred short-lived wrapper objects per step, and a full
    # collection over an interpreter with torch loaded takes milliseconds).
    gc.collect()
    gc.disable()
    barrier()
    e2e_marks.clear()
    t0 = time.perf_counter()
    x_next = e2e_loop(e2e_steps, x_next)
    abi.mg_sync()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    gc.enable()
    # host time between consecutive loss reads on this rank (rank 0's view in the line)
    e2e_gaps = np.diff(np.array([t0] + e2e_marks)) * 1e3
    if os.environ.get("MG_E2E_DIAG"):
        print(f"E2E_DIAG rank {rank}: " + " ".join(f"{g:.1f}" for g in e2e_gaps), file=sys.stderr, flush=True)
    barrier()
    del x_next, inputs
    abi.mg_sync()

    # The host->device leg alone, every rank copying its shard at the same moment:
    # what the host side (PCIe root, memory of the socket the buffers sit on) gives
    # each GPU when all N pull at once.
    staging = abi.empty(rows * SIZES[0])
    copy = lambda: abi.mg_upload(staging.ptr, pinned[0].value, rows * SIZES[0])
    copy()
    barrier()
    h2d_best, h2d_median = best_and_median(abi, copy, reps=6, warm=1)
    h2d_ms_slowest = max_over_ranks(h2d_median)
    h2d = {"bytes": nbytes, "ms_median_slowest_rank": h2d_ms_slowest,
           "gbs_per_rank_slowest": nbytes / h2d_ms_slowest / 1e6,
           "gbs_per_rank_fastest": nbytes / min_over_ranks(h2d_best) / 1e6,
           "gbs_aggregate": world * nbytes / h2d_ms_slowest / 1e6,
           "what": "one cudaMemcpyAsync of the rank's pinned shard per measurement, all ranks at once"}
    del staging
    barrier()
    for pbuf in pinned:
        abi.mg_host_free(pbuf.value)

    # ---- config 5: sharded inference (all ranks) ----
    # The legs below stand beside the headline; a failure in one of them is reported
    # in its place in the JSON line instead of losing the whole line.  (All ranks run
    # the same code on the same shapes, so a failure is the same on every rank.)
    def guarded(fn, *a):
        try:
            return fn(*a)
        except Exception as exc:  # noqa: BLE001 - anything: the error text goes into the line
            return {"error": f"{type(exc).__name__}: {exc}"[:400]}

    c5 = None if args.no_c5 else guarded(inference_leg, abi, K, rank, world, barrier, max_over_ranks,
                                         sum_over_ranks, shard_rows)

    # ---- roofline of the dominant kernel, timed alone (rank 0) ----
    roofline = None
    cpu_baseline = cpu_all = None
    sweeps = c1 = None
    if rank == 0:
        roofline = guarded(gemm_roofline, abi, K, rows)
        if world == 1 and not args.no_sweeps:
            c1 = guarded(small_batch_leg, abi, api)
            sweeps = guarded(metric_sweeps, abi, K)
        if world == 1 and not args.no_cpu_baseline:
            cpu_baseline = guarded(reference_sample, 15.0)
            cpu_all = guarded(port_all_cores_sample, 10.0)
            if c5 is not None and "error" not in c5:
                c5["cpu_baseline"] = guarded(inference_cpu_sample, c5)

    exchange = "none (one rank)"
    if world > 1:
        exchange = ("peer-memory all-reduce kernel (rank-ordered sums over NVLink peer loads/stores)"
                    if abi.mg_comm_peer_path(None) else "ncclAllReduce")
        api.comm_shutdown()
        dist.destroy_process_group()
    if rank != 0:
        return
    ms_per_step = total_ms / args.steps
    value = batch * args.steps / (total_ms * 1e-3)
    out = {
        "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "ms_per_step_spread": step_spread,
        "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "MLP 784-1024-1024-10 fp64 train step (benchmark config 4)",
                   "global_batch": batch, "rows_per_gpu": rows, "lr": LR, "parallelism": f"dp{world}",
                   "gradient_exchange": exchange, "exchange_timing": exchange_timing, "input_grad": False,
                   "batch": "one seeded global batch (4096-row blocks); rank r holds its row shard",
                   "l2": "per-step working set (activations+gradients > 1 GB "
                   "at N=1, > 300 MB at N=8) exceeds the 126 MB L2"},
        "step_tflops": FLOP_PER_SAMPLE * batch / (ms_per_step * 1e-3) / 1e12 / world,
        # Global-mean losses (the ranks' shares summed).  first_losses are steps 1-3 from
        # the seeded parameters: equal at every world size up to summation order.
        # final_loss is the loss of the last timed step (after warmup + steps updates).
        "first_losses": first_losses, "final_loss": final_loss,
        "clocks": clocks,
        "e2e": {"value": batch * e2e_steps / (e2e_ms * 1e-3), "unit": "samples/s",
                "h2d_bytes_per_step": nbytes + rows * 4, "d2h_bytes_per_step": 8,
                "steps": e2e_steps, "timer": "host wall clock around blocking loss reads",
                "ms_between_loss_reads": {"min": float(e2e_gaps.min()), "median": float(np.median(e2e_gaps)),
                                          "max": float(e2e_gaps.max())},
                "inputs": "two input tensors refreshed in turn with Tensor::prefetch_from_host; nothing "
                          "is allocated per batch",
                "pipeline": "while step i runs, batch i+1 is copied from pinned memory on a copy stream and "
                            "the loss of step i-1 is read back; all losses are read inside the timed region",
                "h2d_alone": h2d, "placement": placement},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "cpu_baseline_all_cores": cpu_all,
        "c5": c5,
        "c1": c1,
        "sweeps": sweeps,
    }
    print(json.dumps(out), flush=True)


C1_SIZES = [784, 128, 64, 10]
C5_INPUTS = 1 << 20
C5_SEED = 20240605
C5_FLOP_PER_INPUT = 2 * (784 * 128 + 128 * 64 + 64 * 10)       # 218 368
CHECK_ROWS = 32768


def make_small_params(seed=4321):
    rng = np.random.default_rng(seed)
    return [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o))
            for i, o in zip(C1_SIZES[:-1], C1_SIZES[1:])]


def ids_checksum(ids, first_row):
    """sum of id * (global row + 1) — exact in 64-bit integers for a million rows."""
    rows = np.arange(first_row + 1, first_row + 1 + ids.size, dtype=np.int64)
    return int((ids.astype(np.int64) * rows).sum())


def inference_leg(abi, K, rank, world, barrier, max_over_ranks, sum_over_ranks, shard_rows):
    """Benchmark config 5: forward pass of the 784-128-64-10 MLP (random-init
    weights) on 1,048,576 uniform[0,1) inputs, rows sharded over the ranks with no
    exchange, class id = first strict row maximum (src/main.cpp:29-32 of the
    reference).  Inputs are generated on each GPU from (seed, global element
    index), so every world size classifies the same million rows; the checksum
    sum(id * (row + 1)) over all rows must therefore be identical at N = 1, 2, 4, 8.
    Three fused Linear GEMMs (bias / bias+ReLU epilogues) + argmax per pass, the
    same entry points Linear::forward uses."""
    import torch
    r0, r1 = shard_rows(C5_INPUTS, rank, world)
    rows = r1 - r0
    params = make_small_params()
    X = abi.empty(rows * 784)
    abi.mg_fill_uniform01(X.ptr, rows * 784, C5_SEED, r0 * 784)
    W = [abi.array(w) for w, _ in params]
    B = [abi.array(b) for _, b in params]
    h1, h2, z = abi.empty(rows * 128), abi.empty(rows * 64), abi.empty(rows * 10)
    ids = abi.int_array(np.zeros(rows, dtype=np.int32))

    def forward():
        abi.mg_gemm_nn(X.ptr, W[0].ptr, h1.ptr, rows, 128, 784, 0, K.EPI_BIAS_RELU, B[0].ptr)
        abi.mg_gemm_nn(h1.ptr, W[1].ptr, h2.ptr, rows, 64, 128, 0, K.EPI_BIAS_RELU, B[1].ptr)
        abi.mg_gemm_nn(h2.ptr, W[2].ptr, z.ptr, rows, 10, 64, 0, K.EPI_BIAS, B[2].ptr)
        abi.mg_argmax_rows(z.ptr, ids.ptr, rows, 10)

    for _ in range(2):
        forward()
    barrier()
    reps = 5
    ms = max_over_ranks(abi.timed_ms(lambda: [forward() for _ in range(reps)], 1)) / reps
    barrier()
    t0 = time.perf_counter()
    forward()
    got = ids.numpy()                                   # device -> host, 4 bytes per input
    ms_ids = max_over_ranks((time.perf_counter() - t0) * 1e3)
    abi.mg_check_kernel_status()
    checksum = int(sum_over_ranks(ids_checksum(got, r0), torch.int64)) % (1 << 61)
    histogram = [int(sum_over_ranks(int((got == c).sum()), torch.int64)) for c in range(10)]
    first = ids_checksum(got[:CHECK_ROWS], 0) if rank == 0 and rows >= CHECK_ROWS else None
    tflops = C5_FLOP_PER_INPUT * C5_INPUTS / (ms * 1e-3) / 1e12
    return {"workload": "inference 784-128-64-10 fp64 on 1,048,576 inputs (benchmark config 5)",
            "inputs": C5_INPUTS, "rows_per_gpu": rows, "ms": ms, "inputs_per_s": C5_INPUTS / (ms * 1e-3),
            "tflops_per_gpu": tflops / world, "frac_of_nominal_fp64": tflops / world / NOMINAL_FP64_TFLOPS,
            "input_gbs_per_gpu": rows * 784 * 8 / (ms * 1e-3) / 1e9,
            "ms_with_ids_on_host": ms_ids, "d2h_bytes": rows * 4,
            "ids_checksum": checksum, "ids_checksum_first_32768": first, "ids_histogram": histogram,
            "inputs_source": "mg_fill_uniform01 (splitmix64 of seed and global element index), resident in HBM",
            "scaling": "strong, no exchange"}


def inference_cpu_sample(c5):
    """CPU leg of config 5: the order-preserving CPU port (all cores) classifies the
    first 32768 inputs — regenerated on the host from the same integer formula — is
    timed, and its class ids are compared with the GPU's through the checksum."""
    import oracle
    oracle.fast.set_num_threads(os.cpu_count() or 1)
    X = uniform01_host(C5_SEED, 0, CHECK_ROWS * 784).reshape(CHECK_ROWS, 784)
    params = make_small_params()
    t0 = time.perf_counter()
    logits, _ = oracle.fast.mlp_forward(params, X)
    ids = oracle.fast.argmax_rows(logits)
    dt = time.perf_counter() - t0
    expect = ids_checksum(ids, 0)
    return {"value": CHECK_ROWS / dt, "unit": "inputs/s", "cores": oracle.fast.num_threads(), "kind": "port",
            "sample": f"first {CHECK_ROWS} of the 1,048,576 inputs", "ids_checksum_first_32768": expect,
            "ids_equal_gpu": bool(expect == c5.get("ids_checksum_first_32768"))}


def small_batch_leg(abi, api):
    """Benchmark config 1: one SGD step of the 784-128-64-10 MLP at batch 32
    through the public Tensor API (forward, softmax cross-entropy, backward, SGD).
    Launch-bound: the figure that matters is microseconds per step."""
    params = make_small_params()
    layers = []
    for W, b in params:
        lin = api.Linear(W.shape[0], W.shape[1])
        lin.weights().set_data(W)
        lin.bias().set_data(b)
        layers.append(lin)
    opt = api.SGD([t for lin in layers for t in (lin.weights(), lin.bias())], LR)
    rng = np.random.default_rng(32)
    x = api.Tensor([32, 784], rng.random((32, 784)))
    x.set_requires_grad(False)
    y = api.Tensor([32], rng.integers(0, 10, 32).astype(np.float64))

    def step():
        h = layers[1].forward_relu(layers[0].forward_relu(x))
        loss = api.softmax_cross_entropy(layers[2].forward(h), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss

    for _ in range(20):
        loss = step()
    abi.mg_sync()
    n = 300
    l0 = abi.mg_launch_count()
    t0 = time.perf_counter()
    dev_ms = abi.timed_ms(lambda: [step() for _ in range(n)], 1)
    wall_ms = (time.perf_counter() - t0) * 1e3
    launches = (abi.mg_launch_count() - l0) / n
    flop = 454_400 * 32          # forward + weight gradients + hidden input gradients
    out = {"workload": "MLP 784-128-64-10 fp64 train step at batch 32 (benchmark config 1)",
           "us_per_step": dev_ms * 1e3 / n, "us_per_step_host_wall": wall_ms * 1e3 / n,
           "samples_per_s": 32 * n / (dev_ms * 1e-3), "launches_per_step": launches,
           "frac_of_nominal_fp64": flop / (dev_ms * 1e-3 / n) / 1e12 / NOMINAL_FP64_TFLOPS,
           "bound": "kernel-launch latency (a chain of dependent micro-kernels, see launches_per_step)"}
    # The same step recorded once (CUDA graph) and replayed with one launch per step.
    del loss
    rec = api.RecordedStep()
    try:
        rec.begin()
        loss = step()
        rec.end()
        for _ in range(20):
            rec.replay()
        abi.mg_sync()
        t0 = time.perf_counter()
        rec_ms = abi.timed_ms(lambda: [rec.replay() for _ in range(n)], 1)
        rec_wall_ms = (time.perf_counter() - t0) * 1e3
        float(loss.data()[0])
        out["recorded_step"] = {
            "us_per_step": rec_ms * 1e3 / n, "us_per_step_host_wall": rec_wall_ms * 1e3 / n,
            "samples_per_s": 32 * n / (rec_ms * 1e-3), "kernels_per_replay": rec.kernels(),
            "what": "the same step recorded once with RecordedStep (a CUDA graph) and replayed: "
                    "one launch per step"}
    except RuntimeError as exc:       # reported, not fatal: this leg is beside the headline
        rec.abandon()
        out["recorded_step"] = {"error": str(exc)[:300]}
    return out


def gemm_roofline(abi, K, rows):
    """Layer-2 forward GEMM [rows x 1024].[1024 x 1024] (bias+ReLU epilogue), the
    shape that dominates the step, timed alone with events; inputs (rows*8 KB,
    512 MB at 65536 rows) exceed L2."""
    M, N, Kd = rows, 1024, 1024
    rng = np.random.default_rng(7)
    A = abi.array(rng.standard_normal((min(M, 4096), Kd)))  # tile a smaller host array over M
    big = abi.empty(M * Kd)
    chunk = min(M, 4096) * Kd
    for off in range(0, M * Kd, chunk):
        abi.mg_copy(big.offset(off), A.ptr, min(chunk, M * Kd - off))
    B = abi.array(rng.standard_normal((Kd, N)) / 32.0)
    bias = abi.zeros(N)
    out = abi.empty(M * N)
    call = lambda: abi.mg_gemm_nn(big.ptr, B.ptr, out.ptr, M, N, Kd, 0, K.EPI_BIAS_RELU, bias.ptr)
    for _ in range(3):
        call()
    reps = 10
    ms = abi.timed_ms(call, reps) / reps
    achieved = 2.0 * M * N * Kd / (ms * 1e-3) / 1e12
    probe = {}
    for shape, name in enumerate(("m8n8k4", "m16n8k4", "m16n8k8", "m16n8k16")):
        t = C.c_double()
        abi.mg_probe_dmma_tflops(shape, 4000, C.byref(t))
        probe[name] = round(t.value, 3)
    measured_peak = max(probe.values())
    return {"bound": "tensor", "kernel": "dmma_gemm_kernel (layer-2 forward, bias+ReLU epilogue)",
            "achieved": achieved, "peak": measured_peak, "unit": "TFLOP/s",
            "frac": achieved / measured_peak,
            "peak_source": "FP64 mma.sync issue rate measured on this device by mg_probe_dmma_tflops "
                           "(MEASURED_PEAKS.json has no FP64 entry)",
            "peak_nominal": NOMINAL_FP64_TFLOPS, "frac_of_nominal": achieved / NOMINAL_FP64_TFLOPS,
            "ms_per_launch": ms, "flop_per_launch": 2.0 * M * N * Kd, "dmma_probe_tflops": probe,
            # Not measured in this run: dram__bytes_read.sum + dram__bytes_write.sum of this
            # kernel from an ncu capture at 32768 rows (277.1 + 233.9 MB), scaled by the rows of
            # this launch — traffic grows in proportion to the batch, the 8 MB weight operand
            # stays L2-resident.
            "traffic": 510.1e6 * M / 32768.0,
            "traffic_algorithmic": 8.0 * (M * Kd + Kd * N + M * N),
            "traffic_source": "constant from an ncu capture of this kernel at batch 32768, scaled by rows; "
                              "not re-measured by this run"}


def _measured_hbm_peak():
    """Measured copy bandwidth of this pool's B200s (GB/s): MEASURED_PEAKS.json beside
    this file when present, else the figure that file held when this was written."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6540.2


HBM_PEAK_GBS = _measured_hbm_peak()


def metric_sweeps(abi, K, small=False):
    """The other two parts of the headline metric, measured on one GPU:
    DGEMM TFLOP/s (forward C = A.B, and forward + both gradients; benchmark config 3
    shapes) and elementwise / reduction GB/s (benchmark config 2 ops, forward and
    backward, at 2^20, 2^24 and 2^28 elements).  Every entry is the best and the
    median of 10 repeats; a repeat is one event pair around 20 / 5 / 2 back-to-back
    launches at 2^20 / 2^24 / 2^28 (one launch for the GEMMs except 1024^3: 5).
    Algorithmic bytes per element: binary forward 24, unary forward 16, sums 8,
    backward passes as listed below.  Arrays at 2^24 and 2^28 exceed L2.  The 8 MB
    arrays of 2^20 stay L2-resident when launched back to back, so their GB/s is
    an L2 figure ("l2_resident": true, no HBM fraction); "us_cold" is a single
    launch after an L2 flush, event-pair overhead included."""
    rng = np.random.default_rng(11)
    seed = abi.array(rng.standard_normal(1 << 22))

    def filled(n):
        buf = abi.empty(n)
        for off in range(0, n, 1 << 22):
            abi.mg_copy(buf.offset(off), seed.ptr, min(1 << 22, n - off))
        return buf

    out = {"dgemm_tflops": {}, "dgemm_fwd_bwd_tflops": {}, "elementwise_gbs": {},
           "timing": "best / median of 10 repeats; a repeat = one event pair around 20 / 5 / 2 back-to-back "
                     "launches at 2^20 / 2^24 / 2^28 elements",
           "hbm_peak_gbs": HBM_PEAK_GBS}
    gemm_cases = (("1024^3", (1024, 1024, 1024)), ("4096^3", (4096, 4096, 4096)),
                  ("8192^3", (8192, 8192, 8192)), ("65536x784.784x1024", (65536, 1024, 784)))
    # small=True: the 2^24 / 2^26 elementwise cases only (what a profiler capture needs)
    for tag, (m, n, k) in (() if small else gemm_cases):
        a, b, c = filled(m * k), filled(k * n), abi.empty(m * n)
        inner = 5 if m * n * k <= 1024 ** 3 else 1
        best, med = best_and_median(
            abi, lambda: abi.mg_gemm_nn(a.ptr, b.ptr, c.ptr, m, n, k, 0, K.EPI_NONE, None), inner=inner)
        flop = 2.0 * m * n * k
        out["dgemm_tflops"][tag] = {"best": round(flop / best / 1e9, 2), "median": round(flop / med / 1e9, 2),
                                    "frac_of_nominal": round(flop / med / 1e9 / NOMINAL_FP64_TFLOPS, 3)}
        # forward plus both gradients (dA += G.B^T, dB += A^T.G; G = dC), 6 M N K flop
        g, da, db = filled(m * n), filled(m * k), filled(k * n)

        def fwd_bwd():
            abi.mg_gemm_nn(a.ptr, b.ptr, c.ptr, m, n, k, 0, K.EPI_NONE, None)
            abi.mg_gemm_nt(g.ptr, b.ptr, da.ptr, m, n, k, 1, K.EPI_NONE, None)
            abi.mg_gemm_tn(a.ptr, g.ptr, db.ptr, m, n, k, 1)

        best, med = best_and_median(abi, fwd_bwd, inner=inner)
        out["dgemm_fwd_bwd_tflops"][tag] = {"best": round(3 * flop / best / 1e9, 2),
                                            "median": round(3 * flop / med / 1e9, 2),
                                            "frac_of_nominal": round(3 * flop / med / 1e9 / NOMINAL_FP64_TFLOPS, 3)}
        del a, b, c, g, da, db
    for log2n in ((24, 26) if small else (20, 24, 28)):
        n = 1 << log2n
        a, b, g, o, o2 = filled(n), filled(n), filled(n), filled(n), filled(n)
        side = 1 << (log2n // 2)
        ops = (("add", lambda: abi.mg_binary_fwd(K.ADD, a.ptr, b.ptr, o.ptr, n), 24),
               ("mul", lambda: abi.mg_binary_fwd(K.MUL, a.ptr, b.ptr, o.ptr, n), 24),
               ("sub", lambda: abi.mg_binary_fwd(K.SUB, a.ptr, b.ptr, o.ptr, n), 24),
               ("relu", lambda: abi.mg_unary_fwd(K.RELU, a.ptr, 0.0, o.ptr, n), 16),
               ("tanh", lambda: abi.mg_unary_fwd(K.TANH, a.ptr, 0.0, o.ptr, n), 16),
               ("exp", lambda: abi.mg_unary_fwd(K.EXP, a.ptr, 0.0, o.ptr, n), 16),
               ("add_row", lambda: abi.mg_add_row_fwd(a.ptr, b.ptr, o.ptr, side, side), 16),
               ("sum", lambda: abi.mg_sum_all_fwd(a.ptr, o.ptr, n), 8),
               ("sum_lastaxis", lambda: abi.mg_sum_lastaxis_fwd(a.ptr, o.ptr, side, side), 8),
               ("mul_bwd_one_side", lambda: abi.mg_binary_bwd(K.MUL, a.ptr, b.ptr, g.ptr, o.ptr, None,
                                                               n, 0), 40),
               # backward passes, accumulating into existing gradients (read-modify-write):
               # add 40 B/element (g; ga, gb), mul 56 (g, a, b; ga, gb), unary 32 (g, x or y; gx),
               # row broadcast 24 (g; gx) + the [N] row gradient, sums 16 (gx)
               ("add_bwd", lambda: abi.mg_binary_bwd(K.ADD, a.ptr, b.ptr, g.ptr, o.ptr, o2.ptr, n, 0), 40),
               ("mul_bwd", lambda: abi.mg_binary_bwd(K.MUL, a.ptr, b.ptr, g.ptr, o.ptr, o2.ptr, n, 0), 56),
               ("relu_bwd", lambda: abi.mg_unary_bwd(K.RELU, a.ptr, b.ptr, 0.0, g.ptr, o.ptr, n, 0), 32),
               ("tanh_bwd", lambda: abi.mg_unary_bwd(K.TANH, a.ptr, b.ptr, 0.0, g.ptr, o.ptr, n, 0), 32),
               ("exp_bwd", lambda: abi.mg_unary_bwd(K.EXP, a.ptr, b.ptr, 0.0, g.ptr, o.ptr, n, 0), 32),
               ("add_row_bwd", lambda: abi.mg_add_row_bwd(g.ptr, o.ptr, o2.ptr, side, side, 0), 24),
               ("sum_bwd", lambda: abi.mg_sum_all_bwd(g.ptr, o.ptr, n, 0), 16),
               ("sum_lastaxis_bwd", lambda: abi.mg_sum_lastaxis_bwd(g.ptr, o.ptr, side, side, 0), 16))
        inner = {20: 20, 24: 5}.get(log2n, 2)
        for name, fn, bytes_per in ops:
            best, med = best_and_median(abi, fn, inner=inner)
            entry = {"best": round(bytes_per * n / best / 1e6, 1),
                     "median": round(bytes_per * n / med / 1e6, 1), "us": round(med * 1e3, 2)}
            if log2n == 20:
                _, cold = best_and_median(abi, fn, before=abi.mg_flush_l2)
                entry.update({"l2_resident": True, "us_cold": round(cold * 1e3, 2)})
            else:
                entry["frac_of_measured_hbm"] = round(bytes_per * n / med / 1e6 / HBM_PEAK_GBS, 3)
            out["elementwise_gbs"][f"{name}@2^{log2n}"] = entry
        del a, b, g, o, o2
    return out


# --------------------------------------------------------------------------- reference arm
def reference_sample(budget_s, steps=1, warmup=0):
    """One or more training steps of the config-4 architecture run by the
    reference's own compiled code (oracle/_ref/libref_true.so; the CPU port
    oracle/libref_fast.so if that library is absent), single-threaded, on a batch
    small enough to fit `budget_s`."""
    import oracle
    have_true = os.path.exists(oracle.REF_TRUE_PATH)
    oracle.fast.set_num_threads(1)
    params = make_params()

    def step(p, X, y):
        if have_true:
            return oracle.mlp_train_step_true(p, X, y, LR, input_grad=False)[0]
        return oracle.fast.mlp_train_step(p, X, y, LR, input_grad=True)[0]

    # calibrate on 2 rows, then size the sample to the budget
    X, y = make_batch(2, 99)
    t0 = time.perf_counter()
    step([(W.copy(), b.copy()) for W, b in params], X, y)
    per_row = (time.perf_counter() - t0) / 2
    n_steps = steps + warmup
    rows = int(max(1, min(64, budget_s / max(per_row * n_steps, 1e-9))))
    X, y = make_batch(rows, 100)
    work = [(W.copy(), b.copy()) for W, b in params]
    for _ in range(warmup):
        step(work, X, y)
    t0 = time.perf_counter()
    for _ in range(steps):
        step(work, X, y)
    dt = time.perf_counter() - t0
    return {"value": rows * steps / dt, "unit": "samples/s", "cores": 1,
            "kind": "reference" if have_true else "port",
            "sample": f"{steps} step(s) of the 784-1024-1024-10 MLP at batch {rows} "
                      f"(of {GLOBAL_BATCH}); the reference is single-threaded; its rate does not "
                      f"depend on the batch size (sequential loops)",
            "ms_per_step": dt / steps * 1e3, "rows": rows,
            "host_cores_available": os.cpu_count()}


def port_all_cores_sample(budget_s):
    """The same training step by the order-preserving CPU port (oracle/libref_fast.so:
    the reference's loops on flat arrays, OpenMP across independent outputs, same
    per-element operation order) on every host core — the second CPU line beside
    the reference's own single-threaded code."""
    import oracle
    cores = os.cpu_count() or 1
    oracle.fast.set_num_threads(cores)
    params = make_params()
    X, y = make_batch(64, 98)
    t0 = time.perf_counter()
    oracle.fast.mlp_train_step([(W.copy(), b.copy()) for W, b in params], X, y, LR)
    per_row = (time.perf_counter() - t0) / 64
    rows = int(max(64, min(4096, budget_s / max(per_row, 1e-9))))
    X, y = make_batch(rows, 100)
    work = [(W.copy(), b.copy()) for W, b in params]
    t0 = time.perf_counter()
    oracle.fast.mlp_train_step(work, X, y, LR, input_grad=True)
    dt = time.perf_counter() - t0
    return {"value": rows / dt, "unit": "samples/s", "cores": oracle.fast.num_threads(), "kind": "port",
            "sample": f"1 step of the 784-1024-1024-10 MLP at batch {rows} (of {GLOBAL_BATCH}), "
                      f"input gradient included as the reference computes it",
            "ms_per_step": dt * 1e3, "rows": rows, "host_cores_available": cores}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    budget = float(os.environ.get("MG_REF_BUDGET_S", "90"))
    base = reference_sample(budget, steps=args.steps, warmup=args.warmup)
    value = base["value"]
    out = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "MLP 784-1024-1024-10 fp64 train step (benchmark config 4)",
                   "global_batch": args.batch, "rows_per_step_sample": base["rows"], "lr": LR,
                   "parallelism": "cpu, 1 thread"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch (default: config 4)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweeps", action="store_true",
                    help="skip the batch-32 step and the DGEMM / elementwise sweeps (`c1`, `sweeps`)")
    ap.add_argument("--no-c5", action="store_true", help="skip the sharded inference leg (`c5`)")
    ap.add_argument("--sync-each-step", action="store_true",
                    help="diagnostic: host waits for the device after every step")
    ap.add_argument("--sweeps-only", action="store_true",
                    help="run only the DGEMM / elementwise sweeps on one GPU (for profiler captures)")
    ap.add_argument("--small-only", action="store_true",
                    help="run only the batch-32 step of config 1 on one GPU (for profiler captures)")
    ap.add_argument("--value-only", action="store_true",
                    help="run only the device-resident leg (for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.small_only:
        import micrograd_b200
        abi = micrograd_b200.load_abi()
        abi.mg_init(0)
        print(json.dumps({"c1": small_batch_leg(abi, micrograd_b200.load_api())}), flush=True)
    elif args.sweeps_only:
        import micrograd_b200
        from micrograd_b200 import cabi as K
        abi = micrograd_b200.load_abi()
        abi.mg_init(0)
        print(json.dumps({"sweeps": metric_sweeps(abi, K, small=True)}), flush=True)
    else:
        if args.warmup < 3:
            args.warmup = 3
        run_product(args)


if __name__ == "__main__":
    main()
