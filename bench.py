#!/usr/bin/env python
"""Benchmark of the Strassen-Winograd GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--size S] [--kernel NAME] [--no-cpu-baseline] [--no-sustained] [--no-cublas]

One "step" is one GEMM D = A * B.  The default workload is the configuration the headline metric is quoted on:
f16 inputs, fp32 accumulate, f16 output, Strassen-Winograd level 1 (presum variant), M = N = K = 16384, A and B
i.i.d. uniform[-1, 1) from a seed (synthetic, generated on the device).  With N > 1 GPUs (one process per GPU under
torchrun) the SAME problem is divided over the GPUs (strong scaling): the GPUs form a pr x pc grid, GPU (i, j)
computes the block C[i, j] with a local Strassen-Winograd GEMM, and every step first replicates the row slab of A
inside each grid row and the column slab of B inside each grid column from the shards the GPUs own (inside the timed
region, overlapped with the GEMM of the step before).

The line printed by rank 0 carries: metric / value (effective TFLOPS = 2MNK / t, whole job), frac_of_dense_peak
(value / nominal dense f16 peak per GPU), cublas (cuBLAS on the same buffers in the same process, timed in
alternating rounds with this library so that both see the same thermal state), sustained (both again in loops of at
least two seconds), e2e (same metric through the C ABI with pinned HOST buffers, every step's copies inside the
timed region), roofline of the dominant kernel (tensor-core bound; per-launch time from CUDA events recorded around
every launch inside the timed loop), cpu_baseline (the CPU oracle on a bounded row sample), clocks sampled during
the timed region, gpu_launches.

`--impl reference` times the reference project's own CPU implementation of the path (its oracle kernels compiled
for the host, oracle/_ref) on a bounded row sample of the same workload with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "effective TFLOPS (2MNK/t) f16/tf32 Strassen L1/L2 at 1/2/4/8 B200 vs cuBLAS"
UNIT = "TFLOPS"
DEFAULT_SIZE = 16384
DEFAULT_KERNEL = "blackwell_f16_sw_interleaved_presum_2sm"
# nominal dense tensor-core peak per GPU for the arithmetic type of the kernels (TFLOP/s)
DENSE_PEAK = {"f16": 2250.0, "bf16": 2250.0, "f32": 1125.0, "f64": 40.0}
CUBLAS_ROW = {"f16": "cublas_f16", "bf16": "cublas_bf16", "f32": "cublas_tf32", "f64": "cublas_f64"}
ELEM_BYTES = {"f16": 2, "bf16": 2, "f32": 4, "f64": 8}

# DRAM bytes (read + write) per launch of the dominant kernel from one Nsight Compute capture of that launch
# (dram__bytes_read.sum + dram__bytes_write.sum).  key: (kernel, m, n, k).  Absent = not captured for that workload.
NCU_TRAFFIC_BYTES = {
    ("blackwell_f16_sw_interleaved_presum_2sm", 16384, 16384, 16384): 9.71e9,   # launch 2: read 8.52 GB + write 1.19 GB
    ("blackwell_f16_sw_interleaved_presum_2sm", 8192, 8192, 8192): 1.307e9,     # launch 2: read 1.033 GB + write 0.274 GB
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p["bf16_tflops_sustained"]), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: clocks are reported as unknown
            self._h = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
                r = self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": (statistics.median(self.samples) if self.samples else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def _omp_threads(n=None):
    """Sets (when `n` is given) and returns the OpenMP thread count of this process.  torchrun exports
    OMP_NUM_THREADS=1 to its workers; the CPU arms use every host thread, so they set the count themselves."""
    try:
        gomp = C.CDLL("libgomp.so.1")
        if n is not None:
            gomp.omp_set_num_threads(int(n))
        return int(gomp.omp_get_max_threads())
    except OSError:
        return 1


def _cpu_run(kind, oracle, a_np, b_np, nrows):
    """One CPU pass over a bounded sample: `nrows` quadrant rows (port: C rows r and r + M/2 of each) or the first
    `nrows` C rows (reference build: every output element is an independent thread of its grid).
    Returns (seconds, C rows produced)."""
    import numpy as np

    m, k = a_np.shape
    n = b_np.shape[1]
    t0 = time.perf_counter()
    if kind == "reference":
        lib = oracle.ref_oracle()
        out = np.zeros((m, n), dtype=a_np.dtype)
        rc = lib.ref_sw_gemm_rows(0, 1, m, n, k, C.c_double(1.0), a_np.ctypes.data_as(C.c_void_p), k,
                                  b_np.ctypes.data_as(C.c_void_p), n, C.c_double(0.0),
                                  out.ctypes.data_as(C.c_void_p), n, 0, nrows)
        assert rc == 0
        done = nrows
    else:
        rows = np.linspace(0, m // 2 - 1, nrows).astype(np.int32)
        oracle.sw_gemm("f16", 1, a_np, b_np, rows=rows)
        done = 2 * nrows
    return time.perf_counter() - t0, done


def _cpu_calibrate(kind, oracle, a_np, b_np, target_s):
    """Number of sample rows that makes one pass take about `target_s` seconds."""
    probe = 2 if kind == "reference" else 16
    dt, _ = _cpu_run(kind, oracle, a_np, b_np, probe)
    per_row = max(dt / probe, 1e-6)   # includes the port's fixed cost (B presums), so the sample errs on the short side
    return max(1, min(a_np.shape[0] // 2, int(target_s / per_row)))


def _workload_text(dtn, level, m, n, k):
    if level == 0:
        return f"{dtn} GEMM level 0, M={m} N={n} K={k}, uniform[-1,1) from seed 1"
    return f"{dtn} Strassen-Winograd level {level}, M={m} N={n} K={k}, uniform[-1,1) from seed 1"


def reference_arm(args):
    """CPU reference: rank 0 alone times the reference's oracle kernels on a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)  # before the OpenMP runtime starts (torchrun sets it to 1)
    import numpy as np  # noqa: F401

    from oracle import binding as ob
    from subcuber_b200 import inputs

    ob.build(ref=True)
    threads = _omp_threads(cores)
    kind = "reference" if ob.ref_oracle() is not None else "port"
    if kind == "reference":
        ob.ref_oracle().ref_sw_gemm_rows.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double,
                                                     C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p,
                                                     C.c_int, C.c_int, C.c_int]
    size = args.size
    a_np, b_np = inputs.operands("f16", "uniform1", size, size, size, seed=1)
    # calibrate the sample so one step takes about 1.5 s, then time exactly `steps` steps
    nrows = _cpu_calibrate(kind, ob, a_np, b_np, target_s=1.5)
    times = []
    for i in range(args.warmup + args.steps):
        dt_i, rows_i = _cpu_run(kind, ob, a_np, b_np, nrows)
        if i >= args.warmup:
            times.append((dt_i, rows_i))
    tot_t = sum(t for t, _ in times)
    tot_rows = sum(r for _, r in times)
    value = 2.0 * tot_rows * size * size / tot_t / 1e12
    sample = (f"{times[0][1]} of {size} C rows per step (level-1 Strassen-Winograd, f16, {size}^3), "
              f"{threads} OpenMP threads on {cores} host cores")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * tot_t / max(1, len(times)), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        # the same workload as the CUDA arm; every step covers a bounded sample of its rows (see cpu_baseline.sample)
        "config": {"workload": _workload_text("f16", 1, size, size, size),
                   "kernel": "reference oracle kernels compiled for the host" if kind == "reference"
                   else "CPU restatement of the reference oracle", "m": size, "n": size, "k": size, "level": 1,
                   "l2": "not applicable (CPU)", "parallelism": f"{threads} host threads"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=DEFAULT_SIZE, help="M = N = K of the whole problem")
    ap.add_argument("--kernel", default=DEFAULT_KERNEL)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second loops")
    ap.add_argument("--no-cublas", action="store_true", help="skip the cuBLAS comparison")
    ap.add_argument("--copy-streams", type=int, default=0, help="N > 1: streams the exchange deals its copies over (0 = its default)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        return reference_arm(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # one hardware work queue per stream of the exchange (the driver reads this when it is initialised)
        os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

    import torch
    import torch.distributed as dist

    from subcuber_b200 import _lib, inputs, runner

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)

    lib = _lib.load()
    kernel = args.kernel
    rows_by_name = {r.name: r for r in runner.kernels()}
    if kernel not in rows_by_name or not kernel.startswith("blackwell_"):
        raise SystemExit(f"unknown kernel {kernel!r}: choose a blackwell_* row of the registry")
    info = rows_by_name[kernel]
    dtn = info.dtype                       # the registry row says which element type the kernel reads and writes
    if dtn not in ELEM_BYTES:
        raise SystemExit(f"bench.py cannot fill operands of type {dtn!r}")
    tdt = runner.TORCH_DTYPE[dtn]
    es = ELEM_BYTES[dtn]
    M = N = K = args.size
    resolved = kernel
    if kernel.endswith("_sw_auto"):
        resolved = lib.sb200_auto_kernel(dtn.encode(), M, N, K).decode()
    level = rows_by_name[resolved].strassen_level

    exchange = None
    opts = None
    grid_text = "1 GPU"
    if world > 1:
        from subcuber_b200 import multi_gpu

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_MAX_CTAS", "2")   # NCCL only carries set-up traffic and the final reductions here
        dist.init_process_group("nccl", device_id=device)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        gp = multi_gpu.grid_plan(M, N, K, world, es, level=max(level, 1))
        if gp.kind == "replica":
            raise SystemExit(f"{M}x{N}x{K} does not divide over {world} GPUs")
        m, n, k = gp.local_m, gp.local_n, K
        # SMs left out of the GEMM grid for the few one-CTA flag kernels of the exchange (the persistent GEMM kernels
        # would otherwise hold every SM until they end)
        # symmetric memory needs peer mappings between all GPUs: where they cannot be set up every rank falls back to
        # all-gathers in the grid's groups (the ranks agree first, so that none is left alone in a collective)
        try:
            exchange = multi_gpu.GridExchange(gp, rank, dtn, device, seed=1, max_copy_streams=args.copy_streams)
            ok = 1
        except Exception as exc:  # noqa: BLE001 - any set-up failure means "use the other exchange"
            print(f"[bench] rank {rank}: peer exchange unavailable ({exc}); using collectives", file=sys.stderr)
            ok = 0
        agreed = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            exchange = multi_gpu.CollectiveGridExchange(gp, rank, dtn, device, seed=1)
        reserved = type(exchange).reserved_sms()
        opts = runner.options(sm_limit=sms - reserved) if reserved else None
        grid_text = gp.describe() + "; exchange: " + exchange.describe()
    else:
        m, n, k = M, N, K

    if exchange is None:
        a = inputs.fill_device(dtn, "uniform1", (m, k), seed=1, subsequence=0, device=device)
        b = inputs.fill_device(dtn, "uniform1", (k, n), seed=1, subsequence=1, device=device)
    d = torch.empty((m, n), dtype=tdt, device=device)
    ws = runner.Workspace(kernel, m, n, k, device, opts)
    stream = torch.cuda.current_stream(device)
    launches = lib.sb200_gemm_launches(resolved.encode())
    total_steps = args.warmup + args.steps
    evl = lib.sb200_events_create((launches + 1) * args.steps)
    opts_ref = C.byref(opts) if opts is not None else None

    def gemm(ai, bi, event_index=None):
        if event_index is not None:
            rc = lib.sb200_gemm_events(kernel.encode(), ai.data_ptr(), bi.data_ptr(), d.data_ptr(), m, n, k, ws.ptr,
                                       ws.nbytes, stream.cuda_stream, evl, event_index, opts_ref)
        else:
            rc = lib.sb200_gemm_opt(kernel.encode(), ai.data_ptr(), bi.data_ptr(), d.data_ptr(), m, n, k, ws.ptr,
                                    ws.nbytes, stream.cuda_stream, opts_ref)
        if rc != 0:
            raise runner.KernelError(kernel, rc)

    def step(i):
        if exchange is not None:
            ai, bi = exchange.next()   # this step's replicated slabs; the exchange of the step after is now in flight
        else:
            ai, bi = a, b
        gemm(ai, bi, (launches + 1) * (i - args.warmup) if i >= args.warmup else None)
        if exchange is not None:
            exchange.done()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def check_status():
        status = lib.sb200_gemm_status(ws.ptr, stream.cuda_stream)
        if status != 0:
            raise runner.KernelError(kernel, status)

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank).start()
    t_start = torch.cuda.Event(enable_timing=True)
    t_stop = torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    host_t0 = time.perf_counter()
    for i in range(args.warmup, total_steps):
        step(i)
    host_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps  # host time to enqueue one step
    t_stop.record(stream)
    barrier()
    clocks = sampler.stop()
    elapsed_ms = t_start.elapsed_time(t_stop)
    check_status()
    exchange_wait_ms = None
    if exchange is not None:
        exchange.check_status()
        exchange_wait_ms = exchange.wait_ms(args.steps)
    own_elapsed_ms = elapsed_ms
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    flops_step = 2.0 * M * N * K            # the whole problem, however many GPUs share it
    value = flops_step * args.steps / (elapsed_ms * 1e-3) / 1e12

    # per-launch durations inside the timed region
    per_launch = [0.0] * launches
    ms = C.c_float(0)
    for s in range(args.steps):
        for l in range(launches):
            lib.sb200_events_elapsed_ms(evl, (launches + 1) * s + l, (launches + 1) * s + l + 1, C.byref(ms))
            per_launch[l] += ms.value
    per_launch = [x / args.steps for x in per_launch]
    lib.sb200_events_destroy(evl)
    # several GPUs: what every rank measured on its own stream (ms per step: whole step, its launches, its waits)
    per_rank = None
    if world > 1:
        mine = torch.tensor([own_elapsed_ms / args.steps, sum(per_launch), exchange_wait_ms or 0.0], dtype=torch.float64,
                            device=device)
        everyone = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        per_rank = [{"ms_per_step": round(float(t_[0]), 4), "launches_ms": round(float(t_[1]), 4),
                     "wait_ms": round(float(t_[2]), 4)} for t_ in everyone]
    dom = max(range(launches), key=lambda i: per_launch[i])
    # algorithmic flops of a GEMM are 2MNK at every level; each of its 7 (49) products carries 1/7 (1/49) of them
    if dtn == "f64":
        products = [0] * launches   # the fp64 path interleaves presum and product launches: whole GEMM as one unit
        products[dom] = 1
        share = per_launch[dom] / max(sum(per_launch), 1e-9)
    else:
        products = {0: [1], 1: {1: [7], 2: [2, 5]}.get(launches, [7]), 2: [2, 5] * 7}[level]
        share = products[dom] / sum(products)
    peaks = _peaks()
    timed_s = elapsed_ms * 1e-3
    peak = peaks["burst"] if timed_s < 2.0 else peaks["sustained"]
    achieved = 2.0 * m * n * k * share / (per_launch[dom] * 1e-3) / 1e12
    traffic = NCU_TRAFFIC_BYTES.get((resolved, m, n, k))
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": f"launch {dom + 1} of {launches} ({products[dom]} of {sum(products)} products)",
                "launch_ms": per_launch,
                "peak_source": f"{peaks['source']} cuBLAS bf16 {'burst' if timed_s < 2.0 else 'sustained'}"}

    # correctness evidence for the multi-GPU runs: every rank checks sampled rows of its block of the last step
    # against the fp64 product of the operands it multiplied, and the block's checksum
    parity = None
    if exchange is not None:
        ok = exchange.verify_block(d, ai_bi=exchange.last())
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.SUM)
        parity = {"ranks_ok": int(flag.item()), "ranks": world,
                  "check": "sampled rows of every rank's block vs fp64 (rel. Frobenius < 2e-3) + block checksum"}

    # cuBLAS on the same buffers in the same process.  The GPU runs against its power cap, and the cap's controller has
    # a memory of tens of milliseconds: whichever arm runs second inherits the clocks the first one left.  So every
    # timed burst of either arm starts from the same state: a pause that lets the clocks recover, two untimed calls,
    # then `steps` timed steps; three rounds, median.  The seconds-long loops below give the steady state.
    cublas = None
    sustained = None
    blas_row = CUBLAS_ROW.get(dtn)
    if world == 1 and blas_row and not args.no_cublas:
        burst_steps = max(3, args.steps)
        ours_ms, blas_ms = [], []
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            torch.cuda.synchronize(device)
            time.sleep(0.5)
            for _ in range(2):
                gemm(a, b)
            e0.record(stream)
            for _ in range(burst_steps):
                gemm(a, b)
            e1.record(stream)
            torch.cuda.synchronize(device)
            ours_ms.append(e0.elapsed_time(e1) / burst_steps)
            time.sleep(0.5)
            _, bms = runner.run_kernel(blas_row, a, b, d, warmup=2, iterations=burst_steps)
            blas_ms.append(bms)
        check_status()
        o, c_ = statistics.median(ours_ms), statistics.median(blas_ms)
        cublas = {"kernel": blas_row, "value": flops_step / (c_ * 1e-3) / 1e12, "ours_value": flops_step / (o * 1e-3) / 1e12,
                  "ratio": c_ / o, "unit": UNIT, "rounds": 3, "steps_per_round": burst_steps,
                  "how": "each arm: 0.5 s pause, 2 untimed calls, then the timed steps, on the same device buffers; "
                         "median of the rounds"}
        if not args.no_sustained:
            n_long = max(args.steps, int(math.ceil(2200.0 / max(o, 1e-3))))
            smp = ClockSampler(local_rank).start()
            e0.record(stream)
            for _ in range(n_long):
                gemm(a, b)
            e1.record(stream)
            torch.cuda.synchronize(device)
            s_clocks = smp.stop()
            s_ours = e0.elapsed_time(e1) / n_long
            check_status()
            n_blas = max(args.steps, int(math.ceil(2200.0 / max(c_, 1e-3))))
            smp = ClockSampler(local_rank).start()
            _, s_blas = runner.run_kernel(blas_row, a, b, d, warmup=1, iterations=n_blas)
            b_clocks = smp.stop()
            sv = flops_step / (s_ours * 1e-3) / 1e12
            bv = flops_step / (s_blas * 1e-3) / 1e12
            sustained = {"value": sv, "cublas": bv, "ratio": sv / bv, "unit": UNIT,
                         "frac": sv / peaks["sustained"], "peak": peaks["sustained"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 sustained", "seconds": s_ours * n_long * 1e-3,
                         "steps": n_long, "clocks": s_clocks, "cublas_clocks": b_clocks}

    # end to end: operands in pinned host memory, every step copies its A and B to the device and its D back, inside the
    # timed region; the copies of neighbouring steps overlap the kernels (runner.HostPipeline: three streams, two
    # sets of device buffers), so a step costs the slowest of its three parts
    if exchange is not None:
        a, b = exchange.last()
    e2e_steps = max(4, min(10, args.steps))
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    if exchange is not None and hasattr(exchange, "feed"):
        # several GPUs: every GPU uploads only the shards it owns (1/P of A and of B) from its pinned host memory; the
        # exchange spreads them over NVLink under the kernels of the steps before; every GPU downloads its block of D
        a_own, b_own = exchange.shard_views(0)
        a_host = a_own.cpu().pin_memory()
        b_host = b_own.cpu().pin_memory()
        d_host = torch.empty((m, n), dtype=tdt).pin_memory()
        d_bufs = [d, torch.empty_like(d)]
        s_out = torch.cuda.Stream(device)
        done_mm = [torch.cuda.Event() for _ in range(2)]
        done_out = [torch.cuda.Event() for _ in range(2)]
        h2d_bytes = (a_host.numel() + b_host.numel()) * es
        exchange.start_feeding()

        def e2e_step(i, after=None):
            exchange.feed(a_host, b_host, after)
            ai, bi = exchange.next()
            slot = i % 2
            stream.wait_event(done_out[slot])          # this buffer's previous result has left
            rc = lib.sb200_gemm_opt(kernel.encode(), ai.data_ptr(), bi.data_ptr(), d_bufs[slot].data_ptr(), m, n, k,
                                    ws.ptr, ws.nbytes, stream.cuda_stream, opts_ref)
            if rc != 0:
                raise runner.KernelError(kernel, rc)
            exchange.done()
            done_mm[slot].record(stream)
            s_out.wait_event(done_mm[slot])
            with torch.cuda.stream(s_out):
                d_host.copy_(d_bufs[slot], non_blocking=True)
                done_out[slot].record(s_out)

        for ev in done_out:
            ev.record(stream)
        for i in range(3 + exchange.NBUF):              # the first steps still run on shards issued before
            e2e_step(i)
        barrier()
        e0.record(stream)                               # every stream is idle here: the first upload waits for this
        for i in range(e2e_steps):
            e2e_step(i, after=e0 if i == 0 else None)
        stream.wait_stream(s_out)                       # the last result has reached the host
        e1.record(stream)
        barrier()
        check_status()
        exchange.check_status()
        d2h_bytes = m * n * es
        note = ("bytes per GPU and step: every GPU uploads the shards of A and B it owns from its pinned host memory "
                "(the exchange spreads them over NVLink) and downloads its block of D")
    else:
        a_host = a.cpu().pin_memory()
        b_host = b.cpu().pin_memory()
        d_host = torch.empty((m, n), dtype=tdt).pin_memory()
        pipe = runner.HostPipeline(kernel, m, n, k, tdt, device, opts)
        for _ in range(3):
            pipe.submit(a_host, b_host, d_host)
        pipe.finish()
        barrier()
        e0.record(pipe.s_mm)   # every stream is idle here: the first copy starts after this point
        for _ in range(e2e_steps):
            pipe.submit(a_host, b_host, d_host)
        pipe.join(pipe.s_mm)   # the last result has reached the host
        e1.record(pipe.s_mm)
        pipe.finish()
        barrier()
        h2d_bytes, d2h_bytes = (m * k + k * n) * es, m * n * es
        note = "bytes per GPU and step; every GPU copies the operands it multiplies from its own pinned host memory"
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "note": note}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and dtn == "f16" and level >= 1:
        from oracle import binding as ob

        ob.build(ref=False)
        threads = _omp_threads(os.cpu_count() or 1)
        nrows = _cpu_calibrate("port", ob, a_host.numpy(), b_host.numpy(), target_s=12.0)
        dt, rows = _cpu_run("port", ob, a_host.numpy(), b_host.numpy(), nrows)
        tf = 2.0 * rows * n * k / dt / 1e12
        cpu_baseline = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"{rows} of {m} C rows of the same workload in {dt:.1f} s (CPU oracle, level 1, OpenMP)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": dtn, "data": "synthetic",
            "config": {"workload": _workload_text(dtn, level, M, N, K),
                       "kernel": kernel if resolved == kernel else f"{kernel} -> {resolved}", "m": M, "n": N, "k": K,
                       "level": level,
                       "l2": f"inputs larger than L2: {(m * k + k * n + m * n) * es / 2**20:.0f} MiB touched per GPU and step",
                       "parallelism": grid_text},
            "frac_of_dense_peak": value / (DENSE_PEAK[dtn] * world),
            "dense_peak": {"value": DENSE_PEAK[dtn] * world, "unit": "TFLOP/s", "source": "nominal, dense, per GPU x GPUs"},
            "cublas": cublas, "sustained": sustained, "parity": parity,
            "exchange_wait_ms_per_step": exchange_wait_ms, "per_rank": per_rank,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches * args.steps, "host_enqueue_ms_per_step": host_ms,
            "roofline": roofline, "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        exchange.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
