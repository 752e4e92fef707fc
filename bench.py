#!/usr/bin/env python
"""Benchmark of the Strassen-Winograd GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--size S] [--kernel NAME] [--no-cpu-baseline]

One "step" is one GEMM D = A * B.  The default workload is the single-GPU configuration the headline metric
is quoted on: f16 inputs, fp32 accumulate, f16 output, Strassen-Winograd level 1 (presum variant),
M = N = K = 8192, A and B i.i.d. uniform[-1, 1) from a seed (synthetic, generated on the device).
With N > 1 GPUs (one process per GPU under torchrun) every rank owns an 8192-row slab of A and of C and a
K/N-row shard of B; each step replicates B across the GPUs (inside the timed region) and runs the local GEMM: weak
scaling, per-GPU work fixed.

The line printed by rank 0 carries: metric / value (effective TFLOPS = 2MNK / t, all GPUs), e2e (same metric
through the C ABI with pinned HOST buffers, every step's copies inside the timed region and overlapped with the
kernels of its neighbours), roofline of the dominant kernel
(tensor-core bound; per-launch time from CUDA events recorded around every launch inside the timed loop),
cpu_baseline (the CPU oracle on a bounded row sample), clocks sampled during the timed region, gpu_launches.

`--impl reference` times the reference project's own CPU implementation of the path (its oracle kernels compiled
for the host, oracle/_ref) on a bounded row sample of the same workload with all host threads.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "effective TFLOPS (2MNK/t) f16/tf32 Strassen L1/L2 at 1/2/4/8 B200 vs cuBLAS"
UNIT = "TFLOPS"

# DRAM bytes (read + write) per launch of the dominant kernel from one ncu capture; see profiles/.
# key: (kernel, m, n, k).  None = not captured for that workload.
NCU_TRAFFIC_BYTES = {
    # profiles/sw_tile_program_pair_kernel_f16_level1_8192.md: launch 2 read 1.174 GB + write 0.313 GB
    ("blackwell_f16_sw_interleaved_presum_2sm", 8192, 8192, 8192): 1.488e9,
    # profiles/sw_tile_program_kernel_1cta_f16_level1_8192.md (earlier build): launch 2 read 1.102 GB + write 0.159 GB
    ("blackwell_f16_sw_interleaved_presum", 8192, 8192, 8192): 1.261e9,
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

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": (statistics.median(self.samples) if self.samples else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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


def reference_arm(args):
    """CPU reference: rank 0 alone times the reference's oracle kernels on a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np

    from oracle import binding as ob
    from subcuber_b200 import inputs

    ob.build(ref=True)
    kind = "reference" if ob.ref_oracle() is not None else "port"
    if kind == "reference":
        ob.ref_oracle().ref_sw_gemm_rows.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double,
                                                     C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_double, C.c_void_p,
                                                     C.c_int, C.c_int, C.c_int]
    size = args.size
    a_np, b_np = inputs.operands("f16", "uniform1", size, size, size, seed=1)
    cores = os.cpu_count() or 1
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
    sample = f"{times[0][1]} of {size} C rows per step (level-1 Strassen-Winograd, f16, {size}^3), {cores} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * tot_t / max(1, len(times)), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        # the same workload as the CUDA arm; every step covers a bounded sample of its rows (see cpu_baseline.sample)
        "config": {"workload": f"f16 Strassen-Winograd level 1, M=N=K={size} per GPU, uniform[-1,1) from seed 1",
                   "kernel": "reference oracle kernels compiled for the host", "m": size, "n": size, "k": size,
                   "level": 1},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=8192, help="M = N = K of the per-GPU problem")
    ap.add_argument("--kernel", default="blackwell_f16_sw_interleaved_presum_2sm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from subcuber_b200 import _lib, inputs, runner

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        from subcuber_b200 import multi_gpu

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # B is replicated by peer-to-peer copies on the copy engines (multi_gpu.PeerGather) unless SB200_GATHER=nccl
        # asks for the NCCL all-gather (multi_gpu.PipelinedGather)
        gather_cls = multi_gpu.PipelinedGather if os.environ.get("SB200_GATHER") == "nccl" else multi_gpu.PeerGather
        if os.environ.get("SB200_NCCL_CTAS"):  # tuning knob: CTAs given to NCCL (and SMs kept out of the GEMM grid)
            gather_cls.NCCL_CTAS = int(os.environ["SB200_NCCL_CTAS"])
        # the exchange of B overlaps the GEMM of the step before: NCCL runs on a bounded number of SMs that the GEMM
        # grid leaves free (the persistent GEMM kernels would otherwise hold every SM until they end)
        os.environ.setdefault("NCCL_MAX_CTAS", str(gather_cls.NCCL_CTAS))
        dist.init_process_group("nccl", device_id=device)
        sms = torch.cuda.get_device_properties(device).multi_processor_count

    lib = _lib.load()
    kernel = args.kernel
    dtn = "f16" if "_f16_" in kernel else "f32"
    tdt = torch.float16 if dtn == "f16" else torch.float32
    es = 2 if dtn == "f16" else 4
    m = n = k = args.size
    # operands: this rank's A slab (subsequence 2*rank so slabs differ) and its row shard of B
    a = inputs.fill_device(dtn, "uniform1", (m, k), seed=1, subsequence=2 * rank, device=device)
    gather = None
    if world > 1:
        b_full_ref = inputs.fill_device(dtn, "uniform1", (k, n), seed=1, subsequence=1, device=device)
        shard = multi_gpu.row_shard(k, world, rank)
        b_shard = b_full_ref[shard[0]:shard[1]].contiguous()
        del b_full_ref
        if gather_cls is multi_gpu.PeerGather:
            # symmetric memory needs peer mappings between all GPUs: where that cannot be set up, every rank falls back
            # to the NCCL all-gather (the ranks agree first, so that none is left alone in a collective)
            try:
                gather = multi_gpu.PeerGather(b_shard, k, world, rank)
                ok = 1
            except Exception as exc:  # noqa: BLE001 - any setup failure means "use the other exchange"
                print(f"[bench] rank {rank}: peer exchange unavailable ({exc}); using the NCCL all-gather", file=sys.stderr)
                ok = 0
            agreed = torch.tensor([ok], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:
                gather_cls = multi_gpu.PipelinedGather
                gather = None
                # a new communicator with the all-gather's CTA bound
                dist.destroy_process_group()
                os.environ["NCCL_MAX_CTAS"] = str(gather_cls.NCCL_CTAS)
                dist.init_process_group("nccl", device_id=device)
        if gather is None:
            gather = multi_gpu.PipelinedGather(b_shard, k, world)
        os.environ["SB200_SM_LIMIT"] = str(sms - gather_cls.reserved_sms())
        b = gather.bufs[0]
    else:
        b = inputs.fill_device(dtn, "uniform1", (k, n), seed=1, subsequence=1, device=device)
    d = torch.empty((m, n), dtype=tdt, device=device)
    ws = runner.Workspace(kernel, m, n, k, device)
    stream = torch.cuda.current_stream(device)
    launches = lib.sb200_gemm_launches(kernel.encode())
    total_steps = args.warmup + args.steps
    evl = lib.sb200_events_create((launches + 1) * args.steps)

    def step(i):
        bi = gather.next() if gather else b  # replicated B of this step; the next step's all-gather is now in flight
        if i >= args.warmup:
            rc = lib.sb200_gemm_events(kernel.encode(), a.data_ptr(), bi.data_ptr(), d.data_ptr(), m, n, k, ws.ptr,
                                       ws.nbytes, stream.cuda_stream, evl, (launches + 1) * (i - args.warmup))
        else:
            rc = lib.sb200_gemm(kernel.encode(), a.data_ptr(), bi.data_ptr(), d.data_ptr(), m, n, k, ws.ptr, ws.nbytes,
                                stream.cuda_stream)
        if rc != 0:
            raise runner.KernelError(kernel, rc)
        if gather:
            gather.done(bi)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
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
    status = lib.sb200_gemm_status(ws.ptr, stream.cuda_stream)
    if status != 0:
        raise runner.KernelError(kernel, status)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    flops_step = 2.0 * m * n * k * world
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
    dom = max(range(launches), key=lambda i: per_launch[i])
    # algorithmic flops of a GEMM are 2MNK at every level; each of its 7 (49) products carries 1/7 (1/49) of them
    level = {r.name: r.strassen_level for r in runner.kernels()}[kernel]
    products = {0: [1], 1: {1: [7], 2: [2, 5]}.get(launches, [7]), 2: [2, 5] * 7}[level]
    share = products[dom] / sum(products)
    peaks = _peaks()
    timed_s = elapsed_ms * 1e-3
    peak = peaks["burst"] if timed_s < 2.0 else peaks["sustained"]
    achieved = 2.0 * m * n * k * share / (per_launch[dom] * 1e-3) / 1e12
    traffic = NCU_TRAFFIC_BYTES.get((kernel, m, n, k))
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": f"launch {dom + 1} of {launches} ({products[dom]} of {sum(products)} products)",
                "launch_ms": per_launch,
                "peak_source": f"{peaks['source']} cuBLAS bf16 {'burst' if timed_s < 2.0 else 'sustained'}"}

    # end to end: operands in pinned host memory, every step copies its A and B to the device and its D back, inside the
    # timed region; the copies of neighbouring steps overlap the kernels (runner.HostPipeline: three streams, two
    # sets of device buffers), so a step costs the slowest of its three parts
    e2e_steps = max(4, min(10, args.steps))
    a_host = a.cpu().pin_memory()
    b_host = b.cpu().pin_memory()
    d_host = torch.empty((m, n), dtype=tdt).pin_memory()
    pipe = runner.HostPipeline(kernel, m, n, k, tdt, device)
    for _ in range(3):
        pipe.submit(a_host, b_host, d_host)
    pipe.finish()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(pipe.s_mm)   # every stream is idle here: the first copy starts after this point
    for _ in range(e2e_steps):
        pipe.submit(a_host, b_host, d_host)
    pipe.join(pipe.s_mm)   # the last result has reached the host
    e1.record(pipe.s_mm)
    pipe.finish()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": (m * k + k * n) * es, "d2h_bytes_per_step": m * n * es, "steps": e2e_steps}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and dtn == "f16":
        from oracle import binding as ob

        ob.build(ref=False)
        nrows = _cpu_calibrate("port", ob, a_host.numpy(), b_host.numpy(), target_s=12.0)
        dt, rows = _cpu_run("port", ob, a_host.numpy(), b_host.numpy(), nrows)
        tf = 2.0 * rows * n * k / dt / 1e12
        cpu_baseline = {"value": tf, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                        "sample": f"{rows} of {m} C rows of the same workload in {dt:.1f} s (CPU oracle, OpenMP)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtn, "data": "synthetic",
            "config": {"workload": f"{dtn} Strassen-Winograd level {level}, M=N=K={args.size} per GPU, uniform[-1,1) from "
                       "seed 1" if level else f"{dtn} GEMM level 0, M=N=K={args.size}",
                       "kernel": kernel, "m": m * world, "n": n, "k": k, "level": level,
                       "l2": f"inputs larger than L2: {(m * k + k * n + m * n) * es / 2**20:.0f} MiB touched per step",
                       "parallelism": f"row slabs x{world}" + (f", B replicated every step ({'peer-to-peer copies on the copy engines' if gather_cls is multi_gpu.PeerGather else 'NCCL all-gather'}), overlapped with the GEMM of the step before" if world > 1 else "")},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches * args.steps, "host_enqueue_ms_per_step": host_ms, "roofline": roofline,
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
