"""Multi-GPU plan for one box: C (and A) split into slabs, B replicated by an all-gather.

The reference project is single-GPU (device 0 only, src/cuda/kernel_runner_support.cuh:312 there); this module is
the one exchange step the path needs when it runs on 2, 4 or 8 GPUs of a box.  One process per GPU.  GPU r owns the
row slab A[r] (M/P rows) and produces the same rows of C with an independent local Strassen-Winograd GEMM on an
(M/P) x N x K problem.  Every GPU needs all of B: B starts row-sharded (K/P contiguous rows per GPU, contiguous in
row-major) and is replicated into each GPU's own memory by an NCCL all-gather over NVLink; the kernels then read
local memory only (plain, non-multicast TMA).  When N is much larger than M the symmetric column plan (B column
slabs local, A replicated) moves fewer bytes; `plan` picks between them.

Everything here is host logic and runs on CPU with the gloo backend too (tests/test_multi_gpu_cpu.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import os

import torch
import torch.distributed as dist


def row_shard(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the contiguous block of `rows` owned by `rank`; earlier ranks take the remainder."""
    if world <= 0 or not (0 <= rank < world) or rows < 0:
        raise ValueError("bad shard request")
    base, rem = divmod(rows, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


@dataclass(frozen=True)
class SlabPlan:
    kind: str            # "row": A/C row slabs, B replicated; "col": B/C column slabs, A replicated; "replica"
    world: int
    m: int
    n: int
    k: int
    local_m: int         # shape of the local GEMM
    local_n: int
    exchange_bytes: int  # bytes each GPU receives per GEMM

    def describe(self) -> str:
        return (f"{self.kind} slabs x{self.world}: local {self.local_m}x{self.local_n}x{self.k}, "
                f"{self.exchange_bytes / 2**20:.0f} MiB received per GPU")


def plan(m: int, n: int, k: int, world: int, esize: int, level: int = 1, tile_m: int = 128, tile_n: int = 256) -> SlabPlan:
    """Choose the slab direction: the one whose replicated operand is smaller, provided the local problem still
    splits into quadrants whose rows start on 16 bytes and is not smaller than one tile program per GPU."""
    if world == 1:
        return SlabPlan("row", 1, m, n, k, m, n, 0)
    div = 1 << level
    vec = 16 // esize
    candidates: List[SlabPlan] = []
    if m % world == 0 and (m // world) % div == 0 and (m // world) // div >= tile_m:
        candidates.append(SlabPlan("row", world, m, n, k, m // world, n, (world - 1) * k * n * esize // world))
    if n % world == 0 and (n // world) % (div * vec) == 0 and (n // world) // div >= tile_n:
        candidates.append(SlabPlan("col", world, m, n, k, m, n // world, (world - 1) * m * k * esize // world))
    if not candidates:
        # slabs would be too thin to fill a GPU: run independent replicas instead (no exchange)
        return SlabPlan("replica", world, m, n, k, m, n, 0)
    return min(candidates, key=lambda p: p.exchange_bytes)


def all_gather_rows(full: torch.Tensor, shard: torch.Tensor, world: int, group=None) -> None:
    """Replicate a row-sharded matrix: `full` (rows x cols, this rank's own memory) receives every rank's `shard`.

    Equal shards go through one all_gather_into_tensor (a single NCCL kernel writing straight into `full`); ragged
    shards fall back to a list all-gather.
    """
    rows = full.shape[0]
    if rows % world == 0 and shard.shape[0] == rows // world:
        try:
            dist.all_gather_into_tensor(full, shard, group=group)
            return
        except (RuntimeError, NotImplementedError):
            pass  # backend without the fused form (older gloo): use the list form below
    parts = []
    for r in range(world):
        b, e = row_shard(rows, world, r)
        parts.append(full[b:e])
    if all(p.shape == parts[0].shape for p in parts):
        dist.all_gather(parts, shard, group=group)
    else:
        # ragged: pad to the largest shard
        big = max(p.shape[0] for p in parts)
        padded = torch.zeros((big,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
        padded[: shard.shape[0]] = shard
        bufs = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(bufs, padded, group=group)
        for p, buf in zip(parts, bufs):
            p.copy_(buf[: p.shape[0]])


class PipelinedGather:
    """Double-buffered replication of B that overlaps the exchange with compute.

    Step i multiplies with buffer i % 2 while the all-gather that fills buffer (i + 1) % 2 runs on its own stream;
    events order the two streams (a buffer is refilled only after the GEMM that read it, and read only after its
    gather).  NCCL's kernels need SMs of their own while the persistent GEMM kernels hold theirs, so the caller
    leaves `reserved_sms()` SMs out of the GEMM grid.  Without CUDA (gloo tests) the gathers run synchronously.
    """

    NCCL_CTAS = 8  # upper bound given to NCCL (NCCL_MAX_CTAS) before the process group is created

    def __init__(self, shard: torch.Tensor, rows: int, world: int, group=None, bufs=None):
        self.shard, self.world, self.group = shard, world, group
        self.bufs = bufs if bufs is not None else [
            torch.empty((rows, shard.shape[1]), dtype=shard.dtype, device=shard.device) for _ in range(2)]
        self.cuda = shard.is_cuda
        if self.cuda:
            self.comm = torch.cuda.Stream(device=shard.device)
            self.filled = [torch.cuda.Event() for _ in range(2)]
            self.consumed = [torch.cuda.Event() for _ in range(2)]
            for ev in self.consumed:
                ev.record(torch.cuda.current_stream(shard.device))
        self.issued = 0  # gathers started so far
        self.taken = 0   # buffers handed to compute so far

    @classmethod
    def reserved_sms(cls) -> int:
        """SMs to keep out of the GEMM grid: one TPC (two SMs) per NCCL CTA, since a CTA pair needs a whole TPC."""
        return 2 * cls.NCCL_CTAS

    def _start(self) -> None:
        i = self.issued % 2
        if self.cuda:
            self.comm.wait_event(self.consumed[i])
            with torch.cuda.stream(self.comm):
                all_gather_rows(self.bufs[i], self.shard, self.world, self.group)
                self.filled[i].record(self.comm)
        else:
            all_gather_rows(self.bufs[i], self.shard, self.world, self.group)
        self.issued += 1

    def update_shard(self, values: torch.Tensor) -> None:
        """New contents for this rank's shard, seen by every exchange started after this call (exchanges already
        in flight still read the old contents: the copy is ordered behind them on the exchange stream)."""
        if self.cuda:
            self.comm.wait_stream(torch.cuda.current_stream(self.shard.device))
            with torch.cuda.stream(self.comm):
                self.shard.copy_(values, non_blocking=True)
        else:
            self.shard.copy_(values)

    def next(self) -> torch.Tensor:
        """The replicated B for this step (valid on the current stream); the gather for the next step is started."""
        while self.issued < self.taken + 2:
            self._start()
        i = self.taken % 2
        if self.cuda:
            torch.cuda.current_stream(self.shard.device).wait_event(self.filled[i])
        self.taken += 1
        return self.bufs[i]

    def done(self, buf: torch.Tensor) -> None:
        """Call after the GEMM that reads `buf` has been enqueued: its buffer may be refilled once that GEMM is over."""
        if self.cuda:
            i = 0 if buf is self.bufs[0] else 1
            self.consumed[i].record(torch.cuda.current_stream(self.shard.device))


class PeerGather(PipelinedGather):
    """The same double-buffered replication with the bytes moved by the copy engines instead of NCCL's kernels:
    the buffers live in symmetric memory (torch.distributed._symmetric_memory: every rank's buffer is mapped into
    every process), and every rank pushes its shard into all ranks' buffers with plain device-to-device copies whose
    destination is peer memory, over NVLink.  The exchange takes no SMs from the GEMM and runs at DMA speed
    (measured: 64 MiB to a peer in 0.11 ms).  Two one-word NCCL all-reduces per step order the ranks (everyone's
    buffer is free before the pushes start; every push has landed before the buffer is read); they are the only
    kernels of the exchange, and the caller leaves `reserved_sms()` SMs out of the GEMM grid for them.  The GEMM
    kernels read only their own GPU's buffer, with ordinary TMA loads.
    """

    NCCL_CTAS = 1      # the one-word all-reduces need a single CTA
    COPY_STREAMS = 8   # pushes to different peers go out on streams of their own: under the GEMM's memory load a single
                       # copy is latency-bound, and the step time at 8 GPUs fell from 1.07 ms (one stream) to 0.93 ms (eight)

    def __init__(self, shard: torch.Tensor, rows: int, world: int, rank: int, group=None):
        if not shard.is_cuda:
            raise ValueError("PeerGather moves data between GPUs: CUDA tensors only")
        import torch.distributed._symmetric_memory as symm_mem

        shape = (rows, shard.shape[1])
        bufs = [symm_mem.empty(shape, dtype=shard.dtype, device=shard.device) for _ in range(2)]
        super().__init__(shard, rows, world, group, bufs=bufs)
        self.rank = rank
        pg = group if group is not None else dist.group.WORLD
        handles = [symm_mem.rendezvous(b, pg) for b in bufs]
        # peer[r][j]: rank r's buffer j as a tensor of this process (this rank's own buffers for r == rank)
        self.peer = [bufs if r == rank else [h.get_buffer(r, shape, shard.dtype) for h in handles]
                     for r in range(world)]
        self.word = torch.zeros(1, dtype=torch.int32, device=shard.device)
        self.copy_streams = [torch.cuda.Stream(device=shard.device)
                             for _ in range(int(os.environ.get("SB200_COPY_STREAMS", self.COPY_STREAMS)))]
        self.rows_of = [row_shard(rows, world, r) for r in range(world)]
        self.pieces = max(1, int(os.environ.get("SB200_COPY_PIECES", "1")))  # copies per peer and step
        dist.barrier(group=group)  # every process has mapped every buffer before the first push

    def _start(self) -> None:
        j = self.issued % 2
        self.comm.wait_event(self.consumed[j])            # my GEMM that read buffer j is over
        with torch.cuda.stream(self.comm):
            dist.all_reduce(self.word, group=self.group)  # ... and so is everyone else's: buffer j is free everywhere
        b0, b1 = self.rows_of[self.rank]
        nstreams = len(self.copy_streams)
        if nstreams:
            free = torch.cuda.Event()
            free.record(self.comm)
        pieces = self.pieces
        step = (b1 - b0 + pieces - 1) // pieces
        n = 0
        for idx in range(self.world):
            r = (self.rank + idx) % self.world            # start with the local copy, then the peers in ring order
            for lo in range(0, b1 - b0, step):
                hi = min(lo + step, b1 - b0)
                s = self.copy_streams[n % nstreams] if nstreams else self.comm
                if nstreams and n < nstreams:
                    s.wait_event(free)
                n += 1
                with torch.cuda.stream(s):
                    self.peer[r][j][b0 + lo:b0 + hi].copy_(self.shard[lo:hi], non_blocking=True)
        for s in self.copy_streams:
            self.comm.wait_stream(s)
        with torch.cuda.stream(self.comm):
            dist.all_reduce(self.word, group=self.group)  # every rank's pushes into every buffer j have landed
            self.filled[j].record(self.comm)
        self.issued += 1


def slab_gemm(a_slab: torch.Tensor, b_shard: torch.Tensor, k: int, world: int, rank: int,
              local_gemm: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
              b_full: Optional[torch.Tensor] = None, group=None) -> torch.Tensor:
    """Row-slab plan, one step: all-gather B, then the local GEMM on this rank's rows of A.  Returns this rank's
    rows of C.  `local_gemm` is `runner.gemm` bound to a kernel on a GPU; tests pass a CPU stand-in."""
    n = b_shard.shape[1]
    if b_full is None:
        b_full = torch.empty((k, n), dtype=b_shard.dtype, device=b_shard.device)
    if world > 1:
        all_gather_rows(b_full, b_shard, world, group)
    else:
        b_full.copy_(b_shard)
    return local_gemm(a_slab, b_full)
