"""Multi-GPU plan for one box: one GEMM divided over the GPUs, operands exchanged over NVLink.

The reference project is single-GPU (device 0 only, src/cuda/kernel_runner_support.cuh:312 there); this module is
the one exchange step the path needs when it runs on 2, 4 or 8 GPUs of a box.  One process per GPU.  The GPUs form a
pr x pc grid; GPU (i, j) computes the block C[i, j] = A[i, :] B[:, j] with an independent local Strassen-Winograd
GEMM on an (M/pr) x (N/pc) x K problem.  The row slab A[i, :] is needed by the pc GPUs of grid row i and starts
row-sharded among them; the column slab B[:, j] is needed by the pr GPUs of grid column j and starts K-sharded among
them.  Every step each GPU pushes its two shards into the buffers of the GPUs that share its slabs; the kernels then
read local memory only (plain, non-multicast TMA).  A 1-D split (pr = P) would make every GPU receive (P-1)/P of B;
the grid that `grid_plan` picks moves the fewest bytes (8 GPUs at 16384^3: 256 MiB per GPU and step instead of 448).

`GridExchange` moves the shards with the copy engines into symmetric memory and orders the GPUs with the library's
bounded flag kernels (sb200_peer_signal / sb200_peer_wait); `CollectiveGridExchange` does the same exchange with
all-gathers in sub-groups on any torch.distributed backend - it is what the CPU tests (gloo) run, and the fallback
where peer mappings cannot be set up.  `SlabPlan`, `all_gather_rows`, `PipelinedGather` and `PeerGather` are the 1-D
row-slab forms of the same plan.
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


@dataclass(frozen=True)
class GridPlan:
    kind: str            # "grid" or "replica" (the problem does not divide: independent replicas, no exchange)
    world: int
    pr: int              # grid rows: C and A are cut into pr row slabs
    pc: int              # grid columns: C and B are cut into pc column slabs
    m: int
    n: int
    k: int
    local_m: int         # shape of the local GEMM: local_m x local_n x k
    local_n: int
    a_recv_bytes: int    # bytes each GPU receives per GEMM for its A slab and its B slab
    b_recv_bytes: int

    def coords(self, rank: int) -> Tuple[int, int]:
        return divmod(rank, self.pc)

    def row_group(self, rank: int) -> List[int]:
        """Ranks of this rank's grid row (they share the A slab), in shard order."""
        i, _ = self.coords(rank)
        return [i * self.pc + j for j in range(self.pc)]

    def col_group(self, rank: int) -> List[int]:
        """Ranks of this rank's grid column (they share the B slab), in shard order."""
        _, j = self.coords(rank)
        return [i * self.pc + j for i in range(self.pr)]

    def a_shard_rows(self) -> int:
        return self.local_m // self.pc

    def b_shard_rows(self) -> int:
        return self.k // self.pr

    def describe(self) -> str:
        if self.kind != "grid":
            return f"{self.world} independent replicas"
        return (f"{self.pr} x {self.pc} grid of GPUs, local {self.local_m}x{self.local_n}x{self.k}; per step every GPU "
                f"receives {(self.a_recv_bytes + self.b_recv_bytes) / 2**20:.0f} MiB "
                f"(A slab {self.a_recv_bytes / 2**20:.0f}, B slab {self.b_recv_bytes / 2**20:.0f}) over NVLink")


def grid_plan(m: int, n: int, k: int, world: int, esize: int, level: int = 1, tile: int = 256) -> GridPlan:
    """The pr x pc grid (pr * pc = world) whose exchange moves the fewest bytes, among those whose local problem still
    cuts into whole tiles per quadrant and whose shards are whole rows.  Ties go to the taller grid."""
    if world == 1:
        return GridPlan("grid", 1, 1, 1, m, n, k, m, n, 0, 0)
    div = 1 << level
    best = None
    for pr in range(world, 0, -1):
        if world % pr:
            continue
        pc = world // pr
        if m % pr or n % pc or k % pr:
            continue
        lm, ln = m // pr, n // pc
        if lm % pc or lm % (div * tile) or ln % (div * tile) or k % (div * 64):
            continue
        a_recv = (pc - 1) * (lm // pc) * k * esize
        b_recv = (pr - 1) * (k // pr) * ln * esize
        cand = GridPlan("grid", world, pr, pc, m, n, k, lm, ln, a_recv, b_recv)
        if best is None or a_recv + b_recv < best.a_recv_bytes + best.b_recv_bytes:
            best = cand
    return best if best is not None else GridPlan("replica", world, world, 1, m, n, k, m, n, 0, 0)


A_SUBSEQUENCE = 1000   # generator subsequences of the shards: A shard (i, j) and B shard (i, j) of the grid
B_SUBSEQUENCE = 2000


def make_shards(gp: GridPlan, rank: int, dtype: str, device, seed: int = 1):
    """This rank's shard of its A slab and of its B slab, filled by the seeded generator (every rank can regenerate
    any shard, which is how the exchange is verified)."""
    from . import inputs

    i, j = gp.coords(rank)
    return (_fill(inputs, dtype, (gp.a_shard_rows(), gp.k), seed, A_SUBSEQUENCE + i * gp.pc + j, device),
            _fill(inputs, dtype, (gp.b_shard_rows(), gp.local_n), seed, B_SUBSEQUENCE + i * gp.pc + j, device))


def _fill(inputs, dtype, shape, seed, subsequence, device):
    if torch.device(device).type == "cuda":
        return inputs.fill_device(dtype, "uniform1", shape, seed, subsequence, device)
    return torch.from_numpy(inputs.fill_host(dtype, "uniform1", shape, seed, subsequence))


def expected_slabs(gp: GridPlan, rank: int, dtype: str, device, seed: int = 1):
    """The whole A slab and B slab of this rank as the exchange must deliver them, regenerated locally."""
    from . import inputs

    i, j = gp.coords(rank)
    a = torch.cat([_fill(inputs, dtype, (gp.a_shard_rows(), gp.k), seed, A_SUBSEQUENCE + i * gp.pc + jj, device)
                   for jj in range(gp.pc)])
    b = torch.cat([_fill(inputs, dtype, (gp.b_shard_rows(), gp.local_n), seed, B_SUBSEQUENCE + ii * gp.pc + j, device)
                   for ii in range(gp.pr)])
    return a, b


def verify_block(gp: GridPlan, rank: int, seed: int, d: torch.Tensor, ai_bi, tol: float = 2e-3) -> bool:
    """Correctness evidence for one step of a grid exchange: the slabs this rank multiplied equal the shards their
    owners generated (bit for bit: the exchange delivered the right bytes to the right place), and sampled rows of the
    block D agree with the fp64 product of those slabs, as does the block's checksum."""
    a, b = ai_bi
    dtype = {torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32", torch.float64: "f64"}[a.dtype]
    want_a, want_b = expected_slabs(gp, rank, dtype, a.device, seed)
    ok = bool(torch.equal(a, want_a)) and bool(torch.equal(b, want_b))
    del want_a, want_b
    rows = torch.tensor([0, d.shape[0] // 3, d.shape[0] // 2 + 1, d.shape[0] - 1], device=a.device)
    truth = a[rows].double() @ b.double()
    err = float((d[rows].double() - truth).norm() / truth.norm())
    ok = ok and err < tol
    total = float(d.double().sum())
    want = float(a.double().sum(dim=0) @ b.double().sum(dim=1))
    scale = float(a.double().abs().sum(dim=0) @ b.double().abs().sum(dim=1))
    return ok and abs(total - want) <= 2e-5 * scale


class CollectiveGridExchange:
    """The grid exchange with collectives: an all-gather of the A shards inside every grid row and of the B shards
    inside every grid column, on any torch.distributed backend.  Synchronous with the compute stream."""

    @staticmethod
    def reserved_sms() -> int:
        return 0   # the collectives run between the GEMMs, not beside them

    def __init__(self, gp: GridPlan, rank: int, dtype: str, device, seed: int = 1):
        self.gp, self.rank, self.seed = gp, rank, seed
        self.a_shard, self.b_shard = make_shards(gp, rank, dtype, device, seed)
        # every rank creates every sub-group, in the same order
        self.row_pg = self.col_pg = None
        for i in range(gp.pr):
            ranks = [i * gp.pc + j for j in range(gp.pc)]
            pg = dist.new_group(ranks) if gp.pc > 1 else None
            if rank in ranks:
                self.row_pg = pg
        for j in range(gp.pc):
            ranks = [i * gp.pc + j for i in range(gp.pr)]
            pg = dist.new_group(ranks) if gp.pr > 1 else None
            if rank in ranks:
                self.col_pg = pg
        self.a = torch.empty((gp.local_m, gp.k), dtype=self.a_shard.dtype, device=device)
        self.b = torch.empty((gp.k, gp.local_n), dtype=self.b_shard.dtype, device=device)

    def next(self):
        gp = self.gp
        if gp.pc > 1:
            all_gather_rows(self.a, self.a_shard, gp.pc, self.row_pg)
        else:
            self.a.copy_(self.a_shard)
        if gp.pr > 1:
            all_gather_rows(self.b, self.b_shard, gp.pr, self.col_pg)
        else:
            self.b.copy_(self.b_shard)
        return self.a, self.b

    def done(self) -> None:
        pass

    def last(self):
        return self.a, self.b

    def check_status(self) -> None:
        pass

    def wait_ms(self, last_steps: int):
        return None   # the exchange is part of the compute stream's own work

    def verify_block(self, d: torch.Tensor, ai_bi, tol: float = 2e-3) -> bool:
        return verify_block(self.gp, self.rank, self.seed, d, ai_bi, tol)

    def describe(self) -> str:
        return "all-gathers in the grid's row and column groups before every GEMM (no overlap)"

    def close(self) -> None:
        pass


class GridExchange:
    """The grid exchange on real GPUs, buffered three deep and overlapped with compute.

    The A-slab and B-slab buffers live in symmetric memory (torch.distributed._symmetric_memory: every rank's buffer
    is mapped into every process).  A rank's own shard lives IN PLACE inside its own slab buffers (`shard_views(j)`
    is where the producer of the shard writes it for a step that uses buffer j); a slab that nobody shares is just
    the shard.  For step s every rank pushes its A shard into buffer s % 3 of the other ranks of its grid row and its
    B shard into buffer s % 3 of the other ranks of its grid column: device-to-device copies whose destination is peer
    memory, in several row blocks on streams of their own, so the copy engines move the bytes over NVLink and the
    GEMM keeps its SMs.  Ordering between GPUs uses counters in symmetric memory and the library's bounded flag
    kernels, never a collective:
      filled[j][r]    raised by rank r behind its pushes into my buffer j; my GEMM of step s waits for s + 1
      consumed[j][r]  raised by rank r behind its GEMM that read its buffer j; my pushes for step s into r's buffer
                      wait for s - 2 (the GEMM of step s - 3 is over)
    The pushes for steps s + 1 and s + 2 are in flight while step s computes.  The caller leaves `reserved_sms()` SMs
    out of the GEMM grid for the one-block flag kernels that run beside it; those run on streams of their own and
    meet the compute stream through events, so the GEMM launches of consecutive steps follow one another directly.
    """

    WAIT_LIMIT_US = 5_000_000   # bound of every flag wait (first steps include lazy set-up on the peers)
    PIECES = 2                  # every shard travels as this many row blocks on streams of their own: under the GEMM's
                                # memory load one copy is latency-bound, several copy engines together are not
    NBUF = 3                    # slab buffers per operand: a push has two steps' time to land
    MAX_COPY_STREAMS = 4        # the copies of a step are dealt over at most this many streams.  A process has a small
                                # number of hardware work queues (8 unless CUDA_DEVICE_MAX_CONNECTIONS says otherwise);
                                # with more streams than queues the GEMM's launches share a queue with copies that
                                # wait for another GPU and start late (measured on 4 and 8 B200s: the first launch of
                                # a step took 2.6 ms instead of 0.65 with two streams per peer)

    @staticmethod
    def reserved_sms() -> int:
        return 2

    def __init__(self, gp: GridPlan, rank: int, dtype: str, device, seed: int = 1, max_copy_streams: int = 0):
        import ctypes as C

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        self.lib = _lib.load()
        self.gp, self.rank, self.device, self.seed = gp, rank, torch.device(device), seed
        a_shard, b_shard = make_shards(gp, rank, dtype, device, seed)
        tdt = a_shard.dtype
        world, nbuf = gp.world, self.NBUF
        pg = dist.group.WORLD
        self.share_a, self.share_b = gp.pc > 1, gp.pr > 1
        a_shape, b_shape = (gp.local_m, gp.k), (gp.k, gp.local_n)
        # symmetric allocations are collective: every rank makes the same ones in the same order
        self.a_bufs = [symm_mem.empty(a_shape, dtype=tdt, device=device) for _ in range(nbuf)] if self.share_a else []
        self.b_bufs = [symm_mem.empty(b_shape, dtype=tdt, device=device) for _ in range(nbuf)] if self.share_b else []
        self.flags = symm_mem.empty((2 * nbuf * world,), dtype=torch.int32, device=device)   # [kind][buffer][rank]
        self.flags.zero_()
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        a_h = [symm_mem.rendezvous(t, pg) for t in self.a_bufs]
        b_h = [symm_mem.rendezvous(t, pg) for t in self.b_bufs]
        f_h = symm_mem.rendezvous(self.flags, pg)
        row, col = gp.row_group(rank), gp.col_group(rank)
        self.a_peers = [r for r in row if r != rank] if self.share_a else []
        self.b_peers = [r for r in col if r != rank] if self.share_b else []
        self.peers = sorted(set(self.a_peers) | set(self.b_peers))
        # peer views of the buffers this rank pushes into, and of the flag arrays it raises
        self.a_dst = {r: [h.get_buffer(r, a_shape, tdt) for h in a_h] for r in self.a_peers}
        self.b_dst = {r: [h.get_buffer(r, b_shape, tdt) for h in b_h] for r in self.b_peers}
        self.peer_flags = {r: f_h.get_buffer(r, (2 * nbuf * world,), torch.int32) for r in self.peers}
        self.a_rows = slice(row.index(rank) * gp.a_shard_rows(), (row.index(rank) + 1) * gp.a_shard_rows())
        self.b_rows = slice(col.index(rank) * gp.b_shard_rows(), (col.index(rank) + 1) * gp.b_shard_rows())
        # the shards in place: every buffer of a shared slab holds this rank's rows; an unshared slab is the shard
        self.a_own = [buf[self.a_rows] for buf in self.a_bufs] if self.share_a else [a_shard] * nbuf
        self.b_own = [buf[self.b_rows] for buf in self.b_bufs] if self.share_b else [b_shard] * nbuf
        for j in range(nbuf):
            if self.share_a:
                self.a_own[j].copy_(a_shard)
            if self.share_b:
                self.b_own[j].copy_(b_shard)
        self.comm = torch.cuda.Stream(device=device)
        # the flag kernels of the compute side run on streams of their own, tied to the compute stream by events, so
        # that the GEMM launches of consecutive steps follow one another without a flag kernel in between
        self.arrivals = torch.cuda.Stream(device=device)   # waits for the slabs of step s, one step after the other
        self.releases = torch.cuda.Stream(device=device)   # tells the peers that a buffer has been read
        n_copies = self.PIECES * (len(self.a_peers) + len(self.b_peers))
        limit = max_copy_streams if max_copy_streams > 0 else self.MAX_COPY_STREAMS
        self.copy_streams = [torch.cuda.Stream(device=device) for _ in range(min(limit, max(1, n_copies)))]
        self.consumed_local = [torch.cuda.Event() for _ in range(nbuf)]
        self.free_ev = [torch.cuda.Event() for _ in range(nbuf)]
        self.wait_events = []   # (before, after) event pairs around the compute stream's wait for a step's slabs
        for ev in self.consumed_local:
            ev.record(torch.cuda.current_stream(device))

        # flag addresses, fixed for the life of the exchange: [kind][buffer] -> pointer array
        def pointers(pairs):
            arr = (C.c_void_p * max(1, len(pairs)))()
            for n_, (t, idx) in enumerate(pairs):
                arr[n_] = t.data_ptr() + 4 * idx
            return arr

        self.signal_ptrs = [[pointers([(self.peer_flags[r], self._flag_index(kind, buf, rank)) for r in self.peers])
                             for buf in range(nbuf)] for kind in range(2)]
        self.wait_ptrs = [[pointers([(self.flags, self._flag_index(kind, buf, r)) for r in self.peers])
                           for buf in range(nbuf)] for kind in range(2)]
        self.issued = 0
        self.taken = 0
        self._last = None
        self.feeding = False
        self.fed = 0
        self.pushed = [torch.cuda.Event() for _ in range(nbuf)]     # my pushes out of buffer j have left
        self.uploaded = [torch.cuda.Event() for _ in range(nbuf)]   # fresh shards have reached buffer j (feeding)
        for ev in self.pushed:
            ev.record(torch.cuda.current_stream(device))
        torch.cuda.synchronize(device)
        dist.barrier()  # every process has mapped every buffer and zeroed its flags before the first push

    def _flag_index(self, kind: int, buf: int, rank: int) -> int:
        return (kind * self.NBUF + buf) * self.gp.world + rank

    def shard_views(self, j: int):
        """Where this rank's A shard and B shard live for a step that uses buffer j (write new shard values here
        before the step's `next`: the pushes read them from here)."""
        return self.a_own[j], self.b_own[j]

    def start_feeding(self) -> None:
        """From now on every step's shards come from the caller (`feed`), e.g. from pinned host memory: each GPU
        uploads only the 1/P of A and of B it owns, and the exchange spreads them over NVLink.  Steps whose pushes
        are already in flight keep the shards they were issued with."""
        if self.feeding:
            return
        nbuf = self.NBUF
        with torch.cuda.device(self.device):
            # a slab nobody shares is read by the GEMM where the shard lies: one copy per buffer, so that the upload
            # for a later step cannot touch what a running GEMM reads
            if not self.share_a:
                self.a_own = [self.a_own[0].clone() for _ in range(nbuf)]
            if not self.share_b:
                self.b_own = [self.b_own[0].clone() for _ in range(nbuf)]
            self.upload = torch.cuda.Stream(device=self.device)
            for ev in self.uploaded:
                ev.record(torch.cuda.current_stream(self.device))
        self.feeding = True
        self.fed = self.issued

    def feed(self, a_shard: torch.Tensor, b_shard: torch.Tensor, after: Optional[torch.cuda.Event] = None) -> None:
        """Shards of the next step that has none yet (steps are fed in order, before the `next` that starts their
        pushes: `next` of step s starts the pushes of step s + NBUF - 1).  Host tensors should be pinned: the copies
        are asynchronous, on a stream of their own, and wait for the GEMM and the pushes that last used the buffer
        (and for `after`, when given)."""
        if not self.feeding:
            raise RuntimeError("call start_feeding() first")
        j = self.fed % self.NBUF
        with torch.cuda.device(self.device):
            if after is not None:
                self.upload.wait_event(after)
            self.upload.wait_event(self.consumed_local[j])
            self.upload.wait_event(self.pushed[j])
            with torch.cuda.stream(self.upload):
                self.a_own[j].copy_(a_shard, non_blocking=True)
                self.b_own[j].copy_(b_shard, non_blocking=True)
            self.uploaded[j].record(self.upload)
        self.fed += 1

    def _signal(self, kind: int, buf: int, value: int, stream) -> None:
        """Raise my counter (kind, buf) in every peer's flag array to `value`, behind the work queued on `stream`."""
        if not self.peers:
            return
        rc = self.lib.sb200_peer_signal(self.signal_ptrs[kind][buf], len(self.peers), value, stream.cuda_stream)
        if rc:
            raise RuntimeError(f"sb200_peer_signal failed with {rc}")

    def _wait(self, kind: int, buf: int, value: int, stream) -> None:
        """Make `stream` wait until every peer's counter (kind, buf) in my flag array has reached `value`."""
        if not self.peers or value <= 0:
            return
        rc = self.lib.sb200_peer_wait(self.wait_ptrs[kind][buf], len(self.peers), value, self.WAIT_LIMIT_US,
                                      self.status.data_ptr(), stream.cuda_stream)
        if rc:
            raise RuntimeError(f"sb200_peer_wait failed with {rc}")

    def _start(self) -> None:
        s = self.issued
        j = s % self.NBUF
        if self.feeding and self.fed <= s:
            raise RuntimeError(f"step {s} has not been fed its shards")
        with torch.cuda.device(self.device):
            if self.feeding:
                self.comm.wait_event(self.uploaded[j])                    # the step's shards have arrived
            self.comm.wait_event(self.consumed_local[j])                  # my GEMM that read buffer j is over
            self._wait(1, j, s - self.NBUF + 1, self.comm)                # ... and so are the peers' (step s - NBUF)
            free = self.free_ev[j]
            free.record(self.comm)
            for st in self.copy_streams:
                st.wait_event(free)
            turn = 0
            for piece in range(self.PIECES):
                for dsts, rows, shard in ((self.a_dst, self.a_rows, self.a_own[j]), (self.b_dst, self.b_rows, self.b_own[j])):
                    n_rows = shard.shape[0]
                    lo = piece * n_rows // self.PIECES
                    hi = (piece + 1) * n_rows // self.PIECES
                    # peers in rank order on every rank: the low ranks are served first and start early, the others
                    # follow.  Measured on 8 B200s (256 MiB per GPU and step, about as much as the copy engines move
                    # in a step under the GEMM's memory load): 0.95-0.99 ms per step; with every rank starting at the
                    # peer after itself all ranks wait 0.07-0.18 ms for their slabs and the step takes 1.05 ms.
                    for r in sorted(dsts):
                        with torch.cuda.stream(self.copy_streams[turn % len(self.copy_streams)]):
                            dsts[r][j][rows.start + lo:rows.start + hi].copy_(shard[lo:hi], non_blocking=True)
                        turn += 1
            for st in self.copy_streams:
                self.comm.wait_stream(st)
            self.pushed[j].record(self.comm)
            self._signal(0, j, s + 1, self.comm)                          # my pushes for step s have landed everywhere
        self.issued += 1

    def next(self):
        """(A slab, B slab) of this step, valid on the current stream; the pushes for the steps after are started."""
        while self.issued < self.taken + self.NBUF:
            self._start()
        s = self.taken
        j = s % self.NBUF
        cur = torch.cuda.current_stream(self.device)
        before = torch.cuda.Event(enable_timing=True)
        after = torch.cuda.Event(enable_timing=True)
        before.record(cur)
        with torch.cuda.device(self.device):
            self._wait(0, j, s + 1, self.arrivals)
            arrived = torch.cuda.Event()
            arrived.record(self.arrivals)
            cur.wait_event(arrived)
            if self.feeding:
                cur.wait_event(self.uploaded[j])   # an unshared slab is read where the upload put it
        after.record(cur)
        self.wait_events.append((before, after))
        self.taken += 1
        self._last = (self.a_bufs[j] if self.share_a else self.a_own[j], self.b_bufs[j] if self.share_b else self.b_own[j])
        return self._last

    def done(self) -> None:
        """Call after the GEMM of the step handed out last has been enqueued on the current stream."""
        s = self.taken - 1
        j = s % self.NBUF
        cur = torch.cuda.current_stream(self.device)
        self.consumed_local[j].record(cur)
        with torch.cuda.device(self.device):
            self.releases.wait_event(self.consumed_local[j])
            self._signal(1, j, s + 1, self.releases)

    def last(self):
        return self._last

    def wait_ms(self, last_steps: int) -> float:
        """Mean device time per step the compute stream spent waiting for its slabs, over the last `last_steps` steps
        (call after a synchronize)."""
        pairs = self.wait_events[-last_steps:]
        return sum(b.elapsed_time(a) for b, a in pairs) / max(1, len(pairs))

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"grid exchange: device status {code} (a flag from another GPU did not arrive in time)")

    def verify_block(self, d: torch.Tensor, ai_bi, tol: float = 2e-3) -> bool:
        return verify_block(self.gp, self.rank, self.seed, d, ai_bi, tol)

    def describe(self) -> str:
        return "copy-engine pushes into symmetric memory, ordered by bounded flag kernels, under the GEMM before"

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier()   # nobody unmaps while a peer may still push or raise a flag


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
