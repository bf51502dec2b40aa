"""Fused FSDP collectives over NVLink peer memory (replaces torch FSDP2's NCCL all-gather / reduce-scatter,
reference: llmtuner/parallel/fully_shard_parallel/fully_shard_parallel.py:198-604, policies.py:100-141).

Every rank allocates one symmetric arena (torch symmetric memory does the allocation and the peer mapping) holding
the low-precision parameter shards of the block units, the two rotating flat gradient buffers and a small array of
epoch flags. Collectives are cut into `SideJob` slices and handed to the comm warps of the GEMM kernels that are being
launched anyway (`ops.gemm` asks the queue for a slice sized to the GEMM's work), so the transfer runs inside the
compute kernels, tile by tile, on the compute stream:

  all-gather      each peer's shard is copied by P2P loads into the local gather slot; the job of block i+1 rides on
                  the GEMMs of block i (block i-1 in backward)
  reduce-scatter  this rank's slice of every peer's bf16 gradient buffer is read by P2P loads, summed in fp32 in rank
                  order (deterministic) and written / accumulated into the fp32 gradient shard: the cast and the
                  accumulation are part of the transfer; the job of block i rides on the backward GEMMs of block i-1

Ordering: gradients become readable when their owner publishes a `ready` epoch into every peer's flag array; a
gradient slot is rewritten only after every peer published `done` for its previous use; parameter shards are only read
between the two step-level synchronisations that the optimizer phase provides (the gradient-norm all-reduce before the
update, a one-element all-reduce after it). Every device-side wait is bounded and reports through the status word.
What is left of a job when its data is needed is finished by a standalone kernel that runs the same device code.
"""
from __future__ import annotations

import os
from collections import deque
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

COPY, REDUCE = 1, 2


@dataclass
class Job:
    kind: int
    src: list[int]
    dst: int
    n: int                       # copy: bytes; reduce: elements
    quantum: int                 # slice granularity in units of n (copy: 16 bytes; reduce: 8 elements)
    src_stride: int              # bytes that src pointers advance per unit of n
    dst_stride: int
    accumulate: bool = False
    wait_flags: int = 0
    n_wait: int = 0
    wait_value: int = 0
    tag: object = None
    on_done: list = field(default_factory=list)
    done: int = 0

    @property
    def remaining(self) -> int:
        return self.n - self.done

    def bytes_per_unit(self) -> int:
        return self.src_stride * (len(self.src) if self.kind == REDUCE else 1)

    def cut(self, max_units: int):
        """Take up to `max_units` units (rounded down to the quantum, at least one quantum). Returns a dict of the
        slice's absolute arguments."""
        take = min(self.remaining, max(self.quantum, max_units // self.quantum * self.quantum))
        s = dict(kind=self.kind, src=[p + self.done * self.src_stride for p in self.src], dst=self.dst + self.done * self.dst_stride,
                 n=take, accumulate=self.accumulate, wait_flags=self.wait_flags, n_wait=self.n_wait, wait_value=self.wait_value)
        self.done += take
        return s


class CommQueue:
    """FIFO of pending jobs. `take(flops)` cuts a slice for a GEMM of that size; `flush(tag)` finishes jobs now."""

    def __init__(self, ext=None, bytes_per_gflop: float | None = None, min_flops: float = 2e9):
        self.ext = ext
        self.jobs: deque[Job] = deque()
        self.bytes_per_gflop = bytes_per_gflop if bytes_per_gflop is not None else float(os.environ.get("LLMT_COMM_BYTES_PER_GFLOP", 4e5))
        self.min_flops = min_flops
        self.stats = {"slices_fused": 0, "slices_standalone": 0, "bytes_fused": 0, "bytes_standalone": 0}

    def __bool__(self) -> bool:
        return bool(self.jobs)

    def push(self, job: Job) -> None:
        if job.n > 0:
            self.jobs.append(job)
        else:
            for cb in job.on_done:
                cb()

    def take(self, flops: float):
        """Returns (slice dict | None, callbacks to run after the carrying kernel was launched)."""
        if not self.jobs or flops < self.min_flops:
            return None, ()
        job = self.jobs[0]
        budget_bytes = flops / 1e9 * self.bytes_per_gflop
        s = job.cut(int(budget_bytes // max(1, job.bytes_per_unit())))
        self.stats["slices_fused"] += 1
        self.stats["bytes_fused"] += s["n"] * job.bytes_per_unit()
        cbs = ()
        if job.remaining == 0:
            self.jobs.popleft()
            cbs = tuple(job.on_done)
        return s, cbs

    def _run_standalone(self, job: Job, ctas: int = 64) -> None:
        while job.remaining > 0:
            s = job.cut(job.remaining)
            self.stats["slices_standalone"] += 1
            self.stats["bytes_standalone"] += s["n"] * job.bytes_per_unit()
            if self.ext is not None:
                self.ext.side_job(make_side_job(self.ext, s), ctas)
        for cb in job.on_done:
            cb()

    def flush(self, tag=None) -> None:
        """Finish every job up to and including the last one carrying `tag` (all jobs when tag is None), in order."""
        if not self.jobs:
            return
        if tag is None:
            last = len(self.jobs) - 1
        else:
            idx = [i for i, j in enumerate(self.jobs) if j.tag is tag]
            if not idx:
                return
            last = idx[-1]
        for _ in range(last + 1):
            self._run_standalone(self.jobs.popleft())


def make_side_job(ext, s: dict):
    j = ext.SideJob()
    j.kind, j.src, j.dst, j.n = s["kind"], s["src"], s["dst"], s["n"]
    j.accumulate, j.wait_flags, j.n_wait, j.wait_value = s["accumulate"], s["wait_flags"], s["n_wait"], s["wait_value"]
    return j


_ACTIVE: CommQueue | None = None


def active_queue() -> CommQueue | None:
    return _ACTIVE


def set_active_queue(q: CommQueue | None) -> None:
    global _ACTIVE
    _ACTIVE = q


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


CANARY = 0x5AFEC0DE


_ARENAS: list = []      # weak references to every arena that carries a canary, for `damaged_arenas`


def write_canary(arena: torch.Tensor, nbytes: int = 256) -> None:
    """Fill the last `nbytes` of a symmetric arena with a known pattern; nothing in the arena's layout uses them."""
    import weakref
    arena[-nbytes:].view(torch.int32).fill_(CANARY - (1 << 32) if CANARY >= (1 << 31) else CANARY)
    _ARENAS.append(weakref.ref(arena))


def canary_intact(arena: torch.Tensor, nbytes: int = 256) -> bool:
    """Host-side check (synchronises): False means some kernel, local or on a peer, wrote past a buffer of the arena."""
    want = CANARY - (1 << 32) if CANARY >= (1 << 31) else CANARY
    return bool((arena[-nbytes:].view(torch.int32) == want).all().item())


def damaged_arenas() -> int:
    """How many live symmetric arenas have lost their canary words (synchronises; a debugging check)."""
    bad, live = 0, []
    for r in _ARENAS:
        a = r()
        if a is not None:
            live.append(r)
            bad += 0 if canary_intact(a) else 1
    _ARENAS[:] = live
    return bad


class FusedFSDPComm:
    """Owner of the symmetric arena and of the gather / reduce protocols for the dense block units of one runtime."""

    def __init__(self, rt):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops.cuda_ext import load
        self.rt, self.ext = rt, load()
        self.world, self.rank, self.group = rt.world, rt.rank, rt.group
        self.units = [u for us in rt.block_units.values() for u in us if not u.is_expert and u.world == rt.world and not getattr(u, "persistent", False)]
        if not self.units:
            self._ids = set()
            self.queue = None
            return
        # The two gradient slots and the chunk arithmetic assume units of one size. Where decoder blocks differ (hybrid
        # mixers, a dense first layer before sparse ones) the most common size takes the peer-memory path and the odd
        # units keep the NCCL collectives of the same runtime (`supports(u)` is the switch, unit by unit).
        sizes: dict[int, int] = {}
        for u in self.units:
            sizes[u.padded] = sizes.get(u.padded, 0) + 1
        common = max(sizes, key=lambda k: (sizes[k], k))
        if len(sizes) > 1:
            from ..utils import get_logger
            odd = sum(n for k, n in sizes.items() if k != common)
            get_logger().info(f"fused FSDP collectives cover {sizes[common]} of {len(self.units)} block units (one size); {odd} "
                              f"units of {len(sizes) - 1} other sizes use NCCL")
        self.units = [u for u in self.units if u.padded == common]
        self._ids = {id(u) for u in self.units}
        self.padded = common
        esz = self.units[0].shard_lowp.element_size()
        self.esz = esz
        off, self.shard_off = 0, {}
        for u in self.units:
            self.shard_off[id(u)] = off
            off += _align(u.shard_numel * esz)
        self.grad_off = [off, off + _align(self.padded * esz)]
        off += 2 * _align(self.padded * esz)
        self.flag_off = off
        self.n_flags = 4 * self.world                    # [slot][ready|done][src rank]
        off += _align(self.n_flags * 4)
        self.arena = symm_mem.empty(off + 256, dtype=torch.uint8, device=rt.device)
        self.arena.zero_()
        write_canary(self.arena)
        self.hdl = symm_mem.rendezvous(self.arena, self.group)
        self.peer_base = [int(p) for p in self.hdl.buffer_ptrs]
        self.base = self.peer_base[self.rank]
        assert self.base == self.arena.data_ptr()
        dt = self.units[0].param_dtype
        # move the shards and the gradient slots into the arena
        for u in self.units:
            view = self.arena[self.shard_off[id(u)]: self.shard_off[id(u)] + u.shard_numel * esz].view(dt)
            view.copy_(u.shard_lowp)
            if not u.separate_master:
                u.master = view
            u.shard_lowp = view
        self.grad_slots = [self.arena[o: o + self.padded * esz].view(dt) for o in self.grad_off]
        use_main = dt == torch.bfloat16
        for u in self.units:
            u.bind_grad(self.grad_slots[rt._unit_slot(u)], use_main)
        self.slot_epoch = [0, 0]
        self.queue = CommQueue(self.ext)
        set_active_queue(self.queue)
        torch.cuda.synchronize()
        self.hdl.barrier()
        self._sync = torch.zeros(1, dtype=torch.float32, device=rt.device)

    # ------------------------------------------------------------------ helpers
    def supports(self, u) -> bool:
        return self.queue is not None and id(u) in self._ids

    def _flag_ptr(self, peer: int, slot: int, which: int, src_rank: int = 0) -> int:
        return self.peer_base[peer] + self.flag_off + 4 * ((slot * 2 + which) * self.world + src_rank)

    def _signal(self, slot: int, which: int, value: int) -> None:
        ptrs = [self.peer_base[p] + self.flag_off for p in range(self.world)]
        self.ext.signal_peers(ptrs, (slot * 2 + which) * self.world + self.rank, value)

    # ------------------------------------------------------------------ all-gather
    def all_gather(self, u) -> None:
        S = u.shard_numel * self.esz
        for k in range(self.world):
            p = (self.rank + k) % self.world          # own shard first, then peers in ring order (spreads link load)
            self.queue.push(Job(COPY, [self.peer_base[p] + self.shard_off[id(u)]], u.full.data_ptr() + p * S, S, 16, 1, 1, tag=u))

    def wait_gather(self, u) -> None:
        self.queue.flush(u)

    # ------------------------------------------------------------------ reduce-scatter
    def before_grad_write(self, u) -> None:
        """The gradient slot of `u` is about to be overwritten: every peer must be done reading its previous content."""
        slot = self.rt._unit_slot(u)
        e = self.slot_epoch[slot]
        if e > 0:
            self.ext.wait_flags(self._flag_ptr(self.rank, slot, 1), self.world, e, 6000 + slot)

    def reduce_scatter(self, u, accumulate: bool) -> None:
        slot = self.rt._unit_slot(u)
        self.slot_epoch[slot] += 1
        e = self.slot_epoch[slot]
        self._signal(slot, 0, e)                       # my gradients of this unit are complete (stream-ordered)
        a, _ = u.my_range()
        src = [self.peer_base[p] + self.grad_off[slot] + a * self.esz for p in range(self.world)]
        job = Job(REDUCE, src, u.grad_shard.data_ptr(), u.shard_numel, 8, self.esz, 4, accumulate=accumulate,
                  wait_flags=self._flag_ptr(self.rank, slot, 0), n_wait=self.world, wait_value=e, tag=("rs", id(u)))
        job.on_done.append(lambda s=slot, v=e: self._signal(s, 1, v))
        self.queue.push(job)

    def flush_all(self) -> None:
        self.queue.flush(None)

    def check_canaries(self) -> bool:
        return canary_intact(self.arena)

    def step_barrier(self) -> None:
        """After the optimizer rewrote the shards: nobody may read them before everybody has finished writing."""
        dist.all_reduce(self._sync, group=self.group)


def enable_fused_fsdp(rt) -> FusedFSDPComm | None:
    """Switch the runtime's dense block units to the peer-memory path when the platform allows it."""
    if not rt.is_cuda or rt.world == 1 or rt.implementation != "native":
        return None
    if rt.param_dtype != torch.bfloat16 or rt.world > 8:
        return None
    if os.environ.get("LLMT_DISABLE_FUSED_COMM") == "1":
        return None
    fused = FusedFSDPComm(rt)
    if fused.queue is None:
        return None
    rt.fused = fused
    return fused
