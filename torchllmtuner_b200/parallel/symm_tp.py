"""Tensor-parallel row collectives fused into the GEMMs that consume / produce them
(replaces `torch.ops.symm_mem.fused_all_gather_matmul` / `fused_matmul_reduce_scatter`,
reference: llmtuner/accelerator/linear_collectives.py:197-453, llmtuner/parallel/tensor_parallel/linear.py:23-192).

Every TP rank owns one symmetric arena with
  * two rotating chunk slots  `[T/R, D]` bf16: what this rank contributes to an all-gather,
  * two rotating partial slots `[T, D]` bf16: this rank's partial sums in front of a reduce-scatter,
  * a flag block `ready[R] | done[R]` per slot (values are the slot's epoch).
The all-gather form (`gemm_tp` mode 1) pulls peers' chunks into the local gathered matrix on the GEMM's comm warps while
the tensor-core warps already multiply the chunks that have landed; the reduce-scatter form (mode 2) publishes partial
tiles chunk by chunk from the epilogue and reduces this rank's chunk out of the peers' partial slots on the comm warps.
One gather feeds every column-parallel projection that follows it (q, k, v; gate, up); in backward their input
gradients are accumulated in the partial slot by the dgrad GEMMs themselves and the last one carries the reduce-scatter.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .symm import canary_intact, write_canary

AG, RS = 1, 2


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


class FusedTPComm:
    """Arena, epochs and launch helpers for one TP group. `rows` = T (gathered rows), `cols` = D."""

    N_SLOTS = 2

    def __init__(self, group, device, rows: int, cols: int):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops.cuda_ext import load
        self.ext = load()
        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.cols = rows, cols
        assert rows % (self.world * 128) == 0 and cols % 8 == 0
        self.chunk_rows = rows // self.world
        chunk_b, part_b = _align(self.chunk_rows * cols * 2), _align(rows * cols * 2)
        flag_b = _align(2 * self.world * 4)
        self.off_chunk = [i * chunk_b for i in range(self.N_SLOTS)]
        self.off_part = [self.N_SLOTS * chunk_b + i * part_b for i in range(self.N_SLOTS)]
        base = self.N_SLOTS * (chunk_b + part_b)
        self.off_flag = {(AG, i): base + i * flag_b for i in range(self.N_SLOTS)}
        self.off_flag.update({(RS, i): base + (self.N_SLOTS + i) * flag_b for i in range(self.N_SLOTS)})
        total = base + 2 * self.N_SLOTS * flag_b + 256
        self.arena = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.arena.zero_()
        write_canary(self.arena)
        self.hdl = symm_mem.rendezvous(self.arena, group)
        self.peer_base = [int(p) for p in self.hdl.buffer_ptrs]
        self.base = self.peer_base[self.rank]
        self.counters = {(k, i): torch.zeros(3 * self.world, dtype=torch.int32, device=device) for k in (AG, RS) for i in range(self.N_SLOTS)}
        self.epoch = {(k, i): 0 for k in (AG, RS) for i in range(self.N_SLOTS)}
        self.turn = {AG: 0, RS: 0}
        self.acc = torch.empty(self.chunk_rows * cols, dtype=torch.float32, device=device)
        self.stats = {"ag_fused": 0, "rs_fused": 0}
        torch.cuda.synchronize(device)
        self.hdl.barrier()

    # ------------------------------------------------------------------ helpers
    def check_canaries(self) -> bool:
        return canary_intact(self.arena)

    def fits(self, rows: int, cols: int) -> bool:
        return rows == self.rows and cols <= self.cols and cols % 8 == 0

    def _slot(self, kind: int):
        i = self.turn[kind]
        self.turn[kind] = (i + 1) % self.N_SLOTS
        self.epoch[(kind, i)] += 1
        e = self.epoch[(kind, i)]
        off = self.off_flag[(kind, i)]
        if e > 1:      # every reader of the slot's previous content has finished
            self.ext.wait_flags(self.base + off + 4 * self.world, self.world, e - 1, 7300 + 10 * kind + i)
        return i, e, off

    def _view(self, off: int, rows: int, cols: int) -> torch.Tensor:
        return self.arena[off: off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    # ------------------------------------------------------------------ all-gather -> GEMM
    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, b_mn: bool = False):
        """Returns (gather(x) @ op(w), gather(x)). `w` is [N, K] (b_mn False) or [K, N] (b_mn True)."""
        cr, K = x_shard.shape
        i, e, foff = self._slot(AG)
        self._view(self.off_chunk[i], cr, K).copy_(x_shard)
        self.ext.signal_peers([b + foff for b in self.peer_base], self.rank, e)      # ready[rank] on every rank
        # Rank skew is absorbed here, in a one-warp kernel, so that the waits inside the GEMM stay short.
        self.ext.wait_flags(self.base + foff, self.world, e, 7400 + i)
        gathered = torch.empty(cr * self.world, K, dtype=torch.bfloat16, device=self.device)
        N = w.shape[1] if b_mn else w.shape[0]
        y = torch.empty(cr * self.world, N, dtype=torch.bfloat16, device=self.device)
        self.ext.gemm_tp(gathered, w, y, b_mn, False, AG, self.world, self.rank, e, [b + self.off_chunk[i] for b in self.peer_base],
                         self.base + foff, [b + foff for b in self.peer_base], self.counters[(AG, i)])
        self.stats["ag_fused"] += 1
        return y, gathered

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def rs_begin(self, rows: int, cols: int):
        """Claims a partial slot (waiting until its previous readers are done). Returns a token and the `[rows, cols]`
        bf16 view that plain GEMMs may fill before `rs_finish` adds the last product and reduces."""
        i, e, foff = self._slot(RS)
        return (i, e, foff), self._view(self.off_part[i], rows, cols)

    def rs_finish(self, token, part: torch.Tensor, a: torch.Tensor, w: torch.Tensor, b_mn: bool, accumulate: bool,
                  residual: torch.Tensor | None = None) -> torch.Tensor:
        i, e, foff = token
        rows, N = part.shape
        out = torch.empty(rows // self.world, N, dtype=torch.bfloat16, device=self.device)
        self.ext.gemm_tp(a, w, part, b_mn, accumulate, RS, self.world, self.rank, e, [b + self.off_part[i] for b in self.peer_base],
                         self.base + foff, [b + foff for b in self.peer_base], self.counters[(RS, i)], self.acc, out, residual)
        self.stats["rs_fused"] += 1
        return out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False, residual=None) -> torch.Tensor:
        N = w.shape[1] if b_mn else w.shape[0]
        token, part = self.rs_begin(a.shape[0], N)
        return self.rs_finish(token, part, a, w, b_mn, False, residual)


    # ------------------------------------------------------------------ row collectives without a GEMM to ride on
    def all_gather_rows(self, x_shard: torch.Tensor) -> torch.Tensor:
        """[T/R, D] -> [T, D] by peer loads (the copy kernel of the FSDP path), same slots, flags and epochs as `ag_gemm`."""
        from .symm import COPY, make_side_job
        cr, K = x_shard.shape
        i, e, foff = self._slot(AG)
        self._view(self.off_chunk[i], cr, K).copy_(x_shard)
        self.ext.signal_peers([b + foff for b in self.peer_base], self.rank, e)
        self.ext.wait_flags(self.base + foff, self.world, e, 7500 + i)
        out = torch.empty(cr * self.world, K, dtype=torch.bfloat16, device=self.device)
        nbytes = cr * K * 2
        for k in range(self.world):
            p = (self.rank + k) % self.world
            job = dict(kind=COPY, src=[self.peer_base[p] + self.off_chunk[i]], dst=out.data_ptr() + p * nbytes, n=nbytes,
                       accumulate=False, wait_flags=0, n_wait=0, wait_value=0)
            self.ext.side_job(make_side_job(self.ext, job), 64)
        self.ext.signal_peers([b + foff + 4 * self.world for b in self.peer_base], self.rank, e)      # done[rank] everywhere
        return out

    def reduce_scatter_rows(self, partial: torch.Tensor) -> torch.Tensor:
        """[T, N] partial sums -> [T/R, N]: every rank publishes its partial, then sums its own chunk over all ranks in
        fp32 in rank order with peer loads (the reduce kernel of the FSDP path)."""
        from .symm import REDUCE, make_side_job
        rows, N = partial.shape
        cr = rows // self.world
        i, e, foff = self._slot(RS)
        self._view(self.off_part[i], rows, N).copy_(partial)
        self.ext.signal_peers([b + foff for b in self.peer_base], self.rank, e)                       # ready[rank] everywhere
        self.ext.wait_flags(self.base + foff, self.world, e, 7600 + i)
        n = cr * N
        acc = self.acc[:n]
        job = dict(kind=REDUCE, src=[b + self.off_part[i] + self.rank * n * 2 for b in self.peer_base], dst=acc.data_ptr(), n=n,
                   accumulate=False, wait_flags=0, n_wait=0, wait_value=0)
        self.ext.side_job(make_side_job(self.ext, job), 128)
        self.ext.signal_peers([b + foff + 4 * self.world for b in self.peer_base], self.rank, e)      # done[rank] everywhere
        return acc.view(cr, N).to(torch.bfloat16)


_COMMS: dict = {}


def fused_tp_comm(group, x_shard: torch.Tensor, device=None) -> FusedTPComm | None:
    """The group's fused communicator when the platform and the shape allow it, else None (callers fall back to NCCL).
    `x_shard` may be a meta tensor that only carries the chunk's shape and dtype, with `device` given separately."""
    device = device if device is not None else x_shard.device
    if device.type != "cuda" or x_shard.dtype != torch.bfloat16 or os.environ.get("LLMT_DISABLE_FUSED_TP") == "1":
        return None
    R = dist.get_world_size(group)
    cr, D = x_shard.shape[0], x_shard.shape[-1]
    if R < 2 or R > 8 or x_shard.dim() != 2 or cr % 128 or D % 8:
        return None
    key = id(group)
    comm = _COMMS.get(key)
    if comm is None:
        comm = _COMMS[key] = FusedTPComm(group, device, cr * R, D)
    return comm if comm.fits(cr * R, D) else None


def _wgrad(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor):
    from ..ops.functional import gemm
    main = getattr(w, "main_grad", None)
    if main is not None:
        gemm(dy, x, a_mn=True, b_mn=True, out=main, accumulate=getattr(w, "main_grad_initialized", False))
        w.main_grad_initialized = True
        return None
    return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=w.dtype)


class GatherLinears(torch.autograd.Function):
    """(x_shard [T/R, K], w_1 [N_1, K], ..., w_n) -> (gather(x) @ w_1^T, ..., gather(x) @ w_n^T). The gather rides on
    the first GEMM; in backward the dgrads accumulate in a partial slot and the last one carries the reduce-scatter."""

    @staticmethod
    def forward(ctx, comm: FusedTPComm, x_shard, *ws):
        from ..ops.functional import gemm
        y0, gathered = comm.ag_gemm(x_shard.contiguous(), ws[0])
        ys = [y0] + [gemm(gathered, w) for w in ws[1:]]
        ctx.comm = comm
        ctx.save_for_backward(gathered, *ws)
        return tuple(ys)

    @staticmethod
    def backward(ctx, *dys):
        from ..ops.functional import gemm
        gathered, *ws = ctx.saved_tensors
        comm = ctx.comm
        dys = [d.contiguous() for d in dys]
        dx = None
        if ctx.needs_input_grad[1]:
            token, part = comm.rs_begin(gathered.shape[0], gathered.shape[1])
            for j in range(len(ws) - 1, 0, -1):
                gemm(dys[j], ws[j], b_mn=True, out=part, accumulate=(j != len(ws) - 1))
            dx = comm.rs_finish(token, part, dys[0], ws[0], True, len(ws) > 1)
        dws = [(_wgrad(dys[j], gathered, ws[j]) if ctx.needs_input_grad[2 + j] else None) for j in range(len(ws))]
        return (None, dx, *dws)


class LinearReduceScatter(torch.autograd.Function):
    """(x [T, K/R], w [N, K/R]) -> reduce_scatter_rows(x @ w^T) [T/R, N]; backward gathers dy inside the dgrad GEMM."""

    @staticmethod
    def forward(ctx, comm: FusedTPComm, x, w):
        ctx.comm = comm
        ctx.save_for_backward(x, w)
        return comm.gemm_rs(x.contiguous(), w)

    @staticmethod
    def backward(ctx, dy_shard):
        x, w = ctx.saved_tensors
        comm = ctx.comm
        dx, dy = comm.ag_gemm(dy_shard.contiguous(), w, b_mn=True)             # gather(dy) [T, N] @ W [N, K/R]
        dw = _wgrad(dy, x, w) if ctx.needs_input_grad[2] else None
        return None, (dx if ctx.needs_input_grad[1] else None), dw


class PeerAllGatherRows(torch.autograd.Function):
    """[T/R, D] -> [T, D] over peer memory; backward reduce-scatters the gradient the same way."""

    @staticmethod
    def forward(ctx, comm: FusedTPComm, x):
        ctx.comm = comm
        return comm.all_gather_rows(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return None, ctx.comm.reduce_scatter_rows(g.contiguous())


class PeerReduceScatterRows(torch.autograd.Function):
    """[T, D] partial sums -> [T/R, D] over peer memory; backward all-gathers."""

    @staticmethod
    def forward(ctx, comm: FusedTPComm, x):
        ctx.comm = comm
        return comm.reduce_scatter_rows(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return None, ctx.comm.all_gather_rows(g.contiguous())
