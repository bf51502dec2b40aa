"""Vocabulary-parallel head + cross-entropy and embedding under sequence-parallel tensor parallelism
(reference: llmtuner/components/loss.py:92-238 `LossParallelCrossEntropy`, llmtuner/parallel/vocab_parallel/
vocab_parallel.py:16-96; the reference keeps the head replicated under sequence-parallel TP and rejects a vocab-sharded
one, llmtuner/parallel/execution.py:127-132, so its replicated head costs a 1.24 GB gradient all-reduce per step at
Qwen3-8B size; here the head is sharded and that all-reduce disappears).

Head: rank r owns rows `[r * chunk, (r + 1) * chunk)` of the `[V, D]` head. Hidden states arrive sequence-sharded
`[T/R, D]`. One step is
    logits_r = gather(h) @ W_r^T            all-gather riding on the GEMM (`FusedTPComm.ag_gemm`)
    loss, dlogits_r                         `ce_vocab_parallel` kernel: per token one exchange of (max, sum-exp, target
                                            logit) over peer memory, gradient written over the logits
    dW_r = dlogits_r^T gather(h)            local, needs no reduction
    dh   = reduce_scatter(dlogits_r @ W_r)  reduce-scatter riding on the GEMM (`FusedTPComm.gemm_rs`)
so the two row collectives are the ones every column- / row-parallel linear of the model already uses. On CPU (gloo) and
when the fused communicator is not available the same statement runs on torch.distributed collectives.

Every rank of the group computes the row losses of ALL tokens; the function returns the sum over this rank's own token
shard (so that sums over the loss mesh count each token once) while its backward scales the gradient of every row: the
upstream gradient is the same 1 / global_valid_tokens on all ranks of the group.

Embedding: `embed_scatter` writes each token's table row straight into the output shard of the rank that owns the token
(`vp_embed_scatter` kernel): exactly one rank owns an id, so nothing is reduced.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import IGNORE_INDEX
from ..utils.vocabulary import vocab_shard_bounds


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


class VocabExchange:
    """Symmetric arena of one TP group for the per-token statistics of the loss (`float4 [R][rows]` + `uint32 [R][rows]`
    epoch flags) and the embedding output shard `[rows / R, D]` bf16 with its arrival flags."""

    def __init__(self, group, device, rows: int, hidden: int):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops.cuda_ext import load
        from .symm import write_canary
        self.ext = load()
        self.group, self.device = group, device
        self.R, self.me = dist.get_world_size(group), dist.get_rank(group)
        agreed = torch.tensor([rows, hidden, -rows, -hidden], dtype=torch.int64, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=group)
        a = [int(v) for v in agreed.tolist()]
        if a[0] != rows or -a[2] != rows or a[1] != hidden or -a[3] != hidden:
            raise ValueError(f"tensor-parallel ranks disagree on the vocabulary exchange shape: rows {rows}, hidden {hidden} vs group {a}")
        self.rows, self.D = rows, hidden
        self.chunk = rows // self.R
        self.off_stats = 0
        self.off_flags = _align(self.R * rows * 16)
        self.off_emb = self.off_flags + _align(self.R * rows * 4)
        self.off_eflag = self.off_emb + _align(self.chunk * hidden * 2)
        total = self.off_eflag + _align(2 * self.R * 4) + 256
        self.arena = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.arena.zero_()
        write_canary(self.arena)
        self.hdl = symm_mem.rendezvous(self.arena, group)
        self.peer_base = [int(p) for p in self.hdl.buffer_ptrs]
        self.base = self.peer_base[self.me]
        self.epoch = 0
        self.emb_epoch = 0
        torch.cuda.synchronize(device)
        self.hdl.barrier()

    def ptrs(self, off: int) -> list[int]:
        return [b + off for b in self.peer_base]

    def cross_entropy_(self, logits: torch.Tensor, labels: torch.Tensor, vocab_start: int, write_grad: bool) -> torch.Tensor:
        """In place: `logits` [rows, V/R] becomes d(loss_sum)/d(logits); returns the fp32 row losses (all rows)."""
        self.epoch += 1
        return self.ext.ce_vocab_parallel(logits, labels, vocab_start, self.me, self.ptrs(self.off_stats), self.ptrs(self.off_flags),
                                          self.rows, self.epoch, 1.0, IGNORE_INDEX, write_grad)

    def embed(self, ids_full: torch.Tensor, weight: torch.Tensor, vstart: int, vend: int) -> torch.Tensor:
        """Rows of this rank's token shard, written by whichever rank owns each id."""
        self.emb_epoch += 1
        e = self.emb_epoch
        foff = self.off_eflag
        if e > 1:   # every rank has copied its previous shard out before anybody overwrites it
            self.ext.wait_flags(self.base + foff + 4 * self.R, self.R, e - 1, 8600)
        self.ext.vp_embed_scatter(ids_full, weight, vstart, vend, self.ptrs(self.off_emb), self.chunk)
        self.ext.signal_peers(self.ptrs(foff), self.me, e)                    # written[me] on every rank
        self.ext.wait_flags(self.base + foff, self.R, e, 8610)
        out = self.arena[self.off_emb: self.off_emb + self.chunk * self.D * 2].view(torch.bfloat16).view(self.chunk, self.D).clone()
        self.ext.signal_peers(self.ptrs(foff + 4 * self.R), self.me, e)       # copied[me] on every rank
        return out


_EXCHANGES: dict = {}


def vocab_exchange(group, device, rows: int, hidden: int) -> VocabExchange | None:
    if device.type != "cuda" or dist.get_world_size(group) > 8:
        return None
    key = (id(group), rows, hidden)
    if key not in _EXCHANGES:
        _EXCHANGES[key] = VocabExchange(group, device, rows, hidden)
    return _EXCHANGES[key]


class VocabParallelHead(nn.Module):
    """Rows `[start, end)` of the head. `forward` is the loss path's weight holder; logits for generation are produced
    by `full_logits` (gathers the vocabulary shards of this rank's tokens)."""

    def __init__(self, full: nn.Module, rank: int, size: int, group):
        super().__init__()
        V, D = full.weight.shape
        self.start, self.end = vocab_shard_bounds(V, size, rank)
        self.chunk = -(-V // size)
        w = full.weight
        local = torch.zeros(self.chunk, D, dtype=w.dtype, device=w.device if not w.is_meta else "meta")
        if not w.is_meta and self.end > self.start:
            local[: self.end - self.start] = w[self.start:self.end].detach()
        self.weight = nn.Parameter(local, requires_grad=w.requires_grad)
        self.weight.tp_shard_dim = 0
        self.weight.tp_full_shape = (V, D)
        self.weight.tp_vocab = True
        self.group, self.rank, self.size, self.vocab = group, rank, size, V

    def forward(self, h_shard: torch.Tensor) -> torch.Tensor:
        return self.full_logits(h_shard)

    @torch.no_grad()
    def full_logits(self, h_shard: torch.Tensor) -> torch.Tensor:
        """[T/R, D] -> [T/R, V] for evaluation and generation (not differentiable: training takes the loss path, which
        never forms full-vocabulary logits): every rank multiplies the gathered rows by its shard, the column blocks are
        exchanged."""
        from .tensor_parallel import all_gather_along
        shape = h_shard.shape
        h2 = h_shard.reshape(-1, shape[-1])
        hf = all_gather_along(h2, self.group)                                   # [T, D]
        part = torch.nn.functional.linear(hf, self.weight)                      # [T, chunk]
        cr = h2.shape[0]
        if part.is_cuda:
            pieces = [torch.empty(cr, self.chunk, dtype=part.dtype, device=part.device) for _ in range(self.size)]
            dist.all_to_all(pieces, [p.contiguous() for p in part.split(cr, dim=0)], group=self.group)
        else:       # gloo has no all-to-all: gather every rank's column block and keep this rank's token rows
            every = torch.empty(self.size * part.shape[0], part.shape[1], dtype=part.dtype, device=part.device)
            dist.all_gather_into_tensor(every, part.contiguous(), group=self.group)
            every = every.view(self.size, *part.shape)
            pieces = [every[r, self.rank * cr:(self.rank + 1) * cr] for r in range(self.size)]
        return torch.cat(pieces, dim=-1)[:, : self.vocab].reshape(*shape[:-1], self.vocab)


class _VocabParallelHeadLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h_shard, w, targets_shard, head: VocabParallelHead, num_chunks: int):
        group, R, rank = head.group, head.size, head.rank
        cr, D = h_shard.shape
        T = cr * R
        t_full = torch.empty(T, dtype=targets_shard.dtype, device=targets_shard.device)
        dist.all_gather_into_tensor(t_full, targets_shard.contiguous(), group=group)
        # a padded last shard owns fewer real rows than `chunk`: labels beyond `end` never match (they belong to nobody)
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        fused = None
        if h_shard.is_cuda and h_shard.dtype == torch.bfloat16 and head.chunk % 8 == 0:
            from .symm_tp import fused_tp_comm
            fused = fused_tp_comm(group, h_shard)
        if fused is not None:
            loss, dh, dw = _head_loss_fused(fused, h_shard, w, t_full, head, need_dh, need_dw)
        else:
            loss, dh, dw = _head_loss_torch(h_shard, w, t_full, head, need_dh, need_dw)
        ctx.save_for_backward(dh if dh is not None else torch.empty(0), dw if dw is not None else torch.empty(0))
        ctx.flags = (need_dh, need_dw, w.dtype, h_shard.dtype)
        return loss

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        need_dh, need_dw, wdt, hdt = ctx.flags
        return ((dh.float() * g).to(hdt) if need_dh else None, (dw.float() * g).to(wdt) if need_dw else None, None, None, None)


def _own_rows(rows: torch.Tensor, rank: int, R: int) -> torch.Tensor:
    cr = rows.shape[0] // R
    return rows[rank * cr:(rank + 1) * cr]


def _head_loss_fused(comm, h_shard, w, t_full, head: VocabParallelHead, need_dh: bool, need_dw: bool):
    from ..ops.functional import gemm
    R, rank = head.size, head.rank
    logits, h_full = comm.ag_gemm(h_shard.contiguous(), w)                       # [T, chunk] bf16, [T, D]
    ex = vocab_exchange(head.group, h_shard.device, h_full.shape[0], h_shard.shape[1])
    # columns past the real vocabulary of a padded last shard must not enter the softmax
    real = head.end - head.start
    view = logits if real == head.chunk else logits[:, :real]
    row_loss = ex.cross_entropy_(view, t_full, head.start, need_dh or need_dw)
    if real != head.chunk:
        logits[:, real:].zero_()
    loss = _own_rows(row_loss, rank, R).sum()
    dh = comm.gemm_rs(logits, w, b_mn=True) if need_dh else None                 # reduce_scatter(dlogits @ W_r) [T/R, D]
    dw = None
    if need_dw:
        dw = torch.empty(w.shape, dtype=torch.float32, device=w.device)
        gemm(logits, h_full, a_mn=True, b_mn=True, out=dw)                       # dlogits^T @ gather(h)
    return loss, dh, dw


def _head_loss_torch(h_shard, w, t_full, head: VocabParallelHead, need_dh: bool, need_dw: bool):
    group, R, rank = head.group, head.size, head.rank
    cr, D = h_shard.shape
    h_full = torch.empty(cr * R, D, dtype=h_shard.dtype, device=h_shard.device)
    dist.all_gather_into_tensor(h_full, h_shard.contiguous(), group=group)
    real = head.end - head.start
    lf = (h_full.float() @ w[:real].float().t()) if real > 0 else h_full.new_zeros(cr * R, 0, dtype=torch.float32)
    if h_shard.dtype != torch.float32:
        lf = lf.to(h_shard.dtype).float()          # the kernel path rounds the logits to the activation dtype
    lmax = lf.max(dim=-1).values if real > 0 else torch.full((cr * R,), float("-inf"), device=lf.device)
    gmax = lmax.clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    e = torch.exp(lf - gmax[:, None])
    local = t_full - head.start
    owned = (local >= 0) & (local < real) & (t_full != IGNORE_INDEX)
    tl = torch.where(owned, lf.gather(-1, local.clamp(0, max(real - 1, 0))[:, None]).squeeze(-1) if real > 0 else torch.zeros_like(gmax),
                     torch.zeros_like(gmax))
    packed = torch.stack([e.sum(-1), tl], dim=0)
    dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    sumexp, tlogit = packed[0], packed[1]
    valid = t_full != IGNORE_INDEX
    row_loss = torch.where(valid, torch.log(sumexp) + gmax - tlogit, torch.zeros_like(gmax))
    loss = _own_rows(row_loss, rank, R).sum()
    dh = dw = None
    if need_dh or need_dw:
        grad = e / sumexp[:, None]
        if real > 0:
            grad.scatter_add_(-1, local.clamp(0, real - 1)[:, None], -owned.to(grad.dtype)[:, None])
        grad = grad * valid.to(grad.dtype)[:, None]
        if need_dw:
            dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
            dw[:real] = grad.t() @ h_full.float()
        if need_dh:
            part = (grad @ w[:real].float()).to(h_shard.dtype) if real > 0 else torch.zeros_like(h_full)
            dh = torch.empty(cr, D, dtype=h_shard.dtype, device=h_shard.device)
            dist.reduce_scatter_tensor(dh, part.contiguous(), group=group)
    return loss, dh, dw


def vocab_parallel_head_loss(h_shard: torch.Tensor, head: VocabParallelHead, targets_shard: torch.Tensor, num_chunks: int = 1):
    """Sum of the cross-entropies of this rank's token shard `[T/R]` against the vocabulary-sharded head."""
    h2 = h_shard.reshape(-1, h_shard.shape[-1])
    return _VocabParallelHeadLoss.apply(h2, head.weight, targets_shard.reshape(-1), head, num_chunks)


class _EmbedScatter(torch.autograd.Function):
    """Sequence-sharded embedding output from a vocabulary-sharded table; backward gathers the output gradient rows over
    peer memory (or NCCL) and adds the rows of owned ids into the table shard's gradient."""

    @staticmethod
    def forward(ctx, weight, ids_full, emb, ex: VocabExchange | None):
        R, rank = emb.size, emb.rank
        if ex is not None:
            out = ex.embed(ids_full, weight, emb.start, emb.end)
        else:
            mine = (ids_full >= emb.start) & (ids_full < emb.end)
            rows = torch.nn.functional.embedding((ids_full - emb.start).clamp(0, emb.chunk - 1), weight)
            rows = rows * mine.to(rows.dtype).unsqueeze(-1)
            out = torch.empty(ids_full.shape[0] // R, weight.shape[1], dtype=weight.dtype, device=weight.device)
            dist.reduce_scatter_tensor(out, rows.contiguous(), group=emb.group)
        ctx.emb = emb
        ctx.save_for_backward(ids_full)
        ctx.wshape = weight.shape
        return out

    @staticmethod
    def backward(ctx, g):
        emb = ctx.emb
        (ids_full,) = ctx.saved_tensors
        R = emb.size
        g = g.contiguous()
        gf = None
        if g.is_cuda and g.dtype == torch.bfloat16:
            from .symm_tp import fused_tp_comm
            comm = fused_tp_comm(emb.group, g)
            if comm is not None:
                gf = comm.all_gather_rows(g)
        if gf is None:
            gf = torch.empty(g.shape[0] * R, g.shape[1], dtype=g.dtype, device=g.device)
            dist.all_gather_into_tensor(gf, g, group=emb.group)
        mine = (ids_full >= emb.start) & (ids_full < emb.end)
        dw = torch.zeros(ctx.wshape, dtype=torch.float32, device=g.device)
        dw.index_add_(0, (ids_full - emb.start)[mine], gf[mine].float())
        return dw.to(g.dtype), None, None, None
