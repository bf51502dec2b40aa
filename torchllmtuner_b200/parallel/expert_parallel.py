"""Expert parallelism (reference: llmtuner/parallel/expert_parallel/expert_parallel.py:25-100, block_conversion.py:40-292,
token_dispatch.py:319-678, domino_dispatch.py:36-390).

`apply_ep` gives every MoE block the expert slice `[r*E/ep, (r+1)*E/ep)` of its rank and binds an all-to-all token
dispatcher to the `ep` group. Dispatch: copies sorted by expert (stable), per-(rank, expert) counts exchanged, rows
exchanged, received rows regrouped expert-major into zero-padded 128-row segments for the grouped GEMM; combine runs
the inverse and accumulates score-weighted rows in fp32. The `domino` dispatcher splits the tokens in two halves and
overlaps the exchange of one half with the expert GEMMs of the other on a second stream. On CUDA the default
dispatcher is the peer-memory one of `parallel/symm_ep.py` (device-side counts, P2P row writes, no NCCL).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..errors import ConfigError
from ..models.moe import MoE
from ..models.moe.experts import SEG_ALIGN, padded_capacity, plan_segments


class _AllToAllRows(torch.autograd.Function):
    """all_to_all_single over dim 0 with explicit split sizes; backward swaps them."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits, group=ctx.group)
        return out, None, None, None


class AllToAllTokenDispatcher:
    def __init__(self, num_experts: int, group, ep_size: int, ep_rank: int, fp32_combine: bool = True):
        if num_experts % ep_size:
            raise ConfigError(f"expert_parallel_size {ep_size} must divide num_experts {num_experts}")
        self.num_experts, self.group, self.ep_size, self.ep_rank = num_experts, group, ep_size, ep_rank
        self.local_experts = num_experts // ep_size
        self.fp32_combine = fp32_combine
        self.timer = None

    # -- phases (split so that an overlapping driver can interleave them)
    def prepare_dispatch_counts(self, indices: torch.Tensor):
        flat = indices.reshape(-1)
        counts = torch.bincount(flat, minlength=self.num_experts).view(self.ep_size, self.local_experts)
        recv = torch.empty_like(counts)
        dist.all_to_all_single(recv, counts.contiguous(), group=self.group)      # recv[s, e] = rows rank s sends for my expert e
        # split sizes must be known on the host for the row exchange of this arm
        send_l, recv_l = counts.sum(1).tolist(), recv.sum(1).tolist()
        return flat, counts, recv, send_l, recv_l

    def dispatch(self, x: torch.Tensor, indices: torch.Tensor):
        T, k = indices.shape
        flat, counts, recv, send_l, recv_l = self.prepare_dispatch_counts(indices)
        order = torch.argsort(flat, stable=True)                                   # copies sorted by global expert
        rows_sorted = x.index_select(0, order // k)
        got = _AllToAllRows.apply(rows_sorted, recv_l, send_l, self.group)         # rank-major, expert-sorted per source
        # expert id of every received row, then expert-major padded layout
        eid = torch.repeat_interleave(torch.arange(self.local_experts, device=x.device).repeat(self.ep_size), recv.reshape(-1))
        dest, seg, _ = plan_segments(eid, self.local_experts)
        cap = -(-(int(eid.numel()) + self.local_experts * (SEG_ALIGN - 1)) // SEG_ALIGN) * SEG_ALIGN
        rows = got.new_zeros(cap, x.shape[1]).index_copy(0, dest, got)
        return rows, seg, {"T": T, "k": k, "order": order, "dest": dest, "send": send_l, "recv": recv_l}

    def combine(self, y: torch.Tensor, weights: torch.Tensor, st) -> torch.Tensor:
        back = _AllToAllRows.apply(y.index_select(0, st["dest"]), st["send"], st["recv"], self.group)   # sorted-copy order
        T, k = st["T"], st["k"]
        w = weights.reshape(-1).index_select(0, st["order"])
        acc_dtype = torch.float32 if self.fp32_combine else y.dtype
        out = torch.zeros(T, y.shape[1], dtype=acc_dtype, device=y.device)
        out.index_add_(0, st["order"] // k, back.to(acc_dtype) * w.to(acc_dtype).unsqueeze(-1))
        return out.to(y.dtype)


class DominoTokenDispatcher(AllToAllTokenDispatcher):
    """Two token halves: while the experts work on half 0, half 1 is exchanged on the side stream, and the combine of
    half 0 overlaps the experts of half 1 (reference: domino_dispatch.py:291)."""

    def run(self, experts, x, weights, indices):
        T = x.shape[0]
        h = T // 2
        if h == 0 or not x.is_cuda:
            rows, seg, st = self.dispatch(x, indices)
            return self.combine(experts(rows, seg), weights, st)
        side = getattr(self, "_side", None) or torch.cuda.Stream(x.device)
        self._side = side
        main = torch.cuda.current_stream()
        parts = [(x[:h], weights[:h], indices[:h]), (x[h:], weights[h:], indices[h:])]
        r0, s0, st0 = self.dispatch(*[parts[0][0], parts[0][2]])
        side.wait_stream(main)
        with torch.cuda.stream(side):
            r1, s1, st1 = self.dispatch(parts[1][0], parts[1][2])
        y0 = experts(r0, s0)
        main.wait_stream(side)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            o0 = self.combine(y0, parts[0][1], st0)
        y1 = experts(r1, s1)
        o1 = self.combine(y1, parts[1][1], st1)
        main.wait_stream(side)
        return torch.cat([o0, o1], 0)


def convert_block(moe: MoE, topo, ep_config) -> None:
    ep, r = topo.ep, topo.coord("ep")
    ex = moe.routed.experts
    E = ex.num_experts
    if E % ep:
        raise ConfigError(f"expert_parallel_size {ep} must divide num_experts {E}")
    n = E // ep
    for name in ("w1_EFD", "w3_EFD", "w2_EDF"):
        p = getattr(ex, name)
        if p.is_meta:
            new = nn.Parameter(torch.empty((n, *p.shape[1:]), dtype=p.dtype, device="meta"), requires_grad=p.requires_grad)
        else:
            new = nn.Parameter(p.detach()[r * n:(r + 1) * n].clone(), requires_grad=p.requires_grad)
        for k, v in p.__dict__.items():
            setattr(new, k, v)
        new.is_expert, new.ep_sharded = True, True
        new.ep_full_experts, new.ep_rank, new.ep_size = E, r, ep
        setattr(ex, name, new)
    ex.num_experts = n
    cls = DominoTokenDispatcher if ep_config.ep_token_dispatcher == "domino" else AllToAllTokenDispatcher
    moe.routed.dispatcher = cls(E, topo.get_group("ep"), ep, r)
    if cls is AllToAllTokenDispatcher:
        # 'alltoall' and 'fused': tokens move by P2P stores / loads over peer memory on CUDA bf16 (no NCCL, no host
        # synchronisation); the NCCL dispatcher stays behind it for CPU runs and unsupported shapes.
        from .symm_ep import PeerTokenDispatcher
        moe.routed.dispatcher = PeerTokenDispatcher(E, topo.get_group("ep"), ep, r, fallback=moe.routed.dispatcher,
                                                        capacity_factor=ep_config.ep_capacity_factor)
    if isinstance(moe.routed.dispatcher, DominoTokenDispatcher):
        d = moe.routed.dispatcher
        moe.routed.forward = lambda x, w, i, _d=d, _e=ex: _d.run(_e, x, w, i)


def build_ep_plan(model, topo, ep_config):
    """Resolve every MoE block against the untouched model: the degree must divide the experts of each block, the
    dispatcher must exist. Binds the block objects only: tensor parallelism, which runs first, re-creates the expert
    parameters (intermediate dimension cut) of the very blocks this plan names."""
    from .plan import ParallelPlan, PlanTarget
    targets = []
    for n, m in model.named_modules():
        if isinstance(m, MoE):
            E = m.routed.experts.num_experts
            if E % topo.ep:
                raise ConfigError(f"{n}: expert_parallel_size {topo.ep} must divide {E} experts")
            targets.append(PlanTarget(n, "moe", "ep", m))
    if not targets:
        raise ConfigError("expert_parallel_size > 1 but the model has no MoE block")
    return ParallelPlan("ep", topo.ep, ep_config.ep_token_dispatcher, tuple(targets), binds=("modules",),
                        notes=(f"{targets[0].module.routed.experts.num_experts // topo.ep} experts per rank",))


def apply_ep(model, topo, ep_config) -> dict:
    """Plan every block first (so a bad block raises before any mutation), then install."""
    blocks = [(n, m) for n, m in model.named_modules() if isinstance(m, MoE)]
    for n, m in blocks:
        if m.routed.experts.num_experts % topo.ep:
            raise ConfigError(f"{n}: expert_parallel_size {topo.ep} must divide {m.routed.experts.num_experts} experts")
    for n, m in blocks:
        convert_block(m, topo, ep_config)
    return {n: "ep" for n, _ in blocks}
