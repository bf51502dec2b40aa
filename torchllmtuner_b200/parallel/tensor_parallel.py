"""Tensor parallelism with mandatory sequence parallelism
(reference: llmtuner/parallel/tensor_parallel/tensor_parallel.py:160-1180, linear.py:23-192, sharding.py:21-273,
sequence_boundary.py:18-110, llmtuner/accelerator/linear_collectives.py:120-453,
llmtuner/parallel/vocab_parallel/vocab_parallel.py:16-96).

Outside the GEMMs every activation is sequence-sharded `[T/tp, D]`. A block gathers the rows once in front of the
attention projections and once in front of gate/up (one gather feeds q, k and v; one feeds gate and up), runs
column-sharded GEMMs on full rows and local heads, and reduce-scatters the row-parallel outputs (o_proj, down_proj)
back to `[T/tp, D]`. MoE blocks gather in, run experts whose intermediate dimension is sharded, and reduce-scatter
out. The embedding and the head are vocabulary-parallel (`parallel/vocab_parallel.py`: every id's row is written straight
into the owner's token shard; the loss exchanges three scalars per token); the gradients of the parameters that stay
replicated (norms, q/k norms, router, and the head when `tp_vocab_parallel_head` is off) are summed over the TP group
before the data-parallel reduction.

Two implementations of the row collectives sit behind the same autograd functions: torch.distributed (NCCL / gloo)
and, on CUDA with peer access, staged P2P copies driven by the comm warps of the consuming / producing GEMM
(`parallel/symm_tp.py`).
"""
from __future__ import annotations

import os
import re

import torch
import torch.distributed as dist
import torch.nn as nn

from ..errors import ConfigError, UnsupportedCombinationError
from ..models.common import Linear
from ..utils.vocabulary import vocab_shard_bounds

# ---------------------------------------------------------------------------------------------- row collectives


class AllGatherRows(torch.autograd.Function):
    """[T/R, D] -> [T, D] in group-rank order; backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        R = dist.get_world_size(group)
        x = x.contiguous()
        out = torch.empty((x.shape[0] * R, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        R = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = torch.empty((g.shape[0] // R, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g, group=ctx.group)
        return out, None


class ReduceScatterRows(torch.autograd.Function):
    """[T, D] partial sums -> [T/R, D]; backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        R = dist.get_world_size(group)
        x = x.contiguous()
        out = torch.empty((x.shape[0] // R, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        R = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = torch.empty((g.shape[0] * R, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g, group=ctx.group)
        return out, None


def all_gather_along(x, group):
    return AllGatherRows.apply(x, group)


def reduce_scatter_along(x, group):
    return ReduceScatterRows.apply(x, group)


# ---------------------------------------------------------------------------------------------- sharded modules
class ShardedLinear(Linear):
    """A `Linear` that holds one TP shard of the full weight and remembers how to rebuild / re-cut it."""

    def __init__(self, full: Linear, dim: int, rank: int, size: int):
        n = full.weight.shape[dim]
        if n % size:
            raise UnsupportedCombinationError(f"tensor_parallel_size {size} does not divide dimension {n}")
        step = n // size
        nn.Module.__init__(self)
        self.in_features = full.in_features if dim == 0 else step
        self.out_features = step if dim == 0 else full.out_features
        w = full.weight
        shard = w.narrow(dim, rank * step, step) if not w.is_meta else torch.empty(
            (step, w.shape[1]) if dim == 0 else (w.shape[0], step), dtype=w.dtype, device="meta")
        self.weight = nn.Parameter(shard.detach().clone() if not w.is_meta else shard, requires_grad=w.requires_grad)
        self.weight.tp_shard_dim = dim
        self.weight.tp_full_shape = tuple(w.shape)
        self.tp_dim, self.tp_rank, self.tp_size = dim, rank, size


class ColwiseLinearNoGather(ShardedLinear):
    """Column shard applied to rows that are already complete (the enclosing boundary gathered them)."""

    def __init__(self, full, rank, size):
        super().__init__(full, 0, rank, size)


class ColumnParallelLinear(ShardedLinear):
    """all-gather rows -> GEMM on the column shard."""

    def __init__(self, full, rank, size, group):
        super().__init__(full, 0, rank, size)
        self.group = group

    def forward(self, x):
        return super().forward(all_gather_along(x, self.group))


class RowParallelLinear(ShardedLinear):
    """GEMM on the input-dimension shard -> reduce-scatter rows."""

    def __init__(self, full, rank, size, group):
        super().__init__(full, 1, rank, size)
        self.group = group

    def forward(self, x):
        if x.is_cuda and x.dim() == 2 and x.shape[0] % dist.get_world_size(self.group) == 0:
            from .symm_tp import LinearReduceScatter
            R = dist.get_world_size(self.group)
            comm = _comm_for(self.group, x.shape[0] // R, self.weight.shape[0], x)
            if comm is not None:
                return LinearReduceScatter.apply(comm, x, self.weight)
        return reduce_scatter_along(super().forward(x), self.group)


def _comm_for(group, chunk_rows: int, cols: int, like: torch.Tensor):
    """Fused communicator of the group when a `[chunk_rows, cols]` bf16 chunk fits its arena (created on first use
    with that shape), else None."""
    if not like.is_cuda or like.dtype != torch.bfloat16:
        return None
    from .symm_tp import fused_tp_comm
    return fused_tp_comm(group, torch.empty((chunk_rows, cols), dtype=like.dtype, device="meta"), like.device)


class ShardedRows:
    """Handle for `[T/R, D]` rows whose gather is deferred into the first column-parallel GEMM that consumes them."""

    def __init__(self, comm, x_shard):
        self.comm, self.x_shard = comm, x_shard

    def linears(self, *weights):
        from .symm_tp import GatherLinears
        return GatherLinears.apply(self.comm, self.x_shard, *weights)


class GatherSequenceFirst(nn.Module):
    """Boundary in front of a module that needs complete rows: gathers its first argument over the TP group."""

    def __init__(self, inner: nn.Module, group):
        super().__init__()
        self.inner, self.group = inner, group

    def forward(self, x, *args, **kw):
        if getattr(self.inner, "accepts_sharded_rows", False) and not getattr(self.inner, "fused_qkv", False) and x.dim() == 2:
            comm = _comm_for(self.group, x.shape[0], x.shape[1], x)
            if comm is not None:
                return self.inner(ShardedRows(comm, x), *args, **kw)
        return self.inner(all_gather_along(x, self.group), *args, **kw)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("inner"), name)


class TPMoeSequenceBoundary(nn.Module):
    """all-gather in, MoE with intermediate-sharded experts (partial sums), reduce-scatter out."""

    def __init__(self, inner: nn.Module, group):
        super().__init__()
        self.inner, self.group = inner, group

    def forward(self, x):
        if x.dim() == 2 and os.environ.get("LLMT_PEER_TP_MOE", "1") == "1":
            comm = _comm_for(self.group, x.shape[0], x.shape[1], x)
            if comm is not None and x.shape[1] % 8 == 0 and (x.shape[0] * x.shape[1]) % 8 == 0:
                from .symm_tp import PeerAllGatherRows, PeerReduceScatterRows
                return PeerReduceScatterRows.apply(comm, self.inner(PeerAllGatherRows.apply(comm, x)))
        return reduce_scatter_along(self.inner(all_gather_along(x, self.group)), self.group)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("inner"), name)


class VocabParallelEmbedding(nn.Module):
    """Rows [start, end) of the table live here. ids arrive sequence-sharded; they are gathered, looked up where
    local (zero elsewhere) and the partial rows are reduce-scattered back to the token shard."""

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
        self.group, self.rank, self.size = group, rank, size

    def forward(self, ids_local: torch.Tensor) -> torch.Tensor:
        from .vocab_parallel import _EmbedScatter, vocab_exchange
        R = self.size
        ids = torch.empty(ids_local.shape[0] * R, dtype=ids_local.dtype, device=ids_local.device)
        dist.all_gather_into_tensor(ids, ids_local.contiguous(), group=self.group)
        ex = None
        w = self.weight
        if w.is_cuda and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and ids.shape[0] % R == 0 and \
                os.environ.get("LLMT_DISABLE_FUSED_TP") != "1":
            ex = vocab_exchange(self.group, w.device, ids.shape[0], w.shape[1])
        return _EmbedScatter.apply(w, ids, self, ex)


# ---------------------------------------------------------------------------------------------- plan + apply
DEFAULT_PLAN = {
    "self_attn.q_proj": "colwise", "self_attn.k_proj": "colwise", "self_attn.v_proj": "colwise", "self_attn.o_proj": "rowwise",
    "mlp.gate_proj": "colwise", "mlp.up_proj": "colwise", "mlp.down_proj": "rowwise",
}


def resolve_tp_plan(model, tp_config) -> dict[str, str]:
    """Model default plan overridden by the user's colwise / rowwise module patterns (first match wins)."""
    plan = dict(model.tp_config()) if hasattr(model, "tp_config") else dict(DEFAULT_PLAN)
    for pat in tp_config.tp_colwise_modules:
        plan[pat] = "colwise"
    for pat in tp_config.tp_rowwise_modules:
        plan[pat] = "rowwise"
    return plan


def _shard_experts(experts, rank: int, size: int) -> None:
    """Packed experts: gate/up `(E, F, D)` split on F, down `(E, D, F)` split on F."""
    F_ = experts.w1_EFD.shape[1]
    if F_ % size:
        raise UnsupportedCombinationError(f"tensor_parallel_size {size} does not divide moe_intermediate_size {F_}")
    s = F_ // size
    for name, dim in (("w1_EFD", 1), ("w3_EFD", 1), ("w2_EDF", 2)):
        p = getattr(experts, name)
        if p.is_meta:
            shp = list(p.shape)
            shp[dim] = s
            new = nn.Parameter(torch.empty(shp, dtype=p.dtype, device="meta"), requires_grad=p.requires_grad)
        else:
            new = nn.Parameter(p.detach().narrow(dim, rank * s, s).clone(), requires_grad=p.requires_grad)
        new.is_expert = True
        new.tp_shard_dim, new.tp_full_shape = dim, tuple(p.shape)
        setattr(experts, name, new)
    experts.inter = s


def build_tp_plan(model, topo, tp_config):
    """Resolve, without touching the model, what `apply_tp` will do: every projection with its cut, every MoE block, the
    embedding and the head. Configuration errors (a head count the degree does not divide, tied embeddings, a fused QKV
    projection, sequence parallelism switched off) surface here, before any stage has mutated anything."""
    from ..models.contracts import BoundDecoder
    from ..models.moe import MoE
    from .plan import ParallelPlan, PlanTarget
    size = topo.tp
    if not tp_config.enable_sequence_parallel:
        raise ConfigError("tensor parallelism is sequence-parallel here: enable_sequence_parallel must stay True")
    bound = BoundDecoder(model.decoder_structure, model)
    st = model.decoder_structure
    targets = []
    for key, block in bound.block_items():
        base = f"{st.blocks}.{key}"
        attn = bound.attention_of(block)
        if getattr(attn, "fused_qkv", False):
            raise UnsupportedCombinationError("fused QKV projection cannot be column-sharded per projection")
        cut = getattr(attn, "tp_cut", None) or {"colwise": ("q_proj", "k_proj", "v_proj"), "rowwise": ("o_proj",),
                                                 "heads": ("num_heads", "num_kv_heads")}
        for name in cut["heads"]:
            if getattr(attn, name) % size:
                raise UnsupportedCombinationError(f"tensor_parallel_size {size} does not divide {type(attn).__name__}.{name} = {getattr(attn, name)}")
        targets.append(PlanTarget(f"{base}.{st.attention}", "attention", "sequence-gather", attn))
        for name in cut["colwise"]:
            if getattr(attn, name, None) is not None:
                targets.append(PlanTarget(f"{base}.{st.attention}.{name}", "dense", "colwise", getattr(attn, name)))
        for name in cut["rowwise"]:
            targets.append(PlanTarget(f"{base}.{st.attention}.{name}", "dense", "rowwise", getattr(attn, name)))
        mlp = bound.mlp_of(block)
        if isinstance(mlp, MoE):
            F_ = mlp.routed.experts.w1_EFD.shape[1]
            if F_ % size:
                raise UnsupportedCombinationError(f"tensor_parallel_size {size} does not divide moe_intermediate_size {F_}")
            targets.append(PlanTarget(f"{base}.{st.mlp}", "moe", "expert-intermediate", mlp))
        else:
            for name, lay in (("gate_proj", "colwise"), ("up_proj", "colwise"), ("down_proj", "rowwise")):
                targets.append(PlanTarget(f"{base}.{st.mlp}.{name}", "dense", lay, getattr(mlp, name)))
    if bound.tied_embeddings():
        raise UnsupportedCombinationError("tied embeddings with tensor parallelism are not supported (embedding and head are cut separately)")
    targets.append(PlanTarget(st.embedding, "vocab", "vocab", bound.embedding))
    head_layout = "vocab" if getattr(tp_config, "tp_vocab_parallel_head", True) else "replicated"
    targets.append(PlanTarget(st.head, "head", head_layout, bound.head))
    impl = "peer-memory" if os.environ.get("LLMT_DISABLE_FUSED_TP") != "1" else "torch.distributed"
    return ParallelPlan("tp", size, impl, tuple(targets), binds=("modules", "parameters", "forwards"))


def apply_tp(model, topo, tp_config) -> dict:
    """Swap the planned linears for their sharded forms, install the sequence boundaries and the vocab-parallel
    embedding, and mark every parameter that stays replicated so that its gradient is summed over the TP group."""
    from ..models.contracts import BoundDecoder
    from ..models.moe import MoE
    group, rank, size = topo.get_group("tp"), topo.coord("tp"), topo.tp
    if group is None:
        raise ConfigError("tensor parallelism needs an initialised process group")
    if not tp_config.enable_sequence_parallel:
        raise ConfigError("tensor parallelism is sequence-parallel here: enable_sequence_parallel must stay True")
    plan = resolve_tp_plan(model, tp_config)
    bound = BoundDecoder(model.decoder_structure, model)
    applied = {}
    for key, block in bound.block_items():
        attn = bound.attention_of(block)
        if getattr(attn, "fused_qkv", False):
            raise UnsupportedCombinationError("fused QKV projection cannot be column-sharded per projection")
        # the mixer names its own cut: projections split by heads (column shards), the output projection (input shard)
        # and the head counters that shrink with it; the default is the q/k/v/o layout of softmax attention
        cut = getattr(attn, "tp_cut", None) or {"colwise": ("q_proj", "k_proj", "v_proj"), "rowwise": ("o_proj",),
                                                 "heads": ("num_heads", "num_kv_heads")}
        for name in cut["colwise"]:
            if getattr(attn, name, None) is None:
                continue
            setattr(attn, name, ColwiseLinearNoGather(getattr(attn, name), rank, size))
            applied[f"layers.{key}.self_attn.{name}"] = "colwise"
        for name in cut["rowwise"]:
            setattr(attn, name, RowParallelLinear(getattr(attn, name), rank, size, group))
            applied[f"layers.{key}.self_attn.{name}"] = "rowwise"
        for name in cut["heads"]:
            if getattr(attn, name) % size:
                raise UnsupportedCombinationError(f"tensor_parallel_size {size} does not divide {type(attn).__name__}.{name} = {getattr(attn, name)}")
            setattr(attn, name, getattr(attn, name) // size)
        setattr(block, model.decoder_structure.attention, GatherSequenceFirst(attn, group))
        mlp = bound.mlp_of(block)
        if isinstance(mlp, MoE):
            _shard_experts(mlp.routed.experts, rank, size)
            if mlp.shared_experts is not None:
                se = mlp.shared_experts
                se.gate_proj = ColwiseLinearNoGather(se.gate_proj, rank, size)
                se.up_proj = ColwiseLinearNoGather(se.up_proj, rank, size)
                se.down_proj = ShardedLinear(se.down_proj, 1, rank, size)
            setattr(block, model.decoder_structure.mlp, TPMoeSequenceBoundary(mlp, group))
            applied[f"layers.{key}.mlp"] = "moe"
        else:
            mlp.gate_proj = ColwiseLinearNoGather(mlp.gate_proj, rank, size)
            mlp.up_proj = ColwiseLinearNoGather(mlp.up_proj, rank, size)
            mlp.down_proj = RowParallelLinear(mlp.down_proj, rank, size, group)
            setattr(block, model.decoder_structure.mlp, GatherSequenceFirst(mlp, group))
            applied[f"layers.{key}.mlp"] = "gated"
    # vocab-parallel embedding; tied heads would need the same cut of the head, which the replicated head forbids
    if bound.tied_embeddings():
        raise UnsupportedCombinationError("tied embeddings with tensor parallelism are not supported (the head stays replicated)")
    emb_path = model.decoder_structure.embedding.split(".")
    parent = model
    for part in emb_path[:-1]:
        parent = getattr(parent, part)
    setattr(parent, emb_path[-1], VocabParallelEmbedding(bound.embedding, rank, size, group))
    applied["embedding"] = "vocab"
    if getattr(tp_config, "tp_vocab_parallel_head", True):
        from .vocab_parallel import VocabParallelHead
        head_path = model.decoder_structure.head.split(".")
        parent = model
        for part in head_path[:-1]:
            parent = getattr(parent, part)
        setattr(parent, head_path[-1], VocabParallelHead(getattr(parent, head_path[-1]), rank, size, group))
        applied["head"] = "vocab"
    for _, p in model.named_parameters():
        if not hasattr(p, "tp_shard_dim"):
            p.tp_replicated = True
    model.tp_group, model.tp_size, model.tp_rank = group, size, rank
    return applied


@torch.no_grad()
def allreduce_replicated_tp_grads(params, group) -> None:
    """Sum over the TP group the gradient views of parameters that every TP rank holds in full (one coalesced call)."""
    views = [p._grad_view for p in params if getattr(p, "tp_replicated", False) and hasattr(p, "_grad_view")]
    if not views or group is None:
        return
    flat = torch.cat([v.reshape(-1).float() for v in views])
    dist.all_reduce(flat, group=group)
    off = 0
    for v in views:
        n = v.numel()
        v.copy_(flat[off:off + n].view_as(v))
        off += n
