"""Native parameter sharding (ZeRO-3 / FSDP semantics) with an explicit gather / recompute / reduce schedule
(reference: llmtuner/parallel/fully_shard_parallel/fully_shard_parallel.py:61-784, policies.py:30-161).

Every parameter belongs to one `FlatUnit`: the embedding, each decoder block, the final norm + head (tied
embeddings put embedding and head in one unit), and, under expert parallelism, each block's expert weights (sharded
over the `efsdp` group instead of `dp_shard_cp`). A unit owns
  * one flat low-precision shard (bf16 on CUDA) that the optimizer rewrites and peers read,
  * the fp32 master shard and the fp32 gradient shard,
  * a slot of a small pool of full-size gather buffers that the unit's parameters are views of, and a full-size
    gradient buffer that GEMM wgrads accumulate into directly (`param.main_grad`).
The runtime owns the schedule: unit i+1 is gathered on the communication stream while unit i computes, the
gradient of unit i is reduce-scattered while unit i-1 runs backward, and with full activation checkpointing the
block forward is replayed inside the backward of a custom autograd function, so nothing but the block input is
saved. Gradient division is disabled: the loss is already divided by the global token count.

Two data paths implement the same schedule: NCCL collectives (`implementation="custom"` and every CPU/gloo run) and the
fused peer-memory kernels of `parallel/symm.py` (`implementation="native"` on CUDA with peer access).
"""
from __future__ import annotations

import re
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn

from ..errors import ConfigError

ALIGN = 128  # elements; keeps every shard 256-byte aligned in bf16


@dataclass
class ParamSlot:
    fqn: str
    shape: torch.Size
    numel: int
    offset: int


def _dtype(name: str) -> torch.dtype:
    return {"float32": torch.float32, "bfloat16": torch.bfloat16, "float64": torch.float64, "float16": torch.float16}[name]


class FlatUnit:
    def __init__(self, name: str, named_params, *, group, rank: int, world: int, device, param_dtype: torch.dtype,
                 reduce_dtype: torch.dtype, replicate_group=None, is_expert: bool = False):
        self.name, self.group, self.rank, self.world = name, group, rank, world
        self.device, self.param_dtype, self.reduce_dtype = device, param_dtype, reduce_dtype
        self.replicate_group, self.is_expert = replicate_group, is_expert
        self.params: list[nn.Parameter] = []
        self.slots: list[ParamSlot] = []
        off = 0
        for fqn, p in named_params:
            shape = getattr(p, "_meta_shape", p.shape)
            n = shape.numel()
            self.params.append(p)
            self.slots.append(ParamSlot(fqn, shape, n, off))
            off += -(-n // 8) * 8      # 16-byte aligned starts so every matrix is a legal TMA base
        self.numel = off
        quantum = world * ALIGN
        self.padded = max(quantum, -(-off // quantum) * quantum)
        self.shard_numel = self.padded // world
        self.separate_master = param_dtype != torch.float32
        self.shard_lowp = torch.zeros(self.shard_numel, dtype=param_dtype, device=device)
        self.master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device) if self.separate_master else self.shard_lowp
        self.grad_shard: torch.Tensor | None = None       # fp32 (world > 1) or a view of grad_full (world == 1)
        self.full: torch.Tensor | None = None              # bound gather buffer (views of the params)
        self.grad_full: torch.Tensor | None = None
        self.gathered = False
        self.gather_event = None
        self.free_event = None
        self.reduce_event = None
        self.has_grad = False
        self.needs_param_sync = True

    # ------------------------------------------------------------------ binding
    def bind_full(self, buf: torch.Tensor) -> None:
        """Make the parameters views of `buf` (length `padded`)."""
        self.full = buf
        for p, s in zip(self.params, self.slots):
            p.data = buf[s.offset:s.offset + s.numel].view(s.shape)

    def bind_grad(self, buf: torch.Tensor, use_main_grad: bool) -> None:
        self.grad_full = buf
        for p, s in zip(self.params, self.slots):
            view = buf[s.offset:s.offset + s.numel].view(s.shape)
            p._grad_view = view
            if use_main_grad and p.dim() == 2 and not getattr(p, "no_main_grad", False):
                p.main_grad = view
                p.main_grad_initialized = False

    def my_range(self) -> tuple[int, int]:
        return self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel

    @torch.no_grad()
    def adopt_full(self) -> None:
        """After the full buffer was initialised (or loaded): keep this rank's shard as the source of truth."""
        a, b = self.my_range()
        self.full[self.numel:].zero_()
        self.shard_lowp.copy_(self.full[a:b])
        if self.separate_master:
            self.master.copy_(self.full[a:b])

    @torch.no_grad()
    def adopt_master_from(self, full_fp32: torch.Tensor) -> None:
        a, b = self.my_range()
        self.master.copy_(full_fp32[a:b])
        if self.separate_master:
            self.shard_lowp.copy_(self.master)

    # ------------------------------------------------------------------ per-parameter views of shard state
    def shard_slices(self):
        """Yield (fqn, shape, lo, hi, shard_lo) for every parameter that intersects this rank's shard: elements
        [lo, hi) of the flattened parameter live at shard[shard_lo : shard_lo + hi - lo]."""
        a, b = self.my_range()
        for s in self.slots:
            lo, hi = max(a, s.offset), min(b, s.offset + s.numel)
            if hi > lo:
                yield s.fqn, s.shape, lo - s.offset, hi - s.offset, lo - a


class FSDPRuntime:
    """Schedule owner. `run_block` is installed as the model's `block_runner`."""

    def __init__(self, model: nn.Module, topo, fsdp_config, *, device, param_dtype, ac_mode: str = "none",
                 ac_save_every: int = 2, implementation: str | None = None):
        self.model, self.topo, self.cfg, self.device = model, topo, fsdp_config, device
        self.param_dtype = param_dtype
        self.reduce_dtype = _dtype(fsdp_config.fsdp_reduce_dtype)
        self.ac_mode, self.ac_save_every = ac_mode, ac_save_every
        self.grad_accum_steps = 1          # set by apply_fsdp from the training configuration
        self.named_units: dict = {}
        for name in ("fsdp_forward_prefetch_count", "fsdp_backward_prefetch_count"):
            if getattr(fsdp_config, name, 0) > 1:
                from ..errors import UnsupportedCombinationError
                raise UnsupportedCombinationError(f"{name} > 1: the runtime rotates two gather slots, so exactly one unit is "
                                                  "prefetched ahead of the one that computes (0 and 1 both select that)")
        self.is_cuda = torch.device(device).type == "cuda"
        self.group = topo.get_group("dp_shard_cp")
        self.world = topo.size("dp_shard_cp")
        self.rank = topo.coord("dp_shard_cp")
        self.replicate_group = topo.get_group("dp_replicate")
        self.implementation = implementation or fsdp_config.fsdp_implementation
        self.units: list[FlatUnit] = []
        self.block_units: dict[int, list[FlatUnit]] = {}
        self.unit_of_param: dict[int, FlatUnit] = {}
        self.reshard_after_forward = fsdp_config.fsdp_reshard_after_forward != "never"
        self.comm_stream = torch.cuda.Stream(device) if self.is_cuda else None
        self.is_last_microbatch = True
        self._slot_bufs: dict[tuple, list[torch.Tensor]] = {}
        self._grad_bufs: dict[tuple, list[torch.Tensor]] = {}
        self.fused = None         # set by parallel.symm when the peer-memory kernels are enabled
        self._gslot_event: dict = {}
        self._slot_owner: dict = {}

    # ------------------------------------------------------------------ construction
    def add_unit(self, name, named_params, *, expert: bool = False, replicated: bool = False,
                 block_index: int | None = None) -> FlatUnit | None:
        """`replicated`: the unit is not sharded at all (every rank keeps the whole flat buffer and steps it); its gradient is
        summed over the data ranks (`dp_cp`) before the optimizer, which is how parameters excluded from FSDP by
        `fsdp_ignored_modules` are kept in step (reference: llmtuner/trainer/runtime/gradients.py:50-83)."""
        named_params = [(n, p) for n, p in named_params if id(p) not in self.unit_of_param]
        seen, uniq = set(), []
        for n, p in named_params:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        if not uniq:
            return None
        if replicated:
            group, world, rank = None, 1, 0
        elif expert and self.topo.ep > 1:
            group, world, rank = self.topo.get_group("efsdp"), self.topo.efsdp, self.topo.coord("efsdp")
        else:
            group, world, rank = self.group, self.world, self.rank
        u = FlatUnit(name, uniq, group=group, rank=rank, world=world, device=self.device, param_dtype=self.param_dtype,
                     reduce_dtype=self.reduce_dtype, replicate_group=self.replicate_group, is_expert=expert)
        u.replicated_group = self.topo.get_group("dp_cp") if replicated else None
        u.is_replicated = replicated
        # Gather / gradient buffers rotate between two slots by block parity. Units of one block that have the same size
        # (two selected projections, say) would land in the same buffer, so each gets its own lane of the pool.
        u.slot_index = (block_index % 2) if block_index is not None else 0
        twins = [v for v in self.units if getattr(v, "block_index", None) == block_index and block_index is not None
                 and v.padded == u.padded and v.is_expert == u.is_expert]
        u.block_index, u.lane = block_index, len(twins)
        self.units.append(u)
        for _, p in uniq:
            self.unit_of_param[id(p)] = u
        return u

    def _pool(self, table, unit: FlatUnit, count: int, dtype) -> list[torch.Tensor]:
        key = (unit.padded, dtype, unit.is_expert, getattr(unit, "lane", 0))
        bufs = table.setdefault(key, [])
        while len(bufs) < count:
            bufs.append(torch.zeros(unit.padded, dtype=dtype, device=self.device))
        return bufs

    def finalize(self, init_fn=None, needs_init: set | None = None) -> None:
        """Bind gather/gradient buffers and establish the shards. Parameters that still hold real data (model
        built on CPU/GPU) are copied in; meta parameters are initialised by `init_fn(fqn, param)` inside the bound
        full buffer, unit by unit, so the peak is one unit."""
        use_main = self.is_cuda and self.param_dtype == torch.bfloat16
        for u in self.units:
            # units that no decoder block owns (embedding, head, leftovers such as a stream-collapsing head) are not part of
            # the per-block gather schedule: their full copy stays resident and is refreshed after every optimizer step
            persistent = u.world == 1 or not self.reshard_after_forward or getattr(u, "block_index", None) is None
            if u.world == 1:
                full = u.shard_lowp
            elif persistent:
                full = torch.zeros(u.padded, dtype=u.param_dtype, device=self.device)
            else:
                pool = self._pool(self._slot_bufs, u, 2, u.param_dtype)
                full = pool[self._unit_slot(u)]
            needs_init = needs_init or set()
            old = [(p, None if id(p) in needs_init else p.detach().clone()) for p in u.params]
            u.bind_full(full)
            u.persistent = persistent
            with torch.no_grad():
                for (p, data), s in zip(old, u.slots):
                    if data is not None:
                        p.copy_(data.to(p.dtype))
                    elif init_fn is not None:
                        init_fn(s.fqn, p)
            u.adopt_full()
            u.gathered = u.world == 1 or persistent
            u.needs_param_sync = u.world > 1 and persistent     # persistent full copies are refreshed after each step
            if u.world == 1:
                # one shard rank: the flat buffer itself accumulates over micro-batches, so with gradient accumulation (or
                # a cross-rank sum for a replicated unit) it is fp32 like the sharded path's reduce buffer
                wide = self.grad_accum_steps > 1 or getattr(u, "is_replicated", False)
                gbuf = torch.zeros(u.padded, dtype=torch.float32 if wide else u.param_dtype, device=self.device)
                u.grad_shard = gbuf
            else:
                gpool = self._pool(self._grad_bufs, u, 2, u.param_dtype) if not persistent else [torch.zeros(u.padded, dtype=u.param_dtype, device=self.device)]
                gbuf = gpool[self._unit_slot(u) % len(gpool)]
                u.grad_shard = torch.zeros(u.shard_numel, dtype=torch.float32, device=self.device)
            u.bind_grad(gbuf, use_main)

    def _unit_slot(self, u: FlatUnit) -> int:
        return getattr(u, "slot_index", 0)

    # ------------------------------------------------------------------ collectives (NCCL / gloo arm)
    def _on_comm(self):
        if self.comm_stream is None:
            import contextlib
            return contextlib.nullcontext()
        return torch.cuda.stream(self.comm_stream)

    def unshard(self, u: FlatUnit, wait: bool = True) -> None:
        if u.world == 1:
            return
        if not u.gathered:
            if not getattr(u, "persistent", False):
                key = (u.padded, u.is_expert, self._unit_slot(u), getattr(u, "lane", 0))
                prev = self._slot_owner.get(key)
                if prev is not None and prev is not u:
                    prev.gathered = False
                self._slot_owner[key] = u
            if self.fused is not None and self.fused.supports(u):
                self.fused.all_gather(u)       # queued; carried by the GEMMs launched from here on
            else:
                if self.comm_stream is not None:
                    self.comm_stream.wait_stream(torch.cuda.current_stream())
                with self._on_comm():
                    dist.all_gather_into_tensor(u.full, u.shard_lowp, group=u.group)
                    if self.comm_stream is not None:
                        u.gather_event = self.comm_stream.record_event()
            u.gathered = True
        if wait and self.fused is not None and self.fused.supports(u):
            self.fused.wait_gather(u)          # finish what no GEMM carried
        if wait and u.gather_event is not None:
            torch.cuda.current_stream().wait_event(u.gather_event)
            u.gather_event = None

    def reshard(self, u: FlatUnit) -> None:
        if u.world == 1 or getattr(u, "persistent", False):
            return
        u.gathered = False

    def reduce_grads(self, u: FlatUnit) -> None:
        """Fold parameter `.grad`s into the flat gradient buffer, then reduce-scatter into the fp32 shard.
        With one shard rank the flat buffer itself accumulates over micro-batches; with several it holds one
        micro-batch and the fp32 shard accumulates."""
        accum_in_full = u.world == 1 and u.has_grad
        with torch.no_grad():
            for p in u.params:
                if p.grad is not None:
                    if accum_in_full:
                        p._grad_view.add_(p.grad.to(p._grad_view.dtype))
                    else:
                        p._grad_view.copy_(p.grad)
                    p.grad = None
                elif not accum_in_full and not getattr(p, "main_grad_initialized", False):
                    p._grad_view.zero_()
        if self.topo.tp > 1 and (u.world > 1 or self.is_last_microbatch):
            # parameters that every TP rank holds in full carry partial gradients: sum them over the TP group
            from .tensor_parallel import allreduce_replicated_tp_grads
            allreduce_replicated_tp_grads(u.params, self.topo.get_group("tp"))
        if u.world == 1:
            u.has_grad = True
            for p in u.params:
                if hasattr(p, "main_grad"):
                    p.main_grad_initialized = True
            return
        if self.fused is not None and self.fused.supports(u):
            self.fused.reduce_scatter(u, accumulate=u.has_grad)
        else:
            if self.comm_stream is not None:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
            with self._on_comm():
                src = u.grad_full if u.grad_full.dtype == u.reduce_dtype else u.grad_full.to(u.reduce_dtype)
                out = torch.empty(u.shard_numel, dtype=u.reduce_dtype, device=self.device)
                dist.reduce_scatter_tensor(out, src, op=dist.ReduceOp.SUM, group=u.group)
                if u.has_grad:
                    u.grad_shard.add_(out)
                else:
                    u.grad_shard.copy_(out)
                if self.comm_stream is not None:
                    self._gslot_event[self._gslot_key(u)] = self.comm_stream.record_event()
        u.has_grad = True
        for p in u.params:
            if hasattr(p, "main_grad"):
                p.main_grad_initialized = False      # the flat buffer is reused by the next unit of this slot

    def _gslot_key(self, u: FlatUnit):
        return (u.padded, u.is_expert, self._unit_slot(u), getattr(u, "lane", 0), getattr(u, "persistent", False) and u.name)

    def before_block_backward(self, i: int) -> None:
        """The gradient slot about to be written may still be read by an earlier reduce-scatter."""
        if self.fused is not None:
            for u in self._units(i):
                if self.fused.supports(u):
                    self.fused.before_grad_write(u)
        if self.comm_stream is None:
            return
        for u in self._units(i):
            ev = self._gslot_event.pop(self._gslot_key(u), None)
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)

    def before_forward(self) -> None:
        """Wait for the refresh of persistently gathered units (embedding, head) issued after the last step."""
        for u in self.units:               # whatever the forward touches before its first block; the head is waited for later
            if id(u) not in self._block_owned() and u.name != "head":
                self.wait_param_update(u)
        for u in self.units:                # the head's refresh keeps running under the forward; the last block waits for it
            if getattr(u, "persistent", False) and u.world > 1 and not (u.name == "head" and self.block_units):
                self.unshard(u)

    def finish_backward(self) -> None:
        """Reduce the units that no block owns (embedding, head, leftovers) once backward is over."""
        owned = {id(u) for us in self.block_units.values() for u in us}
        for u in self.units:
            if id(u) not in owned:
                self.reduce_grads(u)

    def wait_reductions(self) -> None:
        """Make the compute stream see every reduce-scattered gradient (called before clipping / the optimizer)."""
        if self.fused is not None:
            self.fused.flush_all()
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self.replicate_group is not None and self.is_last_microbatch:
            for u in self.units:
                if u.has_grad and not getattr(u, "is_replicated", False):
                    dist.all_reduce(u.grad_shard, group=self.replicate_group)
        if self.is_last_microbatch:
            for u in self.units:
                if getattr(u, "replicated_group", None) is not None and u.has_grad:
                    dist.all_reduce(u.grad_shard, group=u.replicated_group)

    def post_optimizer(self) -> None:
        """After the optimizer rewrote the shards: zero gradient state, refresh persistent full copies."""
        if self.fused is not None:
            self.fused.step_barrier()
        for u in self.units:
            u.has_grad = False
            for p in u.params:
                if hasattr(p, "main_grad"):
                    p.main_grad_initialized = False
            if u.world > 1 and getattr(u, "persistent", False):
                u.gathered = False
                self.unshard(u, wait=False)

    # ------------------------------------------------------------------ schedule
    def _units(self, i: int) -> list[FlatUnit]:
        return self.block_units.get(i, [])

    def _prefetch(self, i: int) -> None:
        for u in self._units(i):
            self.unshard(u, wait=False)

    def _recomputes(self, i: int) -> bool:
        """Selective modes: the per-block mask of the region mode wins, else every `ac_save_every`-th block keeps its
        activations."""
        mask = getattr(self.model, "ac_block_mask", None)
        if mask is not None and i < len(mask):
            return bool(mask[i])
        return i % self.ac_save_every != 0

    # ------------------------------------------------------------------ optimizer updates that overlap the next forward
    def wait_param_update(self, u: FlatUnit) -> None:
        """The optimizer may still be rewriting this unit on its own stream (see `ShardedAdamW.step`): the first use of the
        unit's parameters in the next forward waits for exactly that unit's update."""
        ev = getattr(u, "updated_event", None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            u.updated_event = None

    def sync_optimizer(self) -> None:
        """Everything that reads masters, moments or parameters outside the forward path (EMA, checkpoints, exports, a
        caller inspecting the model) first lets every pending update finish."""
        for u in self.units:
            self.wait_param_update(u)

    def _block_owned(self) -> set:
        owned = getattr(self, "_owned_ids", None)
        if owned is None:
            owned = self._owned_ids = {id(u) for us in self.block_units.values() for u in us}
        return owned

    def run_block(self, i: int, layer: nn.Module, x: torch.Tensor, ctx) -> torch.Tensor:
        for u in self._units(i):
            self.wait_param_update(u)
        if self.block_units and i == max(self.block_units):       # head, final norm: updated last, needed after the last block
            for u in self.units:
                if id(u) not in self._block_owned():
                    self.wait_param_update(u)
                    if u.name == "head" and getattr(u, "persistent", False) and u.world > 1:
                        self.unshard(u)
        grad_mode = self.model.training and torch.is_grad_enabled()
        per_op = self.ac_mode == "selective" and getattr(self.model, "ac_per_op", False)
        ac = grad_mode and (self.ac_mode == "full" or per_op or (self.ac_mode == "selective" and self._recomputes(i)))
        if ac:
            return _CheckpointedBlock.apply(x, self, i, layer, ctx, per_op)
        for u in self._units(i):
            self.unshard(u)
        self._prefetch(i + 1)
        if grad_mode:
            x = _PostBackward.apply(x, self, i)
        out = layer(x, ctx)
        if grad_mode:
            out = _PreBackward.apply(out, self, i)
        if not grad_mode:
            for u in self._units(i):
                self.reshard(u)
        return out



class _PreBackward(torch.autograd.Function):
    """Identity in forward; in backward (which runs first for the block) gathers the block and prefetches i-1."""

    @staticmethod
    def forward(ctx, x, rt: FSDPRuntime, i: int):
        ctx.rt, ctx.i = rt, i
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        rt, i = ctx.rt, ctx.i
        for u in rt._units(i):
            rt.unshard(u)
        rt._prefetch(i - 1)
        rt.before_block_backward(i)
        return g, None, None


class _PostBackward(torch.autograd.Function):
    """Identity in forward; in backward (which runs last for the block) reduces the block's gradients."""

    @staticmethod
    def forward(ctx, x, rt: FSDPRuntime, i: int):
        ctx.rt, ctx.i = rt, i
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        rt, i = ctx.rt, ctx.i
        for u in rt._units(i):
            rt.reduce_grads(u)
            rt.reshard(u)
        return g, None, None


class _CheckpointedBlock(torch.autograd.Function):
    """Full activation checkpointing owned by the shard schedule: forward keeps only the block input; backward
    gathers the block, replays its forward with autograd on, runs its backward, and hands the gradients to the
    reduce-scatter."""

    @staticmethod
    def forward(ctx, x, rt: FSDPRuntime, i: int, layer, fctx, per_op: bool = False):
        from ..ops.functional import SelectiveReplay, sac_frame
        ctx.rt, ctx.i, ctx.layer, ctx.fctx = rt, i, layer, fctx
        # per-op policy: attention and every other linear keep their outputs, the replay only rebuilds their graph nodes
        ctx.frame = SelectiveReplay(getattr(rt.model, "ac_recompute_mm_shapes", ())) if per_op else None
        for u in rt._units(i):
            rt.unshard(u)
        rt._prefetch(i + 1)
        with torch.no_grad(), sac_frame(ctx.frame, "record"):
            out = layer(x, fctx)
        for u in rt._units(i):
            rt.reshard(u)
        ctx.save_for_backward(x)
        return out

    @staticmethod
    def backward(ctx, dy):
        rt, i = ctx.rt, ctx.i
        (x,) = ctx.saved_tensors
        for u in rt._units(i):
            rt.unshard(u)
        rt._prefetch(i - 1)
        rt.before_block_backward(i)
        xd = x.detach().requires_grad_(True)
        from ..ops.functional import sac_frame
        with torch.enable_grad(), sac_frame(ctx.frame, "replay"):
            out = ctx.layer(xd, ctx.fctx)
        if ctx.frame is not None:
            ctx.frame.store.clear()
        # Auxiliary (load-balance) losses of MoE blocks: the value that entered the step's loss came from the first,
        # graph-free forward, so their gradient is injected here, from the replayed forward. They are token sums, and
        # d loss / d aux is the step's 1 / global_valid_tokens (`aux_grad_scale`, set by the engine per micro-batch).
        aux = [m.aux_loss for m in ctx.layer.modules() if getattr(m, "aux_loss", None) is not None and m.aux_loss.requires_grad]
        if aux:
            total_aux = aux[0] if len(aux) == 1 else torch.stack(aux).sum()
            scale = getattr(rt, "aux_grad_scale", None)
            seed = torch.ones_like(total_aux) if scale is None else torch.as_tensor(scale, dtype=total_aux.dtype, device=total_aux.device).reshape(total_aux.shape)
            torch.autograd.backward([out, total_aux], [dy, seed])
        else:
            torch.autograd.backward(out, dy)
        for u in rt._units(i):
            rt.reduce_grads(u)
            rt.reshard(u)
        return xd.grad, None, None, None, None, None


def _materialize_meta_params(model: nn.Module, device, dtype) -> set[int]:
    """Replace every meta parameter by an empty parameter on `device` (same object for tied weights) so that the
    units can bind views with `.data =`. Returns the ids of the new parameters: they still need initial values."""
    fresh: dict[int, nn.Parameter] = {}
    for mod in model.modules():
        for name, p in list(mod._parameters.items()):
            if p is None or not p.is_meta:
                continue
            if id(p) not in fresh:
                q = nn.Parameter(torch.empty(0, dtype=dtype, device=device), requires_grad=p.requires_grad)
                for k, v in p.__dict__.items():
                    setattr(q, k, v)
                q._meta_shape = p.shape
                fresh[id(p)] = q
            mod._parameters[name] = fresh[id(p)]
    return {id(q) for q in fresh.values()}


# ---------------------------------------------------------------------------------------------- stage entry
def apply_fsdp(model: nn.Module, topo, fsdp_config, *, device, param_dtype, ac_mode="none", ac_save_every=2,
               init_fn=None, grad_accum_steps: int = 1) -> FSDPRuntime:
    """Build the units in forward order (embedding, blocks, [experts], norm + head), bind buffers, install the
    block runner. Works for any shard degree, including 1 (then gather/reduce are no-ops and the same flat
    buffers serve the fused optimizer)."""
    from ..models.contracts import BoundDecoder
    structure = getattr(model, "decoder_structure", None)
    if structure is None:
        raise ConfigError(f"{type(model).__name__} exposes no decoder_structure; cannot place FSDP units")
    needs_init = _materialize_meta_params(model, device, param_dtype)
    bound = BoundDecoder(structure, model)
    rt = FSDPRuntime(model, topo, fsdp_config, device=device, param_dtype=param_dtype, ac_mode=ac_mode,
                     ac_save_every=ac_save_every)
    rt.grad_accum_steps = max(1, int(grad_accum_steps))
    ignored = [re.compile(p) for p in fsdp_config.fsdp_ignored_modules]
    skip = lambda fqn: any(r.search(fqn) for r in ignored)  # noqa: E731
    prefix_of = {id(m): n for n, m in model.named_modules()}

    def named(mod):
        base = prefix_of[id(mod)]
        return [(f"{base}.{n}" if base else n, p) for n, p in mod.named_parameters() if not skip(f"{base}.{n}")]

    # User-selected units (`fsdp_apply_modules`): every selected module becomes a unit of its own, made of the parameters
    # whose innermost selected ancestor it is. A unit gathers and reduces with the block it lives in, so a selection has
    # to sit inside a decoder block or beside the blocks (embedding, norm, head), not around several blocks.
    own_unit_of: dict[int, str] = {}
    if fsdp_config.fsdp_apply_modules:
        from ..errors import UnsupportedCombinationError
        from .module_patterns import resolve_module_patterns
        names = [n for n, _ in model.named_modules() if n]
        try:
            chosen = resolve_module_patterns(names, fsdp_config.fsdp_apply_modules, "fsdp_apply_modules")
        except ValueError as e:
            raise ConfigError(str(e)) from None
        block_names = {prefix_of[id(b)] for _, b in bound.block_items()}
        for c in chosen:
            if any(b != c and b.startswith(c + ".") for b in block_names):
                raise UnsupportedCombinationError(f"fsdp_apply_modules selects {c!r}, which contains whole decoder blocks: a "
                                                  "sharding unit is gathered with one block and cannot span several")
        for mod_name in sorted(chosen, key=len):            # innermost selection wins: longer names overwrite shorter ones
            mod = model.get_submodule(mod_name)
            for _, p in mod.named_parameters():
                own_unit_of[id(p)] = mod_name

    def split_selected(pairs):
        """(parameters left to the default unit, [(selected module name, its parameters)] in first-appearance order)"""
        rest, groups = [], {}
        for n, p in pairs:
            key = own_unit_of.get(id(p))
            if key is None or key in block_names_default:
                rest.append((n, p))
            else:
                groups.setdefault(key, []).append((n, p))
        return rest, list(groups.items())

    block_names_default = {prefix_of[id(b)] for _, b in bound.block_items()}      # selecting a block itself is the default
    tied = bound.tied_embeddings()
    named_units = {}
    if tied:
        named_units["root"] = rt.add_unit("root", named(bound.embedding) + named(bound.final_norm) + named(bound.head))
        named_units["embedding"] = named_units["head"] = named_units["root"]
    else:
        named_units["embedding"] = rt.add_unit("embedding", named(bound.embedding))
    for key, block in bound.block_items():
        i = getattr(block, "layer_idx", int(key))
        units = []
        exp = [(n, p) for n, p in named(block) if getattr(p, "is_expert", False)]
        dense = [(n, p) for n, p in named(block) if not getattr(p, "is_expert", False)]
        dense, selected = split_selected(dense)
        u = rt.add_unit(f"block{i}", dense, block_index=i)
        if u is not None:
            units.append(u)
        for mod_name, pairs in selected:
            us = rt.add_unit(f"block{i}.{mod_name}", pairs, block_index=i)
            if us is not None:
                units.append(us)
        if exp:
            ue = rt.add_unit(f"block{i}.experts", exp, expert=True, block_index=i)
            if ue is not None:
                units.append(ue)
        rt.block_units[i] = units
    if not tied:
        named_units["head"] = rt.add_unit("head", named(bound.final_norm) + named(bound.head))
    rest = [(n, p) for n, p in model.named_parameters() if id(p) not in rt.unit_of_param and not skip(n)]
    if rest:
        named_units["rest"] = rt.add_unit("rest", rest)
    # Parameters excluded from sharding stay whole on every rank: one replicated unit, gradient summed over the data ranks,
    # stepped by the optimizer like any other unit.
    kept = [(n, p) for n, p in model.named_parameters() if id(p) not in rt.unit_of_param and skip(n)]
    if kept:
        if any(getattr(p, "is_expert", False) for _, p in kept):
            from ..errors import UnsupportedCombinationError
            raise UnsupportedCombinationError("fsdp_ignored_modules may not name expert parameters: their gradient lives on "
                                              "the expert-parallel mesh, not on the data ranks")
        named_units["ignored"] = rt.add_unit("ignored", kept, replicated=True)
    rt.named_units = {k: v for k, v in named_units.items() if v is not None}
    rt.finalize(init_fn=init_fn, needs_init=needs_init)
    from .symm import enable_fused_fsdp
    enable_fused_fsdp(rt)
    model.block_runner = rt.run_block
    model.fsdp_runtime = rt
    return rt
