"""`parallelize_model`: validate, resolve plans (metadata only), then apply the stages in the fixed order
TP -> EP -> CP -> AC -> activation swap -> compile -> FSDP (reference: llmtuner/parallel/parallelize.py:54-314)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..accelerator.collectives import synchronize_local_errors
from .compatibility import check_compatibility
from .stages import STAGE_ORDER


@dataclass
class ParallelAssembly:
    model: torch.nn.Module
    topo: object
    fsdp: object = None
    tp_plan: dict = field(default_factory=dict)
    ep_plan: dict = field(default_factory=dict)
    cp_driver: object = None
    stages_applied: list[str] = field(default_factory=list)
    plans: dict = field(default_factory=dict)          # stage -> ParallelPlan, resolved before any mutation
    execution: object = None                            # ExecutionLayout
    layout: object = None                               # ModelPartLayout of the assembled model


def parallelize_model(model, config, topo, *, device, param_dtype, init_fn=None) -> ParallelAssembly:
    arch = getattr(model, "config", None)
    check_compatibility(config, topo, arch)
    if hasattr(model, "validate_parallel"):
        model.validate_parallel(tp=topo.tp, cp_ulysses=topo.cp_ulysses, ep=topo.ep)
    asm = ParallelAssembly(model, topo)
    t = config.training
    # Resolve first, execute second: every stage's plan is computed against the untouched model (metadata only), so a
    # configuration error of a late stage surfaces before an early stage has rewritten anything.
    with synchronize_local_errors("parallelize:resolve"):
        if topo.tp > 1:
            from .tensor_parallel import build_tp_plan
            asm.plans["tp"] = build_tp_plan(model, topo, config.parallel.tp_config)
        if getattr(arch, "num_experts", 0) > 0 and topo.ep > 1:
            from .expert_parallel import build_ep_plan
            asm.plans["ep"] = build_ep_plan(model, topo, config.parallel.ep_config)
        if topo.cp > 1:
            from .context_parallel import build_cp_plan
            asm.plans["cp"] = build_cp_plan(model, topo, config.parallel.cp_config)
        from .execution import resolve_execution_layout
        asm.execution = resolve_execution_layout(config, topo, model, asm.plans)
    for stage in STAGE_ORDER:
        with synchronize_local_errors(f"parallelize:{stage}"):
            if stage in asm.plans:
                asm.plans[stage].validate_binding(model)      # the model may not have changed under the plan's targets
            if stage == "tp" and topo.tp > 1:
                from .tensor_parallel import apply_tp
                asm.tp_plan = apply_tp(model, topo, config.parallel.tp_config)
            elif stage == "ep" and getattr(arch, "num_experts", 0) > 0 and topo.ep > 1:
                from .expert_parallel import apply_ep
                asm.ep_plan = apply_ep(model, topo, config.parallel.ep_config)
            elif stage == "cp" and topo.cp > 1:
                from .context_parallel import apply_cp
                asm.cp_driver = apply_cp(model, topo, config.parallel.cp_config)
            elif stage == "ac":
                from ..memory.activation_checkpoint import apply_ac
                apply_ac(model, t)
            elif stage == "activation_swap" and t.activation_swap:
                from ..memory.activation_swap import apply_activation_swap
                apply_activation_swap(model, t)
            elif stage == "compile" and t.compile:
                from .graph_capture import apply_compile
                apply_compile(model, t.compile_config)
            elif stage == "fsdp":
                from .fsdp import apply_fsdp
                asm.fsdp = apply_fsdp(model, topo, config.parallel.fsdp_config, device=device, param_dtype=param_dtype,
                                      ac_mode=getattr(model, "activation_checkpoint", "none"),
                                      ac_save_every=getattr(model, "ac_save_every", 2), init_fn=init_fn,
                                      grad_accum_steps=t.gradient_accumulation_steps)
            else:
                continue
        asm.stages_applied.append(stage)
    # tokens one rank feeds to a MoE block per micro-batch: sizes the expert-parallel exchange before the first call
    try:
        from ..config.training_config import resolve_batch_size_per_rank
        rows = resolve_batch_size_per_rank(t.global_batch_size, topo.size("dp"), t.gradient_accumulation_steps)
        seq_split = topo.cp * (topo.tp if topo.ep > 1 else 1)
        max_tokens = -(-rows * t.max_seq_len // seq_split)
    except Exception:
        max_tokens = 0
    _bind_moe_stream_groups(model, topo, config.parallel.ep_config.router_aux_loss_coef, max_tokens)
    # The record optimizer, EMA and checkpointer bind to: final parameter objects under wrapper-free names.
    from .assembly import ModelPartLayout
    with synchronize_local_errors("parallelize:layout"):
        asm.layout = ModelPartLayout(execution=asm.execution, topology=topo.snapshot())
        asm.layout.refresh(model)
        asm.layout.validate(model)
    return asm


def _bind_moe_stream_groups(model, topo, aux_loss_coef=None, max_tokens: int = 0) -> None:
    """Tell every MoE block which process groups split ONE token stream: the context-parallel group always, the
    tensor-parallel group only when the experts are expert-parallel (the block then sees its sequence-parallel shard; under
    plain TP the block boundary has already gathered the whole stream and every TP rank holds identical statistics).
    Balance-loss statistics are summed over these groups (reference: llmtuner/models/common/moe/auxiliary_loss.py:131-140)."""
    from ..models.moe import moe_blocks
    groups = []
    if topo.cp > 1 and topo.get_group("cp") is not None:
        groups.append(topo.get_group("cp"))
    if topo.tp > 1 and topo.ep > 1 and topo.get_group("tp") is not None:
        groups.append(topo.get_group("tp"))
    for blk in moe_blocks(model):
        blk.stream_groups = tuple(groups)
        disp = getattr(blk.routed, "dispatcher", None)
        if max_tokens and hasattr(disp, "max_copies_hint"):
            disp.max_copies_hint = max_tokens * blk.top_k
        if aux_loss_coef is not None:            # the `router_aux_loss_coef` flag overrides the architecture's value
            blk.aux_loss_coef = float(aux_loss_coef)
            blk.router.need_scores = blk.aux_loss_coef > 0
