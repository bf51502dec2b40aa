"""Assembly of the training runtime from a config (reference: llmtuner/trainer/runtime/assembly.py:86-642)."""
from __future__ import annotations

import zlib

import torch

from ...components.loss import LossFunctions
from ...components.optimizer import EMA, GradientClipper, build_lr_scheduler, build_optimizers
from ...models.registry import build_registered_model
from ...parallel.parallelize import parallelize_model
from ...memory.materialization import materialize_meta_model
from .engine import TrainingEngine


def build_model(config, env):
    """Build on the meta device when asked (large models) or on CPU (tests, reference comparisons)."""
    dev = "meta" if config.model.initialization_device == "meta" else ("cpu" if config.model.initialization_device == "cpu" else env.device)
    with torch.device(dev):
        model = build_registered_model(config.model, dtype=env.param_dtype, device=None)
    if dev != "meta":
        model.initialize_parameters(seed=config.training.seed)
    return model


def make_init_fn(model, seed: int):
    """Per-parameter initialiser used while the flat units materialise meta parameters in place."""
    std = getattr(model.config, "initializer_range", 0.02)

    def init(fqn: str, p: torch.Tensor) -> None:
        if fqn.endswith("norm.weight") or "layernorm" in fqn:
            p.fill_(1.0)
        else:
            g = torch.Generator(device=p.device).manual_seed(seed * 1000003 + zlib.crc32(fqn.encode()))
            p.normal_(0.0, std, generator=g)
    return init


def prepare_parallel_model(config, env):
    model = build_model(config, env)
    init_fn = make_init_fn(model, config.training.seed) if config.model.initialization_device == "meta" else None
    asm = parallelize_model(model, config, env.topo, device=env.device, param_dtype=env.param_dtype, init_fn=init_fn)
    materialize_meta_model(model, env.device)
    for m in model.modules():          # persistent fp32 buffers stay fp32 on the compute device
        for name, buf in list(m._buffers.items()):
            if buf is not None and buf.device != env.device:
                m._buffers[name] = buf.to(env.device)
    if asm.layout is not None:         # materialisation may have swapped parameter objects: paths, order and sharing must survive
        asm.layout.refresh(model)
        asm.layout.validate(model)
    return model, asm


def build_loss_functions(config, env, asm) -> LossFunctions:
    """The loss service follows the resolved execution layout: hidden-state path with the layout's chunk count, and, when
    the head is vocabulary-sharded over the tensor-parallel group, the sharded head module whose loss kernel exchanges
    per-token statistics over that group."""
    from ...parallel.vocab_parallel import VocabParallelHead
    layout = asm.execution
    head = None
    if layout is not None and layout.vocabulary_sharded:
        cand = asm.model
        for part in asm.model.decoder_structure.head.split("."):
            cand = getattr(cand, part)
        if not isinstance(cand, VocabParallelHead):
            raise RuntimeError("execution layout says the head is vocabulary-sharded but the tensor-parallel stage left "
                               f"{type(cand).__name__} in place")
        head = cand
    chunks = layout.loss_chunks if layout is not None and layout.output_kind == "hidden" else config.training.chunked_loss_num_chunks
    return LossFunctions(num_chunks=chunks, head=head)


def build_optimizer_stack(config, env, asm):
    optimizers = build_optimizers([asm.fsdp], config.optimizer, host_state=config.parallel.fsdp_config.fsdp_cpu_offload)
    lr = build_lr_scheduler(optimizers, config.optimizer.lr_scheduler_config, config.training.steps)
    ema = EMA([asm.fsdp], config.training.ema_config, config.training.steps, model=asm.model) if config.training.ema_config is not None else None
    clipper = GradientClipper([asm.fsdp], env.topo, config.training.max_norm, env.device)
    if asm.layout is not None:
        # the state consumers remember the layout they were built against; the checkpointer checks it before every save/load
        asm.layout.validate(asm.model)
        optimizers.layout_snapshot = asm.layout.snapshot()
        if ema is not None:
            ema.layout_snapshot = optimizers.layout_snapshot
    return optimizers, lr, ema, clipper


def create_training_engine(config, env, model, asm, loss_fns, optimizers, lr, ema, clipper) -> TrainingEngine:
    return TrainingEngine(model, asm, loss_fns, optimizers, lr, ema, clipper, env.topo, env.device)
