"""Fixed stage order of model parallelisation (reference: llmtuner/parallel/stages.py:33-71):
TP -> EP -> CP -> AC -> activation swap -> compile -> FSDP."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Stage:
    name: str
    description: str


STAGES = (
    Stage("tp", "tensor + sequence parallel linears, vocab-parallel embedding"),
    Stage("ep", "expert-parallel MoE blocks and token dispatchers"),
    Stage("cp", "context-parallel attention"),
    Stage("ac", "activation checkpointing"),
    Stage("activation_swap", "saved-activation offload to pinned host memory"),
    Stage("compile", "CUDA-graph capture of block launch sequences"),
    Stage("fsdp", "parameter sharding, gather/reduce schedule"),
)
STAGE_ORDER = tuple(s.name for s in STAGES)
