"""Structural contracts a model exposes to the parallel layer (reference: llmtuner/models/contracts.py:16-247).

`DecoderStructure` names where the decoder, embedding, blocks, final norm, head and attention modules live, so
that TP/EP/FSDP/AC stages address them without knowing the model class. `MoEBlockContract` names the parts of
a sparse block; `GatedMLPStructure` the three projections of a gated MLP.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch.nn as nn

from ..errors import ConfigError


def resolve_path(root: nn.Module, path: str):
    obj = root
    for part in path.split("."):
        if not part:
            continue
        if not hasattr(obj, part):
            raise ConfigError(f"module path {path!r} does not resolve on {type(root).__name__} (missing {part!r})")
        obj = getattr(obj, part)
    return obj


@dataclass(frozen=True)
class GatedMLPStructure:
    gate: str = "gate_proj"
    up: str = "up_proj"
    down: str = "down_proj"


@dataclass(frozen=True)
class MoEBlockContract:
    router: str = "gate"
    experts: str = "experts"
    shared_experts: str | None = None
    gate_weight: str = "w1_EFD"
    up_weight: str = "w3_EFD"
    down_weight: str = "w2_EDF"
    bias_buffer: str = "expert_bias_E"
    counts_buffer: str = "tokens_per_expert_E"


@dataclass(frozen=True)
class DecoderStructure:
    decoder: str = "model"
    embedding: str = "model.embed_tokens"
    blocks: str = "model.layers"
    final_norm: str = "model.norm"
    head: str = "lm_head"
    attention: str = "self_attn"
    mlp: str = "mlp"
    q_proj: str = "q_proj"
    k_proj: str = "k_proj"
    v_proj: str = "v_proj"
    o_proj: str = "o_proj"
    mlp_structure: GatedMLPStructure = field(default_factory=GatedMLPStructure)
    moe: MoEBlockContract = field(default_factory=MoEBlockContract)

    def bind(self, model: nn.Module) -> "BoundDecoder":
        return BoundDecoder(self, model)


class BoundDecoder:
    """A `DecoderStructure` resolved against a live model; raises `ConfigError` on stale paths."""

    def __init__(self, structure: DecoderStructure, model: nn.Module):
        self.structure, self.model = structure, model
        self.embedding = resolve_path(model, structure.embedding)
        self.blocks = resolve_path(model, structure.blocks)
        self.final_norm = resolve_path(model, structure.final_norm)
        self.head = resolve_path(model, structure.head)
        if not isinstance(self.blocks, (nn.ModuleList, nn.ModuleDict)):
            raise ConfigError(f"{structure.blocks!r} must be a ModuleList/ModuleDict of decoder blocks")

    def block_items(self):
        if isinstance(self.blocks, nn.ModuleDict):
            return list(self.blocks.items())
        return [(str(i), b) for i, b in enumerate(self.blocks)]

    def attention_of(self, block: nn.Module):
        return resolve_path(block, self.structure.attention)

    def mlp_of(self, block: nn.Module):
        return resolve_path(block, self.structure.mlp)

    def tied_embeddings(self) -> bool:
        hw = getattr(self.head, "weight", None)
        ew = getattr(self.embedding, "weight", None)
        return hw is not None and ew is not None and hw is ew
