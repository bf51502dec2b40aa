"""Model registry (reference: llmtuner/models/registry.py:17-305).

`register_model(name, builder, ...)`, `get_model_spec`, `build_registered_model`. Built-ins: `qwen3` (dense alias),
`qwen3_moe`, `qwen3_8b`, `qwen3_30b_a3b`, and the capability-surface families `qwen3_5`, `qwen3_5_moe`,
`qwen3_5_moe_text`, `deepseek_v4`, `kimi_linear`, `kimi_k3` which are registered behind the same contracts.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable

from ..errors import ConfigError


@dataclass
class ModelSpec:
    name: str
    builder: Callable
    state_format: str = "native"            # name of the ModelStateFormat used for HF import/export
    supports: frozenset[str] = field(default_factory=lambda: frozenset({"fsdp", "tp", "ep", "cp", "pp", "ac"}))
    description: str = ""


_MODELS: dict[str, ModelSpec] = {}


def register_model(name: str, builder: Callable, *, state_format: str = "native", supports=None, description: str = "",
                   replace: bool = False) -> ModelSpec:
    if name in _MODELS and not replace:
        raise ConfigError(f"model {name!r} is already registered")
    spec = ModelSpec(name, builder, state_format, frozenset(supports) if supports is not None else ModelSpec.__dataclass_fields__["supports"].default_factory(), description)
    _MODELS[name] = spec
    return spec


def registered_models() -> list[str]:
    _ensure_builtins()
    return sorted(_MODELS)


def get_model_spec(name: str) -> ModelSpec:
    _ensure_builtins()
    if name not in _MODELS:
        raise ConfigError(f"unknown model {name!r}; registered: {sorted(_MODELS)}")
    return _MODELS[name]


def resolve_state_format(name: str):
    from .state import get_state_format
    return get_state_format(get_model_spec(name).state_format)


_TOWER_FIELDS = ("depth", "hidden_size", "intermediate_size", "num_heads", "in_channels", "patch_size", "spatial_merge_size",
                 "temporal_patch_size", "num_position_embeddings")


def build_registered_model(model_config, dtype=None, device=None):
    """`model_name_or_path` is a registry key or a Hugging Face folder whose config.json names the architecture. A folder
    with a `vision_config` builds the text decoder, or, when `arch_overrides` names a `vision_tower`, the family's
    vision-language model with the folder's tower geometry and placeholder token."""
    _ensure_builtins()
    key = model_config.model_name_or_path
    overrides = {}
    if key not in _MODELS and os.path.isdir(key):
        with open(os.path.join(key, "config.json")) as f:
            hf = json.load(f)
        from .state import registered_for_hf_model_type
        mt = hf.get("model_type", "")
        key, fmt = registered_for_hf_model_type(mt)
        if key is None:
            raise ConfigError(f"Hugging Face model_type {mt!r} has no registered model")
        overrides = fmt.arch_from_hf(hf)
        for k in ("dtype", "device", "model_config"):          # config.json keys that are not architecture (`dtype` is in every
            overrides.pop(k, None)                              # file transformers writes) must not collide with the builder's own
        asked = dict(model_config.arch_overrides or {})
        if asked.get("vision_tower") and isinstance(hf.get("vision_config"), dict) and key + "_vl" in _MODELS:
            # a vision-language folder, and the run wants the tower: the family's `_vl` entry with the folder's tower geometry
            import dataclasses
            tower = {k: v for k, v in hf["vision_config"].items() if k in _TOWER_FIELDS}
            tower.update(asked.get("vision") or {})
            asked.update(vision=tower, image_token_id=asked.get("image_token_id", hf.get("image_token_id")))
            model_config = dataclasses.replace(model_config, arch_overrides=asked)
            key = key + "_vl"
    spec = get_model_spec(key)
    model = spec.builder(model_config, dtype=dtype, device=device, **overrides)
    model.state_format = spec.state_format           # read by the HF and reference-layout converters
    return model


_loaded = False


def _ensure_builtins() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    from . import qwen3
    reg = lambda n, b, **kw: register_model(n, b, replace=True, **kw)  # noqa: E731
    reg("qwen3_moe", qwen3.build_qwen3, state_format="qwen3", description="Qwen3 dense / MoE decoder")
    reg("qwen3", qwen3.build_qwen3, state_format="qwen3", description="dense Qwen3 (alias of qwen3_moe without experts)")
    reg("qwen3_8b", lambda mc, dtype=None, device=None, **kw: qwen3.build_qwen3(mc, dtype, device, **{**qwen3.QWEN3_8B, **(mc.arch_overrides or {}), **kw}),
        state_format="qwen3", description="Qwen3-8B architecture")
    reg("qwen3_30b_a3b", lambda mc, dtype=None, device=None, **kw: qwen3.build_qwen3(mc, dtype, device, **{**qwen3.QWEN3_30B_A3B, **(mc.arch_overrides or {}), **kw}),
        state_format="qwen3", description="Qwen3-30B-A3B architecture")
    from . import deepseek_v4, families, kimi_k3, qwen3_5
    families.register_all(reg)
    for name, defaults in (("qwen3_5", qwen3_5.QWEN3_5_DENSE), ("qwen3_5_moe", qwen3_5.QWEN3_5_MOE), ("qwen3_5_moe_text", qwen3_5.QWEN3_5_MOE)):
        reg(name, qwen3_5.build_qwen3_5(defaults), state_format="qwen3_5", supports={"fsdp", "ep", "cp", "ac"},
            description="Qwen3.5 text decoder: gated delta-net layers with a gated full attention every 4th, zero-centred norms")
    reg("kimi_k3_vl", kimi_k3.build_kimi_vl(kimi_k3.KIMI_K3_DEFAULTS), state_format="kimi", supports={"fsdp", "ep", "ac"},
        description="Kimi-K3 with the MoonViT tower: learned interpolated position table, time-pooled patch merger")
    for name, defaults in (("qwen3_5_vl", qwen3_5.QWEN3_5_DENSE), ("qwen3_5_moe_vl", qwen3_5.QWEN3_5_MOE)):
        reg(name, qwen3_5.build_qwen3_5_vl(defaults), state_format="qwen3_5_vl", supports={"fsdp", "ep", "ac"},
            description="Qwen3.5 vision-language model: vision tower with patch merger feeding image rows into the text decoder")
    reg("kimi_linear", kimi_k3.build_kimi(kimi_k3.KIMI_LINEAR_DEFAULTS), state_format="kimi", supports={"fsdp", "ep", "cp", "ac"},
        description="Kimi-Linear decoder: KDA with short convolutions, latent attention without rotary, grouped sigmoid router")
    reg("kimi_k3", kimi_k3.build_kimi(kimi_k3.KIMI_K3_DEFAULTS), state_format="kimi", supports={"fsdp", "ep", "cp", "ac"},
        description="Kimi-K3 text decoder: Kimi-Linear plus attention residuals, SituGLU and latent-space experts")
    reg("deepseek_v4", deepseek_v4.build_deepseek_v4, state_format="deepseek_v4", supports={"fsdp", "ep", "cp", "ac"},
        description="DeepSeek-V4 decoder: hyper-connections, shared-KV sliding/compressed attention with an indexer, hash and "
                    "biased top-k routers")
