"""Model config group (reference: llmtuner/config/model_config.py:14-211)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .utils import require_choice, require_integer_at_least

DTYPES = (None, "float32", "bfloat16", "float16")


@dataclass
class ModelConfig:
    model_name_or_path: str = "qwen3_moe"        # registry key or a Hugging Face model folder
    initialization_device: str = "cpu"           # cpu | meta
    vocab_size: int = 128
    hidden_size: int = 64
    intermediate_size: int = 128
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 4
    experts_implementation: str = "native"       # native (grouped tcgen05 GEMM) | eager (per-expert loop)
    router_compute_dtype: str | None = None
    norm_backend: str = "native"
    linear_attention_backend: str = "native"
    qkv_projection: str = "separate"             # separate | fused
    rotary_init_device: str = "constructor"
    rotary_compute_dtype: str | None = None
    rotary_cache_dtype: str | None = None
    attention_backend: str = "auto"
    compute_dtype: str | None = None
    arch_overrides: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        require_choice("initialization_device", self.initialization_device, ("cpu", "meta", "cuda"))
        for n in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads"):
            require_integer_at_least(n, getattr(self, n), 1)
        require_choice("qkv_projection", self.qkv_projection, ("separate", "fused"))
        require_choice("experts_implementation", self.experts_implementation, ("native", "eager"))
        for n in ("router_compute_dtype", "rotary_compute_dtype", "rotary_cache_dtype", "compute_dtype"):
            require_choice(n, getattr(self, n), DTYPES)
