"""Declared configuration of the teaching framework and the signature that a resume must match."""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass


@dataclass
class MiniConfig:
    vocab_size: int = 128
    hidden_size: int = 64
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 16
    num_experts: int = 4
    top_k: int = 2
    moe_intermediate_size: int = 32
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    # mesh: world = dp * ep * tp, ranks laid out with tp fastest, then ep, then dp
    dp: int = 1
    ep: int = 1
    tp: int = 1
    # training
    batch_size: int = 2                    # sequences per micro-batch and data-parallel rank
    seq_len: int = 32
    gradient_accumulation_steps: int = 1
    learning_rate: float = 3e-3
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    warmup_steps: int = 0
    steps: int = 3                         # target number of optimizer steps (a resume continues up to it)
    seed: int = 0
    device: str = "cpu"

    RESUME_MAY_CHANGE = ("steps", "device")

    def validate(self, world: int) -> None:
        if self.dp * self.ep * self.tp != world:
            raise ValueError(f"world size {world} != dp {self.dp} x ep {self.ep} x tp {self.tp}")
        if self.num_heads % self.tp or self.num_kv_heads % self.tp or self.moe_intermediate_size % self.tp:
            raise ValueError("tp must divide num_heads, num_kv_heads and moe_intermediate_size")
        if self.num_experts % self.ep:
            raise ValueError("ep must divide num_experts")
        if self.num_heads % self.num_kv_heads or self.top_k > self.num_experts:
            raise ValueError("num_heads must be a multiple of num_kv_heads and top_k <= num_experts")

    def signature(self) -> str:
        d = {k: v for k, v in asdict(self).items() if k not in self.RESUME_MAY_CHANGE}
        return hashlib.sha256(json.dumps(d, sort_keys=True).encode()).hexdigest()
