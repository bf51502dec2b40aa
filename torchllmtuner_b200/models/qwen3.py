"""Qwen3 dense and Qwen3-MoE decoder (reference: llmtuner/models/qwen/qwen3/model.py:125-1053).

One class covers both: a layer is sparse when `num_experts > 0`, it is not listed in `mlp_only_layers` and
`(i + 1) % decoder_sparse_step == 0`; a dense model is `num_experts == 0` (or every layer in `mlp_only_layers`, which
is how the reference spells dense Qwen3). GQA attention with per-head RMSNorm on q/k, half-rotation RoPE (theta 1e6),
SwiGLU MLP, softmax top-k router with renormalisation, packed experts.

Rows are packed: the model works on `[T, D]` with T = all tokens of the micro-batch; documents and the causal
structure come from `AttnMeta` (cu_seqlens), never from a dense mask.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass, field

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..ops import AttnMeta
from .common import Embedding, GatedMLP, Linear, RMSNorm, next_token_targets
from .contracts import DecoderStructure
from .moe import MoE


@dataclass
class Qwen3Config:
    vocab_size: int = 128
    hidden_size: int = 64
    intermediate_size: int = 128
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 4
    head_dim: int | None = None
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    tie_word_embeddings: bool = False
    qk_norm: bool = True
    initializer_range: float = 0.02
    max_position_embeddings: int = 131072
    # sparse part
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: list[int] = field(default_factory=list)
    router_score_fn: str = "softmax"
    route_scale: float = 1.0
    router_bias_update_coeff: float = 0.0      # aux-loss-free balancing (0 disables)
    router_aux_loss_coef: float = 0.0
    moe_quantile_balancing: bool = False
    fixed_router: bool = False
    # runtime knobs
    qkv_projection: str = "separate"
    experts_implementation: str = "native"
    model_type: str = "qwen3_moe"

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")

    def is_moe_layer(self, i: int) -> bool:
        return (self.num_experts > 0 and i not in self.mlp_only_layers and (i + 1) % max(1, self.decoder_sparse_step) == 0)

    def flops_per_token(self, seq_len: int) -> float:
        from ..utils.flops import generic_flops_per_token
        mask = [self.is_moe_layer(i) for i in range(self.num_hidden_layers)]
        return generic_flops_per_token(hidden_size=self.hidden_size, num_layers=self.num_hidden_layers,
                                       num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
                                       head_dim=self.head_dim, intermediate_size=self.intermediate_size,
                                       vocab_size=self.vocab_size, seq_len=seq_len, num_experts=self.num_experts,
                                       top_k=self.num_experts_per_tok, moe_intermediate_size=self.moe_intermediate_size,
                                       shared_intermediate_size=self.shared_expert_intermediate_size, moe_layer_mask=mask)


QWEN3_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, rope_theta=1e6, tie_word_embeddings=False)
QWEN3_30B_A3B = dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32,
                     num_key_value_heads=4, head_dim=128, rope_theta=1e6, num_experts=128, num_experts_per_tok=8,
                     moe_intermediate_size=768, norm_topk_prob=True, tie_word_embeddings=False)


@dataclass
class ForwardContext:
    """Per-micro-batch constants shared by all layers."""
    cos: torch.Tensor
    sin: torch.Tensor
    attn_meta: AttnMeta
    cp: object | None = None          # context-parallel attention driver, see parallel/context_parallel.py


class Qwen3Attention(nn.Module):
    def __init__(self, cfg: Qwen3Config, dtype=None, device=None):
        super().__init__()
        D, d = cfg.hidden_size, cfg.head_dim
        self.num_heads, self.num_kv_heads, self.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, d
        self.eps = cfg.rms_norm_eps
        self.fused_qkv = cfg.qkv_projection == "fused"
        if self.fused_qkv:
            self.qkv_proj = Linear(D, (self.num_heads + 2 * self.num_kv_heads) * d, dtype, device)
        else:
            self.q_proj = Linear(D, self.num_heads * d, dtype, device)
            self.k_proj = Linear(D, self.num_kv_heads * d, dtype, device)
            self.v_proj = Linear(D, self.num_kv_heads * d, dtype, device)
        self.o_proj = Linear(self.num_heads * d, D, dtype, device)
        self.q_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.k_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device) if cfg.qk_norm else None
        self.scale = 1.0 / math.sqrt(d)

    accepts_sharded_rows = True     # `x` may be a row-sharded handle whose `linears` gathers inside the first GEMM

    def project_qkv(self, x):
        d = self.head_dim
        if hasattr(x, "linears") and not self.fused_qkv:
            q, k, v = x.linears(self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)
            T = q.shape[0]
            return q.view(T, -1, d), k.view(T, -1, d), v.view(T, -1, d)
        T = x.shape[0]
        if self.fused_qkv:
            qkv = self.qkv_proj(x)
            nq, nk = self.num_heads * d, self.num_kv_heads * d
            return (qkv[:, :nq].view(T, -1, d), qkv[:, nq:nq + nk].view(T, -1, d), qkv[:, nq + nk:].view(T, -1, d))
        q, k, v = ops.linears(x, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)
        return q.view(T, -1, d), k.view(T, -1, d), v.view(T, -1, d)

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        q, k, v = self.project_qkv(x)
        q, k = ops.qk_norm_rope(q, k, self.q_norm.weight if self.q_norm is not None else None,
                                self.k_norm.weight if self.k_norm is not None else None, ctx.cos, ctx.sin, self.eps)
        if ctx.cp is not None:
            o = ctx.cp.attention(q, k, v, ctx.attn_meta, self.scale)
        else:
            o = ops.attention(q, k, v, ctx.attn_meta, self.scale)
        return self.o_proj(o.reshape(o.shape[0], -1))


class Qwen3DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen3Config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = Qwen3Attention(cfg, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        if cfg.is_moe_layer(layer_idx):
            shared = (lambda inter: GatedMLP(cfg.hidden_size, inter, dtype, device))
            self.mlp = MoE(cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                           shared_inter=cfg.shared_expert_intermediate_size, score_fn=cfg.router_score_fn,
                           norm_topk_prob=cfg.norm_topk_prob, route_scale=cfg.route_scale,
                           bias_update_coeff=cfg.router_bias_update_coeff, aux_loss_coef=cfg.router_aux_loss_coef,
                           quantile_balancing=cfg.moe_quantile_balancing, fixed_router=cfg.fixed_router,
                           experts_implementation=cfg.experts_implementation, dtype=dtype, device=device,
                           shared_mlp_factory=shared)
        else:
            self.mlp = GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device)

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        a = self.self_attn(self.input_layernorm(x), ctx)
        h, x = self.post_attention_layernorm(a, x)      # x <- x + a ; h = norm(x), one pass
        return x + self.mlp(h)


class Qwen3Model(nn.Module):
    def __init__(self, cfg: Qwen3Config, dtype=None, device=None):
        super().__init__()
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.layers = nn.ModuleList(Qwen3DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


class Qwen3ForCausalLM(nn.Module):
    """`forward(tokens [T], ctx, skip_lm_head)` -> hidden [T, D] or logits [T, V]."""

    decoder_structure = DecoderStructure()

    def __init__(self, cfg: Qwen3Config, dtype=None, device=None):
        super().__init__()
        self.config = cfg
        self.model = Qwen3Model(cfg, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype, device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.activation_checkpoint = "none"     # set by the AC stage: none | full | selective
        self.ac_save_every = 2
        self.block_runner = None                # set by the FSDP stage to own gather/recompute/reduce per block
        self.pp_first = self.pp_last = True     # pipeline stage position (both True without pipeline parallelism)

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def initialize_parameters(self, seed: int | None = None) -> None:
        """normal(0, initializer_range) for matrices, ones for norm weights (reference: model.py:729)."""
        gen = None
        std = self.config.initializer_range
        for name, p in self.named_parameters():
            if p.is_meta:
                continue
            if name.endswith("norm.weight") or "layernorm" in name:
                p.fill_(1.0)
            else:
                if seed is not None:
                    gen = torch.Generator(device=p.device).manual_seed(seed * 1000003 + zlib.crc32(name.encode()))
                p.normal_(0.0, std, generator=gen)
        for m in self.modules():
            if isinstance(m, MoE):
                m.expert_bias_E.zero_()
                m.tokens_per_expert_E.zero_()

    # ------------------------------------------------------------------ contracts
    def tp_config(self) -> dict[str, str]:
        """Default tensor-parallel plan (reference: model.py:750-773): q/k/v colwise, o rowwise, q/k norms replicated,
        gate/up colwise, down rowwise, packed experts colwise / rowwise, lm_head replicated, embedding vocab-parallel."""
        return {
            "self_attn.q_proj": "colwise", "self_attn.k_proj": "colwise", "self_attn.v_proj": "colwise",
            "self_attn.o_proj": "rowwise", "mlp.gate_proj": "colwise", "mlp.up_proj": "colwise", "mlp.down_proj": "rowwise",
            "mlp.routed.experts": "moe", "mlp.shared_experts.gate_proj": "colwise", "mlp.shared_experts.up_proj": "colwise",
            "mlp.shared_experts.down_proj": "rowwise", "model.embed_tokens": "vocab", "lm_head": "replicate",
        }

    def validate_parallel(self, tp: int = 1, cp_ulysses: int = 1, ep: int = 1) -> None:
        from ..errors import UnsupportedCombinationError
        from ..parallel.attention_heads import require_heads_divisible_by
        c = self.config
        require_heads_divisible_by(self, size=tp, axis="tensor_parallel_size",
                                   why="every tensor-parallel rank owns whole query and key/value heads")
        require_heads_divisible_by(self, size=tp * cp_ulysses, axis="tensor_parallel_size * context_parallel_ulysses_size",
                                   why="the Ulysses exchange hands each rank whole heads of its tensor-parallel share")
        if c.num_experts and c.num_experts % ep:
            raise UnsupportedCombinationError(f"expert_parallel_size {ep} must divide num_experts {c.num_experts}")

    def flops_per_token(self, seq_len: int) -> float:
        return self.config.flops_per_token(seq_len)

    # ------------------------------------------------------------------ inputs
    def prepare_inputs(self, batch: dict, device=None, parallel_dims=None) -> dict:
        """Batch dict with `input` [B,S] ids, `labels` [B,S] (already shifted targets), optional `positions` [B,S] and
        `cu_seqlens` -> packed model inputs. Context/tensor-parallel sharding of the rows is applied by
        `parallel.input_sharding.shard_model_inputs` when `parallel_dims` has cp or tp > 1
        (reference: model.py:796-842, models/common/input_preparation.py:112-197)."""
        from ..parallel.input_sharding import shard_model_inputs
        ids, labels = batch["input"], batch["labels"]
        B, S = ids.shape
        positions = batch.get("positions")
        if positions is None:
            positions = torch.arange(S, dtype=torch.int64).repeat(B, 1)
        cu = batch.get("cu_seqlens")
        if cu is None:
            cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32)
        out = {"tokens": ids.reshape(-1), "targets": labels.reshape(-1), "positions": positions.reshape(-1),
               "cu_seqlens": cu, "batch": B, "seq": S}
        out = shard_model_inputs(out, parallel_dims)
        dev = device if device is not None else next(self.parameters()).device
        for k in ("tokens", "targets", "positions"):
            out[k] = out[k].to(dev, non_blocking=True)
        if "attn_meta" not in out:
            out["attn_meta"] = AttnMeta.build(out["cu_seqlens"], causal=True, device=dev)
        return out

    def build_context(self, positions: torch.Tensor, attn_meta: AttnMeta, cp=None) -> ForwardContext:
        cos, sin = ops.rope_tables(positions, self.config.head_dim, self.config.rope_theta)
        return ForwardContext(cos, sin, attn_meta, cp)

    # ------------------------------------------------------------------ forward
    def run_block(self, i: int, layer: nn.Module, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        if self.block_runner is not None:
            return self.block_runner(i, layer, x, ctx)
        ac = self.activation_checkpoint
        mask = getattr(self, "ac_block_mask", None)
        recompute = bool(mask[i]) if mask is not None and i < len(mask) else i % self.ac_save_every != 0
        use_ac = self.training and torch.is_grad_enabled() and (ac == "full" or (ac == "selective" and recompute))
        if use_ac:
            return checkpoint(layer, x, ctx, use_reentrant=False)
        return layer(x, ctx)

    def forward(self, tokens: torch.Tensor, ctx: ForwardContext, skip_lm_head: bool = False, inputs_embeds=None) -> torch.Tensor:
        """`tokens` are ids on the first pipeline stage (or without pipeline parallelism) and the previous stage's hidden
        rows otherwise; a stage that is not the last returns hidden rows. `inputs_embeds` [T, D] replaces the embedding
        lookup (multimodal wrappers splice image rows in first)."""
        x = inputs_embeds if inputs_embeds is not None else (self.model.embed_tokens(tokens) if self.pp_first else tokens)
        layers = self.model.layers
        for i, layer in enumerate(layers.values() if isinstance(layers, nn.ModuleDict) else layers):
            x = self.run_block(getattr(layer, "layer_idx", i), layer, x, ctx)
        if not self.pp_last:
            return x
        h = self.model.norm(x)
        if skip_lm_head:
            return h
        return self.lm_head(h)


def build_qwen3(model_config, dtype=None, device=None, **overrides) -> Qwen3ForCausalLM:
    """From the `ModelConfig` group: toy sizes from the flat fields, anything else through `arch_overrides`."""
    kw = dict(vocab_size=model_config.vocab_size, hidden_size=model_config.hidden_size,
              intermediate_size=model_config.intermediate_size, num_hidden_layers=model_config.num_hidden_layers,
              num_attention_heads=model_config.num_attention_heads, num_key_value_heads=model_config.num_key_value_heads,
              qkv_projection=model_config.qkv_projection, experts_implementation=model_config.experts_implementation)
    kw.update(model_config.arch_overrides or {})
    kw.update(overrides)
    names = set(Qwen3Config.__dataclass_fields__)
    cfg = Qwen3Config(**{k: v for k, v in kw.items() if k in names})
    return Qwen3ForCausalLM(cfg, dtype=dtype, device=device)
