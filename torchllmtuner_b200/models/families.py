"""Further model families behind the same registry and contracts as Qwen3
(reference: llmtuner/models/qwen/qwen3_5*, llmtuner/models/deepseek/deepseek_v4/*, llmtuner/models/kimi/kimi_k3/*).

They share one hybrid decoder: every layer has a token mixer and an MLP (dense or the shared MoE block).
  qwen3_5 / qwen3_5_moe / qwen3_5_moe_text   3 of 4 layers use a gated delta-net linear attention, every 4th layer a
                                             softmax attention with an output gate; gated RMSNorm on the mixer output
  kimi_linear / kimi_k3                      KDA (delta rule with per-channel decay) layers with an MLA (latent
                                             attention) layer every 4th; sigmoid router with shared experts
  deepseek_v4                                latent attention (low-rank KV with a decoupled rotary key), sigmoid router
                                             with the aux-loss-free selection bias, hyper-connections (several residual
                                             streams mixed by learned weights)
Softmax attention and every GEMM run on the sm_100a kernels; the recurrent delta-rule scan is plain PyTorch (chunked
over documents). The vision tower, the 3-axis rotary positions and the wrapper that splices image rows into these decoders
are in `models/vision.py`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .common import GatedMLP, Linear, RMSNorm
from .moe import MoE
from .qwen3 import Embedding, ForwardContext, Qwen3Attention, Qwen3Config, Qwen3ForCausalLM, Qwen3Model


@dataclass
class HybridConfig(Qwen3Config):
    mixer_pattern: list[str] = field(default_factory=lambda: ["delta", "delta", "delta", "attention"])
    delta_heads: int = 4
    delta_head_dim: int = 32
    delta_channel_decay: bool = False          # True: KDA (per-channel decay), False: gated delta-net (per-head decay)
    attention_output_gate: bool = True
    kv_lora_rank: int = 64                     # latent attention
    qk_rope_dim: int = 32
    hyper_connection_streams: int = 1
    model_type: str = "qwen3_5"


def _doc_starts(meta, T: int, device) -> torch.Tensor:
    s = torch.zeros(T, dtype=torch.bool, device=device)
    for p in meta.pieces:
        if 0 <= p[0] < T:
            s[p[0]] = True
    return s


class DeltaRuleMixer(nn.Module):
    """Gated delta rule: S_t = a_t * S_{t-1} (I - b_t k_t k_t^T) + b_t k_t v_t^T ; o_t = S_t^T q_t, per head, state reset
    at document starts. `channel_decay` makes a_t a vector over the key dimension (KDA)."""

    def __init__(self, cfg: HybridConfig, dtype=None, device=None):
        super().__init__()
        D, H, d = cfg.hidden_size, cfg.delta_heads, cfg.delta_head_dim
        self.H, self.d, self.channel = H, d, cfg.delta_channel_decay
        self.q_proj, self.k_proj, self.v_proj = (Linear(D, H * d, dtype, device) for _ in range(3))
        self.beta_proj = Linear(D, H, dtype, device)
        self.decay_proj = Linear(D, H * d if self.channel else H, dtype, device)
        self.gate_proj = Linear(D, H * d, dtype, device)
        self.out_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.o_proj = Linear(H * d, D, dtype, device)

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        T, H, d = x.shape[0], self.H, self.d
        q = F.normalize(self.q_proj(x).view(T, H, d).float(), dim=-1)
        k = F.normalize(self.k_proj(x).view(T, H, d).float(), dim=-1)
        v = self.v_proj(x).view(T, H, d).float()
        beta = torch.sigmoid(self.beta_proj(x).float())                                   # [T, H]
        dec = torch.exp(-F.softplus(self.decay_proj(x).float()))                          # in (0, 1)
        dec = dec.view(T, H, d) if self.channel else dec.view(T, H, 1).expand(T, H, d)
        starts = _doc_starts(ctx.attn_meta, T, x.device)
        S = x.new_zeros(H, d, d, dtype=torch.float32)
        outs = []
        for t in range(T):
            if starts[t]:
                S = torch.zeros_like(S)
            kt, vt, bt = k[t], v[t], beta[t].unsqueeze(-1)
            S = S * dec[t].unsqueeze(-1)
            pred = torch.einsum("hkv,hk->hv", S, kt)
            S = S + torch.einsum("hk,hv->hkv", kt, bt * (vt - pred))
            outs.append(torch.einsum("hkv,hk->hv", S, q[t]))
        o = torch.stack(outs).to(x.dtype)                                                 # [T, H, d]
        o = self.out_norm(o.reshape(T * H, d)).view(T, H * d) * F.silu(self.gate_proj(x))  # gated RMSNorm
        return self.o_proj(o)


class GatedAttention(Qwen3Attention):
    """Softmax attention whose output is multiplied by sigmoid(W_g x) before the output projection."""

    def __init__(self, cfg: HybridConfig, dtype=None, device=None):
        super().__init__(cfg, dtype, device)
        self.gate = Linear(cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, dtype, device) if cfg.attention_output_gate else None

    def forward(self, x, ctx):
        q, k, v = self.project_qkv(x)
        q, k = ops.qk_norm_rope(q, k, self.q_norm.weight if self.q_norm is not None else None,
                                self.k_norm.weight if self.k_norm is not None else None, ctx.cos, ctx.sin, self.eps)
        o = ops.attention(q, k, v, ctx.attn_meta, self.scale).reshape(x.shape[0], -1)
        if self.gate is not None:
            o = o * torch.sigmoid(self.gate(x))
        return self.o_proj(o)


class LatentAttention(nn.Module):
    """Multi-head latent attention: keys and values are up-projected from a shared low-rank latent; a small rotary key
    shared by all heads is concatenated to the per-head non-rotary key."""

    def __init__(self, cfg: HybridConfig, dtype=None, device=None):
        super().__init__()
        D, H, d = cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim
        self.H, self.d, self.dr = H, d, cfg.qk_rope_dim
        self.dn = d - self.dr
        self.q_proj = Linear(D, H * d, dtype, device)
        self.kv_down = Linear(D, cfg.kv_lora_rank, dtype, device)
        self.kv_norm = RMSNorm(cfg.kv_lora_rank, cfg.rms_norm_eps, dtype, device)
        self.k_up = Linear(cfg.kv_lora_rank, H * self.dn, dtype, device)
        self.v_up = Linear(cfg.kv_lora_rank, H * d, dtype, device)
        self.k_rope = Linear(D, self.dr, dtype, device)
        self.o_proj = Linear(H * d, D, dtype, device)
        self.scale = 1.0 / math.sqrt(d)

    def _rope(self, t, cos, sin):
        half = t.shape[-1] // 2
        c, s = cos[:, None, :half].to(t.dtype), sin[:, None, :half].to(t.dtype)
        a, b = t[..., :half], t[..., half:]
        return torch.cat((a * c - b * s, b * c + a * s), -1)

    def forward(self, x, ctx):
        T, H = x.shape[0], self.H
        q = self.q_proj(x).view(T, H, self.d)
        c = self.kv_norm(self.kv_down(x))
        kn = self.k_up(c).view(T, H, self.dn)
        v = self.v_up(c).view(T, H, self.d)
        kr = self._rope(self.k_rope(x).view(T, 1, self.dr), ctx.cos, ctx.sin).expand(T, H, self.dr)
        q = torch.cat((q[..., :self.dn], self._rope(q[..., self.dn:], ctx.cos, ctx.sin)), -1)
        k = torch.cat((kn, kr), -1)
        o = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), ctx.attn_meta, self.scale)
        return self.o_proj(o.reshape(T, -1))


_MIXERS = {"attention": GatedAttention, "delta": DeltaRuleMixer, "kda": DeltaRuleMixer, "mla": LatentAttention}


class HybridDecoderLayer(nn.Module):
    def __init__(self, cfg: HybridConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        kind = cfg.mixer_pattern[layer_idx % len(cfg.mixer_pattern)]
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = _MIXERS[kind](cfg, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        if cfg.is_moe_layer(layer_idx):
            self.mlp = MoE(cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                           shared_inter=cfg.shared_expert_intermediate_size, score_fn=cfg.router_score_fn,
                           norm_topk_prob=cfg.norm_topk_prob, route_scale=cfg.route_scale,
                           bias_update_coeff=cfg.router_bias_update_coeff, aux_loss_coef=cfg.router_aux_loss_coef,
                           dtype=dtype, device=device, shared_mlp_factory=lambda inter: GatedMLP(cfg.hidden_size, inter, dtype, device))
        else:
            self.mlp = GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device)
        n = cfg.hyper_connection_streams
        self.streams = n
        if n > 1:   # hyper-connections: read weights, write weights and a stream-mixing matrix per sub-layer
            self.hc_read = nn.Parameter(torch.full((2, n), 1.0 / n, dtype=dtype, device=device))
            self.hc_write = nn.Parameter(torch.ones(2, n, dtype=dtype, device=device))
            self.hc_mix = nn.Parameter(torch.eye(n, dtype=dtype, device=device).repeat(2, 1, 1))

    def _sub(self, i, xs, fn):
        if self.streams == 1:
            return xs + fn(xs)
        h = torch.einsum("n,ntd->td", self.hc_read[i].to(xs.dtype), xs)
        y = fn(h)
        return torch.einsum("mn,ntd->mtd", self.hc_mix[i].to(xs.dtype), xs) + self.hc_write[i].to(xs.dtype)[:, None, None] * y

    def forward(self, x, ctx):
        x = self._sub(0, x, lambda h: self.self_attn(self.input_layernorm(h), ctx))
        return self._sub(1, x, lambda h: self.mlp(self.post_attention_layernorm(h)))


class HybridForCausalLM(Qwen3ForCausalLM):
    def __init__(self, cfg: HybridConfig, dtype=None, device=None):
        nn.Module.__init__(self)
        self.config = cfg
        self.model = Qwen3Model.__new__(Qwen3Model)
        nn.Module.__init__(self.model)
        self.model.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.model.layers = nn.ModuleList(HybridDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers))
        self.model.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype, device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.activation_checkpoint, self.ac_save_every, self.block_runner = "none", 2, None
        self.pp_first = self.pp_last = True

    def initialize_parameters(self, seed=None):
        super().initialize_parameters(seed)
        with torch.no_grad():
            for m in self.modules():
                if isinstance(m, HybridDecoderLayer) and m.streams > 1:
                    m.hc_read.fill_(1.0 / m.streams)
                    m.hc_write.fill_(1.0)
                    m.hc_mix.copy_(torch.eye(m.streams).repeat(2, 1, 1))

    def validate_parallel(self, tp=1, cp_ulysses=1, ep=1):
        from ..errors import UnsupportedCombinationError
        if tp > 1 or cp_ulysses > 1:
            raise UnsupportedCombinationError(f"{self.config.model_type}: tensor / context parallelism is defined for the Qwen3 family only")
        super().validate_parallel(1, 1, ep)

    def forward(self, tokens, ctx, skip_lm_head=False, inputs_embeds=None):
        n = self.config.hyper_connection_streams
        x = inputs_embeds if inputs_embeds is not None else (self.model.embed_tokens(tokens) if self.pp_first else tokens)
        if n > 1:
            x = x.unsqueeze(0).repeat(n, 1, 1)
        for i, layer in enumerate(self.model.layers):
            x = self.run_block(i, layer, x, ctx)
        if n > 1:
            x = x.sum(0)
        h = self.model.norm(x)
        return h if skip_lm_head else self.lm_head(h)


def _builder(defaults: dict):
    def build(model_config, dtype=None, device=None, **overrides):
        kw = dict(vocab_size=model_config.vocab_size, hidden_size=model_config.hidden_size, intermediate_size=model_config.intermediate_size,
                  num_hidden_layers=model_config.num_hidden_layers, num_attention_heads=model_config.num_attention_heads,
                  num_key_value_heads=model_config.num_key_value_heads)
        kw.update(defaults)
        kw.update(model_config.arch_overrides or {})
        kw.update(overrides)
        names = set(HybridConfig.__dataclass_fields__)
        return HybridForCausalLM(HybridConfig(**{k: v for k, v in kw.items() if k in names}), dtype=dtype, device=device)
    return build


FAMILIES = {
    "qwen3_5": dict(model_type="qwen3_5", mixer_pattern=["delta", "delta", "delta", "attention"]),
    "qwen3_5_moe": dict(model_type="qwen3_5_moe", mixer_pattern=["delta", "delta", "delta", "attention"], num_experts=8,
                        num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64),
    "qwen3_5_moe_text": dict(model_type="qwen3_5_moe_text", mixer_pattern=["delta", "delta", "delta", "attention"], num_experts=8,
                             num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64),
    "kimi_linear": dict(model_type="kimi_linear", mixer_pattern=["kda", "kda", "kda", "mla"], delta_channel_decay=True, num_experts=8,
                        num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64, router_score_fn="sigmoid",
                        mlp_only_layers=[0]),
    "kimi_k3": dict(model_type="kimi_k3", mixer_pattern=["kda", "kda", "kda", "mla"], delta_channel_decay=True, num_experts=8,
                    num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64, router_score_fn="sigmoid",
                    mlp_only_layers=[0]),
    "deepseek_v4": dict(model_type="deepseek_v4", mixer_pattern=["mla"], num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                        shared_expert_intermediate_size=64, router_score_fn="sigmoid", router_bias_update_coeff=1e-3,
                        hyper_connection_streams=2, mlp_only_layers=[0]),
}


def register_all(reg) -> None:
    for name, defaults in FAMILIES.items():
        reg(name, _builder(defaults), state_format="native", supports={"fsdp", "ep", "ac"},
            description=f"{name} text decoder (hybrid mixer family)")
