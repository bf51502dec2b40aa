"""Qwen3.5 / Qwen3.5-MoE text decoder (reference: llmtuner/models/qwen/qwen3_5_moe/model.py:57-1036, gated_delta.py:13-189,
rotary.py:1-108, llmtuner/models/qwen/qwen3_5/*).

  * three of four layers are gated delta-net mixers: ONE projection produces q, k and v, which pass together through a
    short depthwise causal convolution with SiLU (restarting at every document); L2-normalised q and k, q scaled by
    d_k^-1/2; value heads may outnumber key heads (keys and queries are repeated); one decay per value head,
    log a = -exp(A_log) * softplus(a(x) + dt_bias); write strength sigmoid(b(x)); the output is RMS-normalised per head,
    multiplied by silu(z(x)) and projected;
  * every fourth layer is softmax attention whose query projection also yields a per-channel output gate
    (o * sigmoid(gate)); q and k are normalised per head; only the first `partial_rotary_factor` of each head rotates
    (half-rotation layout); positions may be three-axis (time, height, width) with the axes interleaved over the
    frequencies;
  * every norm over the model width is "zero-centred": y = x_hat * (1 + w), w initialised to 0;
  * the feed-forward is a sparse block in the MoE family (softmax router, renormalised top-k, packed experts, one shared
    expert whose output is scaled by sigmoid(w_g . x)) or a dense gated MLP in the dense family.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .common import Embedding, GatedMLP, Linear
from .contracts import DecoderStructure
from .families import chunked_delta_rule
from .kimi_k3 import CausalConvolution
from .moe import MoE
from .qwen3 import ForwardContext, Qwen3Config, Qwen3ForCausalLM, Qwen3Model


@dataclass
class Qwen35Config(Qwen3Config):
    layer_types: list[str] = field(default_factory=list)
    full_attention_interval: int = 4
    linear_num_value_heads: int = 4
    linear_num_key_heads: int = 2
    linear_key_head_dim: int = 16
    linear_value_head_dim: int = 16
    linear_conv_kernel_dim: int = 4
    linear_chunk_size: int = 64
    partial_rotary_factor: float = 0.25
    mrope_section: list[int] = field(default_factory=list)      # frequencies per axis (time, height, width); default: near-equal thirds
    attn_output_gate: bool = True
    rope_theta: float = 10_000_000.0
    model_type: str = "qwen3_5_moe"

    def __post_init__(self):
        super().__post_init__()
        n = self.num_hidden_layers
        if not self.layer_types:
            self.layer_types = ["full_attention" if (i + 1) % self.full_attention_interval == 0 else "linear_attention" for i in range(n)]
        if len(self.layer_types) != n or any(t not in ("linear_attention", "full_attention") for t in self.layer_types):
            raise ValueError("Qwen3.5 layer_types must name every layer as linear_attention or full_attention")
        if self.linear_num_value_heads % self.linear_num_key_heads:
            raise ValueError("linear_num_value_heads must be a multiple of linear_num_key_heads")
        rot = int(self.head_dim * self.partial_rotary_factor)
        if rot <= 0 or rot % 2:
            raise ValueError("head_dim * partial_rotary_factor must be a positive even number")
        self.rotary_dim = rot
        if not self.mrope_section:
            half = rot // 2
            self.mrope_section = [half - 2 * (half // 3), half // 3, half // 3]
        if sum(self.mrope_section) != rot // 2:
            raise ValueError(f"mrope_section {self.mrope_section} must sum to {rot // 2}")


@dataclass
class Qwen35Context(ForwardContext):
    positions: torch.Tensor | None = None      # [T] index inside the document (drives the convolution's restarts)


# --------------------------------------------------------------------------------------------------- small pieces
class ZeroCenteredRMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.eps)
        return (y * (1.0 + self.weight.float())).to(x.dtype)


class GatedRMSNorm(nn.Module):
    """norm(x) * w, then * silu(gate); the gate multiplies in fp32."""

    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x, gate):
        xf = x.float()
        y = (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight
        return (y * F.silu(gate.float())).to(x.dtype)


def mrope_tables(positions: torch.Tensor, rotary_dim: int, theta: float, section: list[int]):
    """positions [T] (text) or [3, T] (time, height, width). Frequency j takes its angle from axis j % 3 while j lies inside
    that axis's interleaved range, else from the time axis. Returns cos, sin [T, rotary_dim] (halves duplicated)."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=positions.device) / rotary_dim))
    if positions.dim() == 1:
        ang = positions.float()[:, None] * inv[None, :]
    else:
        per_axis = positions.float()[:, :, None] * inv[None, None, :]          # [3, T, rot/2]
        ang = per_axis[0].clone()
        for axis, offset in ((1, 1), (2, 2)):
            idx = slice(offset, section[axis] * 3, 3)
            ang[:, idx] = per_axis[axis][:, idx]
    emb = torch.cat((ang, ang), -1)
    return emb.cos(), emb.sin()


def rotate_leading(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, H, d]; the first cos.shape[-1] channels rotate in the half-rotation layout, the rest pass through."""
    r = cos.shape[-1]
    xr, xp = x[..., :r], x[..., r:]
    half = r // 2
    rot = torch.cat((-xr[..., half:], xr[..., :half]), -1)
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return torch.cat((xr * c + rot * s, xp), -1)


def attend(q, k, v, ctx, scale):
    if ctx.cp is not None:
        return ctx.cp.attention(q, k, v, ctx.attn_meta, scale)
    return ops.attention(q, k, v, ctx.attn_meta, scale)


# --------------------------------------------------------------------------------------------------- mixers
class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: Qwen35Config, dtype=None, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.Hv, self.Hk, self.dk, self.dv = cfg.linear_num_value_heads, cfg.linear_num_key_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.Hk * self.dk, self.Hv * self.dv
        self.chunk = cfg.linear_chunk_size
        self.in_proj_qkv = Linear(D, 2 * self.key_dim + self.value_dim, dtype, device)
        self.in_proj_z = Linear(D, self.value_dim, dtype, device)
        self.in_proj_b = Linear(D, self.Hv, dtype, device)
        self.in_proj_a = Linear(D, self.Hv, dtype, device)
        self.conv1d = CausalConvolution(2 * self.key_dim + self.value_dim, cfg.linear_conv_kernel_dim, dtype, device)
        self.dt_bias = nn.Parameter(torch.ones(self.Hv, dtype=torch.float32, device=device))
        self.A_log = nn.Parameter(torch.empty(self.Hv, dtype=torch.float32, device=device))
        self.norm = GatedRMSNorm(self.dv, cfg.rms_norm_eps, dtype, device)
        self.out_proj = Linear(self.value_dim, D, dtype, device)

    def forward(self, x: torch.Tensor, ctx: Qwen35Context) -> torch.Tensor:
        T = x.shape[0]
        cp = ctx.cp if ctx.cp is not None and getattr(ctx.cp, "size", 1) > 1 else None
        mixed = self.in_proj_qkv(x)
        halo = cp.prev_rows(mixed, self.conv1d.kernel - 1) if cp is not None else None
        mixed = self.conv1d(mixed, ctx.positions, halo)
        q = mixed[:, :self.key_dim].view(T, self.Hk, self.dk).float()
        k = mixed[:, self.key_dim:2 * self.key_dim].view(T, self.Hk, self.dk).float()
        v = mixed[:, 2 * self.key_dim:].view(T, self.Hv, self.dv).float()
        q = q * torch.rsqrt(q.square().sum(-1, keepdim=True) + 1e-6) * self.dk ** -0.5
        k = k * torch.rsqrt(k.square().sum(-1, keepdim=True) + 1e-6)
        rep = self.Hv // self.Hk
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
        beta = torch.sigmoid(self.in_proj_b(x).float())
        log_decay = (-self.A_log.float().exp() * F.softplus(self.in_proj_a(x).float() + self.dt_bias.float())).unsqueeze(-1)   # [T, Hv, 1]
        if cp is not None:
            o = cp.delta_rule(q, k, v, beta, log_decay, self.chunk)
        else:
            outs = [chunked_delta_rule(q[a:a + n], k[a:a + n], v[a:a + n], beta[a:a + n], log_decay[a:a + n], self.chunk)
                    for a, n in ((int(p[0]), int(p[1])) for p in ctx.attn_meta.pieces)]
            o = torch.cat(outs) if len(outs) > 1 else outs[0]
        z = self.in_proj_z(x).view(T * self.Hv, self.dv)
        o = self.norm(o.to(x.dtype).reshape(T * self.Hv, self.dv), z)
        return self.out_proj(o.view(T, self.value_dim))


class GatedFullAttention(nn.Module):
    def __init__(self, cfg: Qwen35Config, dtype=None, device=None):
        super().__init__()
        D, d = cfg.hidden_size, cfg.head_dim
        self.H, self.Hkv, self.d, self.gated = cfg.num_attention_heads, cfg.num_key_value_heads, d, cfg.attn_output_gate
        self.q_proj = Linear(D, self.H * d * (2 if self.gated else 1), dtype, device)
        self.k_proj = Linear(D, self.Hkv * d, dtype, device)
        self.v_proj = Linear(D, self.Hkv * d, dtype, device)
        self.o_proj = Linear(self.H * d, D, dtype, device)
        self.q_norm = ZeroCenteredRMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.k_norm = ZeroCenteredRMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.scale = d ** -0.5

    def forward(self, x: torch.Tensor, ctx: Qwen35Context) -> torch.Tensor:
        T = x.shape[0]
        qg = self.q_proj(x)
        if self.gated:                                         # per head: [query | gate]
            qg = qg.view(T, self.H, 2 * self.d)
            q, gate = qg[..., :self.d], qg[..., self.d:].reshape(T, self.H * self.d)
        else:
            q, gate = qg.view(T, self.H, self.d), None
        q = rotate_leading(self.q_norm(q), ctx.cos, ctx.sin)
        k = rotate_leading(self.k_norm(self.k_proj(x).view(T, self.Hkv, self.d)), ctx.cos, ctx.sin)
        v = self.v_proj(x).view(T, self.Hkv, self.d)
        o = attend(q.contiguous(), k.contiguous(), v.contiguous(), ctx, self.scale).reshape(T, self.H * self.d)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self.o_proj(o)


class Qwen35DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen35Config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.layer_type = cfg.layer_types[layer_idx]
        self.self_attn = (GatedDeltaNet if self.layer_type == "linear_attention" else GatedFullAttention)(cfg, dtype, device)
        if cfg.is_moe_layer(layer_idx):
            self.mlp = MoE(cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                           shared_inter=cfg.shared_expert_intermediate_size, score_fn="softmax", norm_topk_prob=cfg.norm_topk_prob,
                           aux_loss_coef=cfg.router_aux_loss_coef, experts_implementation=cfg.experts_implementation, dtype=dtype,
                           device=device, shared_mlp_factory=lambda inter: GatedMLP(cfg.hidden_size, inter, dtype, device),
                           shared_gate=True)
        else:
            self.mlp = GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device)
        self.input_layernorm = ZeroCenteredRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = ZeroCenteredRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)

    def forward(self, x, ctx):
        x = x + self.self_attn(self.input_layernorm(x), ctx)
        return x + self.mlp(self.post_attention_layernorm(x))


class Qwen35ForCausalLM(Qwen3ForCausalLM):
    decoder_structure = DecoderStructure()
    accepts_three_axis_positions = True      # `build_context` takes [3, T] (time, height, width) positions

    def __init__(self, cfg: Qwen35Config, dtype=None, device=None):
        nn.Module.__init__(self)
        self.config = cfg
        self.model = Qwen3Model.__new__(Qwen3Model)
        nn.Module.__init__(self.model)
        self.model.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.model.layers = nn.ModuleList(Qwen35DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers))
        self.model.norm = ZeroCenteredRMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype, device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.activation_checkpoint, self.ac_save_every, self.block_runner = "none", 2, None
        self.pp_first = self.pp_last = True

    @torch.no_grad()
    def initialize_parameters(self, seed: int | None = None) -> None:
        super().initialize_parameters(seed)
        gen = torch.Generator().manual_seed((seed or 0) * 7919 + 29)
        for m in self.modules():
            if isinstance(m, ZeroCenteredRMSNorm) and not m.weight.is_meta:
                m.weight.zero_()
            elif isinstance(m, GatedDeltaNet) and not m.A_log.is_meta:
                m.A_log.copy_(torch.empty(m.Hv).uniform_(0.01, 16, generator=gen).log())
                m.dt_bias.fill_(1.0)
                bound = 1.0 / math.sqrt(m.conv1d.kernel)
                m.conv1d.weight.copy_(torch.empty(m.conv1d.weight.shape).uniform_(-bound, bound, generator=gen))
                m.norm.weight.fill_(1.0)

    def tp_config(self) -> dict[str, str]:
        return {}

    def validate_parallel(self, tp: int = 1, cp_ulysses: int = 1, ep: int = 1) -> None:
        from ..errors import UnsupportedCombinationError
        if tp > 1 or cp_ulysses > 1:
            raise UnsupportedCombinationError("qwen3_5: the fused q/k/v projection and its convolution are not cut by heads here; the "
                                              "hybrid family `qwen3_5_hybrid` carries the tensor-parallel cuts of these mixers")
        if self.config.num_experts and self.config.num_experts % ep:
            raise UnsupportedCombinationError(f"expert_parallel_size {ep} must divide num_experts {self.config.num_experts}")

    def build_context(self, positions, attn_meta, cp=None) -> Qwen35Context:
        c = self.config
        cos, sin = mrope_tables(positions, c.rotary_dim, c.rope_theta, c.mrope_section)
        doc_pos = positions if positions.dim() == 1 else None
        if doc_pos is None:                       # three-axis positions: the convolution restarts come from the document table
            doc_pos = torch.cat([torch.arange(int(p[1]), device=positions.device) for p in attn_meta.pieces])
        return Qwen35Context(cos, sin, attn_meta, cp, positions=doc_pos)


def build_qwen3_5(defaults: dict):
    def build(model_config, dtype=None, device=None, **overrides):
        kw = dict(vocab_size=model_config.vocab_size, hidden_size=model_config.hidden_size, intermediate_size=model_config.intermediate_size,
                  num_hidden_layers=model_config.num_hidden_layers, num_attention_heads=model_config.num_attention_heads,
                  num_key_value_heads=model_config.num_key_value_heads, experts_implementation=model_config.experts_implementation)
        kw.update(defaults)
        kw.update(model_config.arch_overrides or {})
        kw.update(overrides)
        names = set(Qwen35Config.__dataclass_fields__)
        return Qwen35ForCausalLM(Qwen35Config(**{k: v for k, v in kw.items() if k in names}), dtype=dtype, device=device)
    return build


QWEN3_5_DENSE = dict(model_type="qwen3_5")
QWEN3_5_MOE = dict(model_type="qwen3_5_moe", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64,
                   norm_topk_prob=True)


def build_qwen3_5_vl(defaults: dict):
    """Text decoder + vision tower under one model: `arch_overrides` may carry `image_token_id` (default: the last token of
    the vocabulary), `vision` (a dict of the tower's config fields; the output width always follows the text width) and
    `vision_tower`: "generic" (default, `models/vision.py`) or "qwen3_5" (the published tower, `models/qwen_vit.py`)."""
    text_builder = build_qwen3_5(defaults)

    def build(model_config, dtype=None, device=None, **overrides):
        from .vision import VisionConfig, VisionLanguageModel
        text = text_builder(model_config, dtype=dtype, device=device, **overrides)
        extra = dict(model_config.arch_overrides or {})
        image_id = int(extra.get("image_token_id", text.config.vocab_size - 1))
        if extra.get("vision_tower", "generic") == "qwen3_5":        # the published tower, weight for weight (models/qwen_vit.py)
            from .qwen_vit import QwenViTConfig, QwenViTTower
            vkw = dict(extra.get("vision") or {})
            vkw["out_hidden_size"] = text.config.hidden_size
            return VisionLanguageModel(text, QwenViTConfig(**vkw), image_id, dtype=dtype, device=device, tower=QwenViTTower)
        vkw = dict(hidden_size=128, intermediate_size=256, depth=2, num_heads=2)
        vkw.update(extra.get("vision") or {})
        vkw["out_hidden_size"] = text.config.hidden_size
        return VisionLanguageModel(text, VisionConfig(**vkw), image_id, dtype=dtype, device=device)
    return build
