"""Kimi-Linear / Kimi-K3 text decoder (reference: llmtuner/models/kimi/kimi_k3/model.py:83-576, delta_attention.py:33-374,
causal_convolution.py:13-111, latent_attention.py:38-255, moe.py:73-711, mlp.py:15-106, attention_residual.py:9-27,
normalization.py:7-77, configuration.py:20-185).

  * KDA layers: q/k/v projections each followed by a short depthwise causal convolution with SiLU that restarts at
    every document; L2-normalised q and k; a delta rule whose state decays PER KEY CHANNEL with
    log a = -exp(A_log[h]) * softplus(f_b(f_a(x)) + dt_bias) (or a bounded sigmoid form when `gate_lower_bound` is
    set); write strength sigmoid(b(x)); output scaled by d^-1/2, normalised per head and gated by sigmoid(g_b(g_a(x))).
    The recurrence runs in the chunk-parallel form of `models/families.py` (batched products and one triangular solve).
  * MLA layers (those not listed in `kda_layers`): latent attention WITHOUT rotary embedding: a low-rank key/value
    latent is expanded per head, one extra key of `qk_rope_head_dim` channels is shared by all heads, values may be
    narrower than keys, optional sigmoid output gate.
  * feed-forward: dense gated MLP for the first `first_k_dense_replace` layers, then a sparse block: sigmoid (or softmax)
    scores, selection on scores + correction bias, optionally restricted to the `topk_group` best of `num_expert_group`
    groups (a group scores the sum of its two best), weights from the plain scores, renormalised when k > 1, times
    `routed_scaling_factor`; experts may work in a narrower latent space (down-projection before dispatch, norm and
    up-projection after the weighted combine); shared experts of width `moe_intermediate_size * num_shared_experts`.
    Activation silu(g)·u or SituGLU: beta·tanh(g/beta)·sigmoid(g) · (linear_beta·tanh(u/linear_beta) | u).
  * optional attention residuals (`attn_res_block_size`): every `block` layers the running residual is filed as a
    block; each sub-layer reads a per-token softmax mixture of the filed blocks and the current running sum, scored by a
    learned direction on the RMS-normalised candidates.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .common import Embedding, GatedMLP, Linear, RMSNorm
from .contracts import DecoderStructure
from .families import chunked_delta_rule
from .moe import MoE
from .qwen3 import ForwardContext, Qwen3Config, Qwen3ForCausalLM, Qwen3Model


@dataclass
class KimiConfig(Qwen3Config):
    # linear attention (KDA)
    kda_layers: list[int] = field(default_factory=list)      # 1-based indices, as in the published configs; default: all but every 4th
    linear_heads: int = 4
    linear_head_dim: int = 16
    short_conv_kernel_size: int = 4
    use_full_rank_gate: bool = False
    gate_lower_bound: float | None = None
    kda_chunk_size: int = 16
    # latent attention
    q_lora_rank: int | None = None
    kv_lora_rank: int = 32
    qk_nope_head_dim: int = 16
    qk_rope_head_dim: int = 8
    v_head_dim: int = 16
    mla_use_output_gate: bool = False
    # feed-forward
    first_k_dense_replace: int = 1
    moe_layer_freq: int = 1
    num_shared_experts: int = 1
    num_expert_group: int = 1
    topk_group: int = 1
    moe_renormalize: bool = True
    routed_scaling_factor: float = 1.0
    moe_router_activation_func: str = "sigmoid"
    routed_expert_hidden_size: int | None = None
    latent_moe_use_norm: bool = True
    hidden_act: str = "silu"
    activation_situ_beta: float | None = None
    activation_situ_linear_beta: float | None = None
    attn_res_block_size: int | None = None
    model_type: str = "kimi_linear"

    def __post_init__(self):
        super().__post_init__()
        n = self.num_hidden_layers
        if not self.kda_layers:
            self.kda_layers = [i + 1 for i in range(n) if (i + 1) % 4 != 0]
        if self.moe_router_activation_func not in ("sigmoid", "softmax"):
            raise ValueError("Kimi moe_router_activation_func must be sigmoid or softmax")
        if self.hidden_act not in ("silu", "situ"):
            raise ValueError("Kimi hidden_act must be silu or situ")
        if self.attn_res_block_size is not None and (type(self.attn_res_block_size) is not int or self.attn_res_block_size <= 0):
            raise ValueError("attn_res_block_size must be a positive integer")
        if self.num_experts:
            g, tg, E, k = self.num_expert_group, self.topk_group, self.num_experts, self.num_experts_per_tok
            for name, v in (("num_experts", E), ("num_experts_per_tok", k), ("num_expert_group", g), ("topk_group", tg)):
                if type(v) is not int or v <= 0:
                    raise ValueError(f"Kimi {name} must be a positive integer")
            if E % g or not 1 <= tg <= g:
                raise ValueError("Kimi expert groups must divide num_experts and contain topk_group")
            if not 1 <= k <= E:
                raise ValueError("Kimi num_experts_per_tok must be in [1, num_experts]")
            if g > tg and (E // g < 2 or k > E // g * tg):
                raise ValueError("Kimi retained groups must contain top_k and two experts per group")
            if not math.isfinite(self.routed_scaling_factor):
                raise ValueError("Kimi routed_scaling_factor must be finite")
        self.router_score_fn = self.moe_router_activation_func
        self.route_scale = self.routed_scaling_factor

    def is_kda_layer(self, i: int) -> bool:
        return (i + 1) in self.kda_layers

    def is_moe_layer(self, i: int) -> bool:
        return bool(self.num_experts) and i >= self.first_k_dense_replace and i % max(1, self.moe_layer_freq) == 0


@dataclass
class KimiContext(ForwardContext):
    positions: torch.Tensor | None = None


# --------------------------------------------------------------------------------------------------- small pieces
class SituGLU(nn.Module):
    """Bounded gate beta·tanh(g/beta)·sigmoid(g), optionally bounded up projection; fp32 inside."""

    def __init__(self, beta: float = 1.0, linear_beta: float | None = None):
        super().__init__()
        if not math.isfinite(beta) or beta <= 0:
            raise ValueError("SituGLU beta must be finite and positive")
        if linear_beta is not None and (not math.isfinite(linear_beta) or linear_beta < 0):
            raise ValueError("SituGLU linear_beta must be finite and non-negative")
        self.beta, self.linear_beta = beta, linear_beta

    def forward(self, gate, up):
        g, u = gate.float(), up.float()
        a = self.beta * torch.tanh(g / self.beta) * torch.sigmoid(g)
        if self.linear_beta not in (None, 0.0):
            u = self.linear_beta * torch.tanh(u / self.linear_beta)
        return (a * u).to(gate.dtype)


def _glu(cfg: KimiConfig):
    if cfg.hidden_act != "situ":
        return None
    return SituGLU(1.0 if cfg.activation_situ_beta is None else cfg.activation_situ_beta, cfg.activation_situ_linear_beta)


class KimiMLP(GatedMLP):
    def __init__(self, cfg: KimiConfig, inter: int, dtype=None, device=None):
        super().__init__(cfg.hidden_size, inter, dtype, device)
        self.glu = _glu(cfg)

    accepts_sharded_rows = False

    def forward(self, x):
        if self.glu is None:
            return super().forward(x)
        return self.down_proj(self.glu(self.gate_proj(x), self.up_proj(x)))


class CausalConvolution(nn.Module):
    """Depthwise causal convolution + SiLU over packed rows; `weight` [channels, 1, kernel] with the LAST tap on the
    current token. A tap that would reach before the first token of the row's document contributes nothing."""

    def __init__(self, channels: int, kernel: int, dtype=None, device=None):
        super().__init__()
        self.kernel = kernel
        self.weight = nn.Parameter(torch.empty(channels, 1, kernel, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor, positions: torch.Tensor, halo: torch.Tensor | None = None) -> torch.Tensor:
        """x [T, C]; positions [T]: index of each row inside its document. `halo` [B, K-1, C]: under sequence
        parallelism the rows that precede each of the B local spans on the rank before (the position mask still decides
        whether a tap may use them)."""
        K = self.kernel
        w = self.weight[:, 0, :].to(x.dtype)                       # [C, K]
        T, C = x.shape
        out = x * w[:, K - 1]
        if halo is not None:
            B = halo.shape[0]
            ext = torch.cat((halo.to(x.dtype), x.view(B, T // B, C)), 1)           # [B, K-1 + t, C]
        for j in range(1, K):
            if halo is not None:
                shifted = ext[:, K - 1 - j: K - 1 - j + T // B].reshape(T, C)
            else:
                shifted = F.pad(x[:-j], (0, 0, j, 0)) if T > j else torch.zeros_like(x)
            out = out + shifted * (positions >= j).to(x.dtype)[:, None] * w[:, K - 1 - j]
        return F.silu(out)


def attention_residual(prefix: torch.Tensor, blocks: torch.Tensor, proj_w: torch.Tensor, norm_w: torch.Tensor, eps: float):
    """prefix [T, D] (running sum), blocks [T, n, D] (filed residuals) -> per-token softmax mixture of the n + 1
    candidates. Scores come from the RMS-normalised candidates; the mixture uses them at their own magnitude."""
    vals = torch.cat((blocks, prefix.unsqueeze(1)), 1).float()
    normed = vals * torch.rsqrt(vals.square().mean(-1, keepdim=True) + eps)
    p = (normed * (norm_w.float() * proj_w.reshape(-1).float())).sum(-1).softmax(-1)
    return (p.unsqueeze(1) @ vals).squeeze(1).to(prefix.dtype)


# --------------------------------------------------------------------------------------------------- mixers
class KimiDeltaAttention(nn.Module):
    def __init__(self, cfg: KimiConfig, dtype=None, device=None):
        super().__init__()
        D, H, d = cfg.hidden_size, cfg.linear_heads, cfg.linear_head_dim
        self.H, self.d, self.chunk, self.lower = H, d, cfg.kda_chunk_size, cfg.gate_lower_bound
        W = H * d
        for n in ("q", "k", "v"):
            setattr(self, f"{n}_proj", Linear(D, W, dtype, device))
            setattr(self, f"{n}_conv1d", CausalConvolution(W, cfg.short_conv_kernel_size, dtype, device))
        self.f_a_proj, self.f_b_proj = Linear(D, d, dtype, device), Linear(d, W, dtype, device)
        self.b_proj = Linear(D, H, dtype, device)
        self.A_log = nn.Parameter(torch.empty(H, dtype=torch.float32, device=device))
        self.dt_bias = nn.Parameter(torch.zeros(W, dtype=torch.float32, device=device))
        self.full_gate = cfg.use_full_rank_gate
        if self.full_gate:
            self.g_proj = Linear(D, W, dtype, device)
        else:
            self.g_a_proj, self.g_b_proj = Linear(D, d, dtype, device), Linear(d, W, dtype, device)
        self.o_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.o_proj = Linear(W, D, dtype, device)
        self.eps = cfg.rms_norm_eps
        if self.lower is not None and not -5 <= self.lower < 0:
            raise ValueError(f"KDA gate lower bound must be in [-5, 0); got {self.lower}")

    def log_decay(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        raw = self.f_b_proj(self.f_a_proj(x)).float().view(T, self.H, self.d) + self.dt_bias.float().view(self.H, self.d)
        rate = self.A_log.float().exp().view(1, self.H, 1)
        if self.lower is not None:
            return self.lower * torch.sigmoid(rate * raw)
        return -rate * F.softplus(raw)

    def forward(self, x: torch.Tensor, ctx: KimiContext) -> torch.Tensor:
        T, H, d = x.shape[0], self.H, self.d
        cp = ctx.cp if ctx.cp is not None and getattr(ctx.cp, "size", 1) > 1 else None
        pos = ctx.positions
        proj = [getattr(self, f"{n}_proj")(x) for n in ("q", "k", "v")]
        halos = (None, None, None)
        if cp is not None:                  # one exchange for the three convolutions: the rows before this rank's spans
            halos = cp.prev_rows(torch.cat(proj, -1), self.q_conv1d.kernel - 1).split(H * d, dim=-1)
        q, k, v = (getattr(self, f"{n}_conv1d")(y, pos, h).view(T, H, d).float() for n, y, h in zip(("q", "k", "v"), proj, halos))
        q = q * torch.rsqrt(q.square().sum(-1, keepdim=True) + 1e-6) * d ** -0.5
        k = k * torch.rsqrt(k.square().sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(self.b_proj(x).float())
        ld = self.log_decay(x)
        if cp is not None:
            o = cp.delta_rule(q, k, v, beta, ld, self.chunk)                               # state handed from rank to rank
        else:
            outs = [chunked_delta_rule(q[a:a + n], k[a:a + n], v[a:a + n], beta[a:a + n], ld[a:a + n], self.chunk)
                    for a, n in ((int(p[0]), int(p[1])) for p in ctx.attn_meta.pieces)]
            o = (torch.cat(outs) if len(outs) > 1 else outs[0])                            # [T, H, d] fp32
        gate = (self.g_proj(x) if self.full_gate else self.g_b_proj(self.g_a_proj(x))).view(T, H, d)
        o = o * torch.rsqrt(o.square().mean(-1, keepdim=True) + self.eps) * self.o_norm.weight.float() * torch.sigmoid(gate.float())
        return self.o_proj(o.to(x.dtype).reshape(T, H * d))


class KimiLatentAttention(nn.Module):
    def __init__(self, cfg: KimiConfig, dtype=None, device=None):
        super().__init__()
        D, H = cfg.hidden_size, cfg.num_attention_heads
        self.H, self.dn, self.dr, self.dv = H, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.dq = self.dn + self.dr
        self.scale = self.dq ** -0.5
        self.q_lora = cfg.q_lora_rank
        if self.q_lora is not None:
            self.q_a_proj = Linear(D, self.q_lora, dtype, device)
            self.q_a_layernorm = RMSNorm(self.q_lora, 1e-6, dtype, device)
            self.q_b_proj = Linear(self.q_lora, H * self.dq, dtype, device)
        else:
            self.q_proj = Linear(D, H * self.dq, dtype, device)
        self.kv_a_proj_with_mqa = Linear(D, cfg.kv_lora_rank + self.dr, dtype, device)
        self.kv_a_layernorm = RMSNorm(cfg.kv_lora_rank, 1e-6, dtype, device)
        self.kv_b_proj = Linear(cfg.kv_lora_rank, H * (self.dn + self.dv), dtype, device)
        self.o_proj = Linear(H * self.dv, D, dtype, device)
        self.g_proj = Linear(D, H * self.dv, dtype, device) if cfg.mla_use_output_gate else None
        self.rank = cfg.kv_lora_rank

    def forward(self, x: torch.Tensor, ctx: KimiContext) -> torch.Tensor:
        T, H = x.shape[0], self.H
        qs = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x))) if self.q_lora is not None else self.q_proj(x)
        q = qs.view(T, H, self.dq)
        ckv = self.kv_a_proj_with_mqa(x)
        kv = self.kv_b_proj(self.kv_a_layernorm(ckv[:, :self.rank])).view(T, H, self.dn + self.dv)
        k = torch.cat((kv[..., :self.dn], ckv[:, None, self.rank:].expand(T, H, self.dr)), -1)      # no rotary: positions come from the KDA layers
        v = kv[..., self.dn:]
        if ctx.cp is not None:                    # the exchange moves q, k and v as one head-sharded block: one width
            vv = v if self.dv == self.dq else F.pad(v, (0, self.dq - self.dv))
            o = ctx.cp.attention(q.contiguous(), k.contiguous(), vv.contiguous(), ctx.attn_meta, self.scale)[..., :self.dv]
        else:                                     # widths without a kernel variant (192 / 128 here) are padded inside
            o = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), ctx.attn_meta, self.scale)
        o = o.reshape(T, H * self.dv)
        if self.g_proj is not None:
            o = o * torch.sigmoid(self.g_proj(x))
        return self.o_proj(o)


class KimiMoE(MoE):
    """The shared sparse block plus Kimi's latent expert space."""

    def __init__(self, cfg: KimiConfig, dtype=None, device=None):
        width = cfg.routed_expert_hidden_size
        grouped = cfg.num_expert_group > cfg.topk_group
        super().__init__(cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                         shared_inter=cfg.moe_intermediate_size * cfg.num_shared_experts, score_fn=cfg.moe_router_activation_func,
                         norm_topk_prob=cfg.moe_renormalize and cfg.num_experts_per_tok > 1, route_scale=cfg.routed_scaling_factor,
                         bias_update_coeff=cfg.router_bias_update_coeff, aux_loss_coef=cfg.router_aux_loss_coef,
                         experts_implementation=cfg.experts_implementation, dtype=dtype, device=device,
                         shared_mlp_factory=lambda inter: KimiMLP(cfg, inter, dtype, device),
                         num_groups=cfg.num_expert_group if grouped else 1, topk_groups=cfg.topk_group if grouped else 1,
                         expert_width=width, glu_fn=_glu(cfg))
        self.always_bias = True            # the correction bias takes part in the selection whether or not it is being updated
        if width is not None:
            self.routed_expert_down_proj = Linear(cfg.hidden_size, width, dtype, device)
            self.routed_expert_up_proj = Linear(width, cfg.hidden_size, dtype, device)
            self.routed_expert_norm = RMSNorm(width, cfg.rms_norm_eps, dtype, device) if cfg.latent_moe_use_norm else None
        self.latent = width is not None

    def routed_input(self, x2):
        return self.routed_expert_down_proj(x2) if self.latent else x2

    def routed_output(self, y):
        if not self.latent:
            return y
        if self.routed_expert_norm is not None:
            y = self.routed_expert_norm(y)
        return self.routed_expert_up_proj(y)


# --------------------------------------------------------------------------------------------------- layer, model
class KimiDecoderLayer(nn.Module):
    def __init__(self, cfg: KimiConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx, self.block = layer_idx, cfg.attn_res_block_size
        D, eps = cfg.hidden_size, cfg.rms_norm_eps
        if self.block is not None:
            for n in ("self_attention_res", "mlp_res"):
                setattr(self, f"{n}_norm", RMSNorm(D, eps, dtype, device))
                setattr(self, f"{n}_proj", Linear(D, 1, dtype, device))
        self.is_linear_attn = cfg.is_kda_layer(layer_idx)
        self.self_attn = (KimiDeltaAttention if self.is_linear_attn else KimiLatentAttention)(cfg, dtype, device)
        self.is_sparse = cfg.is_moe_layer(layer_idx)
        self.mlp = KimiMoE(cfg, dtype, device) if self.is_sparse else KimiMLP(cfg, cfg.intermediate_size, dtype, device)
        self.input_layernorm = RMSNorm(D, eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(D, eps, dtype, device)
        self.eps = eps

    def forward(self, state: torch.Tensor, ctx: KimiContext) -> torch.Tensor:
        """Without attention residuals `state` is the hidden rows [T, D]. With them it is [T, 1 + n, D]: the running
        hidden rows followed by the n blocks filed so far (one tensor, so that block runners and recompute wrappers that
        pass a single activation through a layer keep working)."""
        if self.block is None:
            h = state + self.self_attn(self.input_layernorm(state), ctx)
            return h + self.mlp(self.post_attention_layernorm(h))
        prefix, blocks = state[:, 0], state[:, 1:]
        h = prefix
        if blocks.shape[1]:
            h = attention_residual(prefix, blocks, self.self_attention_res_proj.weight, self.self_attention_res_norm.weight, self.eps)
        if self.layer_idx % self.block == 0:                 # file the running sum as a block and start a new one
            blocks = torch.cat((blocks, prefix.unsqueeze(1)), 1)
            prefix = None
        a = self.self_attn(self.input_layernorm(h), ctx)
        prefix = a if prefix is None else prefix + a
        h = attention_residual(prefix, blocks, self.mlp_res_proj.weight, self.mlp_res_norm.weight, self.eps)
        out = prefix + self.mlp(self.post_attention_layernorm(h))
        return torch.cat((out.unsqueeze(1), blocks), 1)


class KimiForCausalLM(Qwen3ForCausalLM):
    decoder_structure = DecoderStructure()
    positions_are_document_indices = True      # no rotary anywhere: positions only tell where documents restart

    def __init__(self, cfg: KimiConfig, dtype=None, device=None):
        nn.Module.__init__(self)
        self.config = cfg
        self.model = Qwen3Model.__new__(Qwen3Model)
        nn.Module.__init__(self.model)
        if cfg.attn_res_block_size is not None:
            self.model.output_attn_res_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
            self.model.output_attn_res_proj = Linear(cfg.hidden_size, 1, dtype, device)
        self.model.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.model.layers = nn.ModuleList(KimiDecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers))
        self.model.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype, device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.activation_checkpoint, self.ac_save_every, self.block_runner = "none", 2, None
        self.pp_first = self.pp_last = True

    @torch.no_grad()
    def initialize_parameters(self, seed: int | None = None) -> None:
        super().initialize_parameters(seed)
        gen = torch.Generator().manual_seed((seed or 0) * 7919 + 13)
        for m in self.modules():
            if isinstance(m, KimiDeltaAttention) and not m.A_log.is_meta:
                m.A_log.copy_(torch.empty(m.H).uniform_(1, 16, generator=gen).log())       # decay rates spread over 1..16
                m.dt_bias.zero_()
            elif isinstance(m, CausalConvolution) and not m.weight.is_meta:
                bound = 1.0 / math.sqrt(m.kernel)
                m.weight.copy_(torch.empty(m.weight.shape).uniform_(-bound, bound, generator=gen))

    def tp_config(self) -> dict[str, str]:
        return {}

    def validate_parallel(self, tp: int = 1, cp_ulysses: int = 1, ep: int = 1) -> None:
        from ..errors import UnsupportedCombinationError
        if tp > 1 or cp_ulysses > 1:
            raise UnsupportedCombinationError("kimi: tensor and Ulysses parallelism are defined for the Qwen3 family; use data, expert "
                                              "and FSDP parallelism")
        if self.config.num_experts and self.config.num_experts % ep:
            raise UnsupportedCombinationError(f"expert_parallel_size {ep} must divide num_experts {self.config.num_experts}")

    def build_context(self, positions, attn_meta, cp=None) -> KimiContext:
        z = positions.new_zeros(0)
        return KimiContext(z, z, attn_meta, cp, positions=positions)

    def forward(self, tokens, ctx, skip_lm_head: bool = False, inputs_embeds=None):
        x = inputs_embeds if inputs_embeds is not None else (self.model.embed_tokens(tokens) if self.pp_first else tokens)
        res = self.config.attn_res_block_size is not None
        if res and self.pp_first:
            x = x.unsqueeze(1)                                  # [T, 1 + 0 blocks, D]
        for i, layer in enumerate(self.model.layers):
            x = self.run_block(getattr(layer, "layer_idx", i), layer, x, ctx)
        if not self.pp_last:
            return x
        if res:
            x = attention_residual(x[:, 0], x[:, 1:], self.model.output_attn_res_proj.weight, self.model.output_attn_res_norm.weight,
                                   self.config.rms_norm_eps)
        h = self.model.norm(x)
        return h if skip_lm_head else self.lm_head(h)


def build_kimi(defaults: dict):
    def build(model_config, dtype=None, device=None, **overrides):
        kw = dict(vocab_size=model_config.vocab_size, hidden_size=model_config.hidden_size, intermediate_size=model_config.intermediate_size,
                  num_hidden_layers=model_config.num_hidden_layers, num_attention_heads=model_config.num_attention_heads,
                  num_key_value_heads=model_config.num_attention_heads, experts_implementation=model_config.experts_implementation)
        kw.update(defaults)
        kw.update(model_config.arch_overrides or {})
        kw.update(overrides)
        names = set(KimiConfig.__dataclass_fields__)
        return KimiForCausalLM(KimiConfig(**{k: v for k, v in kw.items() if k in names}), dtype=dtype, device=device)
    return build


KIMI_LINEAR_DEFAULTS = dict(model_type="kimi_linear", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                            first_k_dense_replace=1, router_bias_update_coeff=1e-3)
KIMI_K3_DEFAULTS = dict(KIMI_LINEAR_DEFAULTS, model_type="kimi_k3", attn_res_block_size=2, hidden_act="situ", activation_situ_beta=4.0,
                        routed_expert_hidden_size=32, mla_use_output_gate=True, num_expert_group=4, topk_group=2)


def build_kimi_vl(defaults: dict):
    """Kimi-K3 with its vision tower (MoonViT): `arch_overrides` may carry `image_token_id` (default: the last token) and
    `vision` (fields of `MoonViTConfig`; the output width follows the text width). Text positions stay one-dimensional."""
    text_builder = build_kimi(defaults)

    def build(model_config, dtype=None, device=None, **overrides):
        from .moonvit import MoonViTConfig, MoonViTTower
        from .vision import VisionLanguageModel
        text = text_builder(model_config, dtype=dtype, device=device, **overrides)
        extra = dict(model_config.arch_overrides or {})
        vkw = dict(extra.get("vision") or {})
        vkw["out_hidden_size"] = text.config.hidden_size
        image_id = int(extra.get("image_token_id", text.config.vocab_size - 1))
        return VisionLanguageModel(text, MoonViTConfig(**vkw), image_id, dtype=dtype, device=device, tower=MoonViTTower)
    return build
