"""Further model families behind the same registry and contracts as Qwen3
(reference: llmtuner/models/qwen/qwen3_5*, llmtuner/models/deepseek/deepseek_v4/*, llmtuner/models/kimi/kimi_k3/*).

They share one hybrid decoder: every layer has a token mixer and an MLP (dense or the shared MoE block).
  hybrid_gdn / hybrid_gdn_moe                3 of 4 layers use a gated delta-net linear attention, every 4th layer a
                                             softmax attention with an output gate; gated RMSNorm on the mixer output
(Qwen3.5 has its own module, `models/qwen3_5.py`.)
  hybrid_kda_mla                             KDA (delta rule with per-channel decay) layers with an MLA (latent
                                             attention) layer every 4th; sigmoid router with shared experts
(Kimi-Linear / Kimi-K3 have their own module, `models/kimi_k3.py`.)
(DeepSeek-V4 has its own module, `models/deepseek_v4.py`.)
Softmax attention and every GEMM run on the sm_100a kernels; the delta rule runs in chunk-parallel form (batched matrix
products and one triangular solve per layer, a short loop over chunks for the state; per document). The vision tower,
the 3-axis rotary positions and the wrapper that splices image rows into these decoders are in `models/vision.py`.
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
    delta_chunk_size: int = 0                  # tokens per chunk of the chunk-parallel delta rule; 0: 64 (per-head decay) / 16 (KDA)
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


def delta_rule_scan(q, k, v, beta, log_decay):
    """Token-by-token statement of the gated delta rule, zero initial state (the oracle of `chunked_delta_rule`).
    q, k [T, H, dk]; v [T, H, dv]; beta [T, H]; log_decay [T, H, dk] or [T, H, 1] (<= 0). Returns [T, H, dv]."""
    T, H, dk = q.shape
    S = q.new_zeros(H, dk, v.shape[-1])
    dec = log_decay.exp().expand(T, H, dk)
    outs = []
    for t in range(T):
        S = S * dec[t].unsqueeze(-1)
        pred = torch.einsum("hkv,hk->hv", S, k[t])
        S = S + torch.einsum("hk,hv->hkv", k[t], beta[t].unsqueeze(-1) * (v[t] - pred))
        outs.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(outs)


def chunked_delta_rule(q, k, v, beta, log_decay, chunk: int = 64, initial_state=None, return_state: bool = False):
    """The same recurrence in chunk-parallel form (`initial_state` [H, dk, dv] instead of zero; `return_state` also
    returns the state after the last token). The value columns evolve independently of each other, which sequence
    parallelism uses: extra value columns that start as an identity come back as the segment's transition matrix.
     Inside a chunk of C tokens that starts from state S0, with the
    cumulative log decay G_t, the pseudo-values u_t = beta_t (v_t - S'_t^T k_t) solve the triangular system
        (I + A) U = beta (V - K~ S0),   A[t, i] = beta_t sum_c k_t[c] k_i[c] exp(G_t[c] - G_i[c])   (i < t),
    with K~_t = exp(G_t) k_t; then O = Q~ S0 + tril(QK) U and S_end = exp(G_C) S0 + (exp(G_C - G) K)^T U.
    Everything that does not depend on S0 is computed for all chunks at once (batched matrix products and one batched
    triangular solve); only the [dk, dv] state update runs chunk after chunk. Decay ratios are only ever formed as
    exp(G_t - G_i) with i <= t, so nothing overflows however strong the decay."""
    T, H, dk = q.shape
    dv, C = v.shape[-1], chunk
    pad = (-T) % C
    if pad:                                           # padded tokens: beta = 0, k = 0, decay 1 -> no effect on the state
        z = lambda t: F.pad(t, (0, 0, 0, 0, 0, pad))  # noqa: E731
        q, k, v, log_decay = z(q), z(k), z(v), z(log_decay)
        beta = F.pad(beta, (0, 0, 0, pad))
    N = (T + pad) // C
    r = lambda t: t.reshape(N, C, H, -1).permute(0, 2, 1, 3)  # noqa: E731  -> [N, H, C, *]
    q, k, v, beta, G = r(q), r(k), r(v), r(beta.unsqueeze(-1)), r(log_decay).cumsum(2)
    tri = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    if G.shape[-1] == 1:                              # one decay per head: the ratio matrix factors out of the products
        M = (G - G.transpose(2, 3)).clamp(max=0).exp()
        KK, QK = (k @ k.transpose(2, 3)) * M, (q @ k.transpose(2, 3)) * M
    else:                                             # a decay per key channel: pairwise ratios, in slabs of chunks
        KK, QK = [], []
        slab = max(1, (1 << 25) // (H * C * C * dk))
        for a in range(0, N, slab):
            g = G[a:a + slab]
            Ek = (g.unsqueeze(3) - g.unsqueeze(2)).clamp(max=0).exp() * k[a:a + slab].unsqueeze(2)      # [n, H, t, i, dk]
            # k_t and q_t against the same decayed keys: one batched [2, dk] x [dk, C] product per (chunk, head, t)
            both = torch.stack((k[a:a + slab], q[a:a + slab]), 3) @ Ek.transpose(-1, -2)                # [n, H, t, 2, i]
            KK.append(both[..., 0, :])
            QK.append(both[..., 1, :])
        KK, QK = torch.cat(KK), torch.cat(QK)
    A = (beta * KK).masked_fill(~tri.tril(-1), 0.0)
    QK = QK.masked_fill(~tri, 0.0)
    eG = G.exp()
    IA = A + torch.eye(C, dtype=q.dtype, device=q.device)
    # (I + A)^-1 by forward substitution against the identity (C columns), then one product with the dv + dk right-hand
    # sides: the substitution is the slow part on the device and this way it runs on a quarter of the columns
    inv = torch.linalg.solve_triangular(IA, torch.eye(C, dtype=q.dtype, device=q.device).expand_as(IA), upper=False)
    W = inv @ torch.cat((beta * v, beta * eG * k), -1)
    W1, W2 = W.split((dv, W.shape[-1] - dv), -1)
    Qt = eG * q
    Kend = (G[:, :, -1:, :] - G).exp() * k
    dec_end = G[:, :, -1, :].exp().unsqueeze(-1)                              # [N, H, dk | 1, 1]
    S = q.new_zeros(H, dk, dv) if initial_state is None else initial_state
    if N <= SEQUENTIAL_CHUNKS:
        outs = []
        for n in range(N):
            U = W1[n] - W2[n] @ S
            outs.append(Qt[n] @ S + QK[n] @ U)
            S = dec_end[n] * S + Kend[n].transpose(1, 2) @ U
        o = torch.stack(outs)
    else:
        # The state update is affine in the state: S_{n+1} = A_n S_n + B_n with A_n = diag(decay_n) - Kend_n^T W2_n and
        # B_n = Kend_n^T W1_n, both known for every chunk at once. A two-level scan over those maps leaves about
        # 2 sqrt(N) dependent steps instead of N, and every output product becomes one batched product over all chunks.
        # Blocks of chunks bound the [chunks, H, dk, dk] maps (and what autograd keeps of them); the state carries over.
        blk = max(SEQUENTIAL_CHUNKS + 1, SCAN_BLOCK_BYTES // (H * dk * dk * q.element_size()))
        outs = []
        for w1, w2, qt, qk, kend, dec in zip(*(t.split(blk) for t in (W1, W2, Qt, QK, Kend, dec_end))):
            kendT = kend.transpose(2, 3)
            A = (-kendT) @ w2
            A.diagonal(dim1=-2, dim2=-1).add_(dec.squeeze(-1).expand(A.shape[0], H, dk))
            S_all, S = affine_scan(A, kendT @ w1, S)
            outs.append(qt @ S_all + qk @ (w1 - w2 @ S_all))
        o = torch.cat(outs) if len(outs) > 1 else outs[0]
    o = o.permute(0, 2, 1, 3).reshape(N * C, H, dv)
    return (o[:T], S) if return_state else o[:T]


SEQUENTIAL_CHUNKS = 8       # up to this many chunks the plain chunk-after-chunk loop is the cheaper form
SCAN_BLOCK_BYTES = 1 << 29  # size of the state-transition maps of one scan block


def affine_scan(A, B, S0):
    """States of S_{n+1} = A_n S_n + B_n for n = 0..N-1. A [N, H, a, a], B [N, H, a, b], S0 [H, a, b].
    Returns (the state each step starts from [N, H, a, b], the state after the last step [H, a, b]).
    Two levels: the N steps are cut into groups of about sqrt(N); inside all groups at once the prefix maps
    (P_j, Q_j) with S_{g, j} = P_j S_g + Q_j are built step by step (batched over groups), then the group-start states
    follow group after group, then every state comes from one batched product. Steps that pad the last group are the
    identity map."""
    N, H, a, _ = A.shape
    R = max(1, int(math.isqrt(N)))
    M = -(-N // R)
    if M * R != N:
        eye = torch.eye(a, dtype=A.dtype, device=A.device).expand(M * R - N, H, a, a)
        A = torch.cat((A, eye))
        B = torch.cat((B, B.new_zeros(M * R - N, *B.shape[1:])))
    # unbind, not indexing: the backward of an index is a zero-filled tensor of the whole size per step
    Aj, Bj = A.view(M, R, *A.shape[1:]).unbind(1), B.view(M, R, *B.shape[1:]).unbind(1)
    P, Q = [Aj[0]], [Bj[0]]                                       # the maps after 1, 2, ... R steps of a group
    for j in range(1, R):
        P.append(Aj[j] @ P[-1])
        Q.append(Aj[j] @ Q[-1] + Bj[j])
    starts = [S0]
    for Pg, Qg in zip(P[-1].unbind(0), Q[-1].unbind(0)):
        starts.append(Pg @ starts[-1] + Qg)
    Sg = torch.stack(starts[:-1]).unsqueeze(1)                    # [M, 1, H, a, b]
    inner = torch.stack(P[:-1], 1) @ Sg + torch.stack(Q[:-1], 1) if R > 1 else None      # after 1 .. R-1 steps
    S_all = Sg if inner is None else torch.cat((Sg, inner), 1)
    return S_all.reshape(M * R, *S_all.shape[2:])[:N], starts[-1]


class DeltaRuleMixer(nn.Module):
    """Gated delta rule: S_t = a_t * S_{t-1} (I - b_t k_t k_t^T) + b_t k_t v_t^T ; o_t = S_t^T q_t, per head, state reset
    at document starts. `channel_decay` makes a_t a vector over the key dimension (KDA)."""

    # tensor parallelism cuts every projection by heads; the output norm (over head_dim) stays replicated
    tp_cut = {"colwise": ("q_proj", "k_proj", "v_proj", "beta_proj", "decay_proj", "gate_proj"), "rowwise": ("o_proj",), "heads": ("H",)}

    def __init__(self, cfg: HybridConfig, dtype=None, device=None):
        super().__init__()
        D, H, d = cfg.hidden_size, cfg.delta_heads, cfg.delta_head_dim
        self.H, self.d, self.channel = H, d, cfg.delta_channel_decay
        self.chunk = cfg.delta_chunk_size or (16 if self.channel else 64)
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
        log_decay = -F.softplus(self.decay_proj(x).float()).view(T, H, d if self.channel else 1)
        if ctx.cp is not None and ctx.cp.size > 1:
            o = ctx.cp.delta_rule(q, k, v, beta, log_decay, self.chunk).to(x.dtype)       # state handed from rank to rank
        else:
            cuts = sorted({0, T} | {int(i) for i in _doc_starts(ctx.attn_meta, T, "cpu").nonzero().flatten().tolist()})
            outs = [chunked_delta_rule(q[a:b], k[a:b], v[a:b], beta[a:b], log_decay[a:b], self.chunk)
                    for a, b in zip(cuts[:-1], cuts[1:])]                                 # the state starts at zero per document
            o = torch.cat(outs).to(x.dtype)                                               # [T, H, d]
        o = self.out_norm(o.reshape(T * H, d)).view(T, H * d) * F.silu(self.gate_proj(x))  # gated RMSNorm
        return self.o_proj(o)


class GatedAttention(Qwen3Attention):
    """Softmax attention whose output is multiplied by sigmoid(W_g x) before the output projection."""
    accepts_sharded_rows = False    # the gate reads the complete rows too
    tp_cut = {"colwise": ("q_proj", "k_proj", "v_proj", "gate"), "rowwise": ("o_proj",), "heads": ("num_heads", "num_kv_heads")}

    def __init__(self, cfg: HybridConfig, dtype=None, device=None):
        super().__init__(cfg, dtype, device)
        self.gate = Linear(cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, dtype, device) if cfg.attention_output_gate else None

    def forward(self, x, ctx):
        q, k, v = self.project_qkv(x)
        q, k = ops.qk_norm_rope(q, k, self.q_norm.weight if self.q_norm is not None else None,
                                self.k_norm.weight if self.k_norm is not None else None, ctx.cos, ctx.sin, self.eps)
        attend = ctx.cp.attention if ctx.cp is not None else ops.attention
        o = attend(q, k, v, ctx.attn_meta, self.scale).reshape(x.shape[0], -1)
        if self.gate is not None:
            o = o * torch.sigmoid(self.gate(x))
        return self.o_proj(o)


class LatentAttention(nn.Module):
    """Multi-head latent attention: keys and values are up-projected from a shared low-rank latent; a small rotary key
    shared by all heads is concatenated to the per-head non-rotary key."""
    # tensor parallelism: per-head projections are cut, the latent down-projection, its norm and the rotary key stay whole
    tp_cut = {"colwise": ("q_proj", "k_up", "v_up"), "rowwise": ("o_proj",), "heads": ("H",)}

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
        attend = ctx.cp.attention if ctx.cp is not None else ops.attention
        o = attend(q.contiguous(), k.contiguous(), v.contiguous(), ctx.attn_meta, self.scale)
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
        c = self.config
        if cp_ulysses > 1:
            raise UnsupportedCombinationError(f"{c.model_type}: Ulysses context parallelism is defined for the Qwen3 family only (the "
                                              "delta-rule layers hand their state from rank to rank: context_parallel_kcp_size / "
                                              "context_parallel_kv_allgather_size)")
        kinds = {c.mixer_pattern[i % len(c.mixer_pattern)] for i in range(c.num_hidden_layers)}
        if tp > 1 and kinds & {"delta", "kda"} and c.delta_heads % tp:
            raise UnsupportedCombinationError(f"tensor_parallel_size {tp} must divide delta_heads {c.delta_heads}")
        if tp > 1 and "mla" in kinds and c.num_attention_heads % tp:
            raise UnsupportedCombinationError(f"tensor_parallel_size {tp} must divide num_attention_heads {c.num_attention_heads}")
        super().validate_parallel(tp if "attention" in kinds else 1, 1, ep)

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
    # gated delta-net layers with a gated softmax attention every 4th, on the generic hybrid decoder: the carrier of the
    # tensor-parallel cuts of these mixers (the faithful Qwen3.5 decoder is models/qwen3_5.py)
    "hybrid_gdn": dict(model_type="hybrid_gdn", mixer_pattern=["delta", "delta", "delta", "attention"]),
    "hybrid_gdn_moe": dict(model_type="hybrid_gdn_moe", mixer_pattern=["delta", "delta", "delta", "attention"], num_experts=8,
                           num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64),
    # KDA layers with a latent-attention layer every 4th, on the generic hybrid decoder: the carrier of the tensor-parallel
    # cuts of these mixers (the faithful Kimi decoder is models/kimi_k3.py and, like the reference's, declares no TP plan)
    "hybrid_kda_mla": dict(model_type="hybrid_kda_mla", mixer_pattern=["kda", "kda", "kda", "mla"], delta_channel_decay=True, num_experts=8,
                           num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=64, router_score_fn="sigmoid",
                           mlp_only_layers=[0]),
}


def register_all(reg) -> None:
    for name, defaults in FAMILIES.items():
        reg(name, _builder(defaults), state_format="native", supports={"fsdp", "ep", "ac"},
            description=f"{name} text decoder (hybrid mixer family)")
