"""DeepSeek-V4 decoder (reference: llmtuner/models/deepseek/deepseek_v4/modeling.py:69-791, attention.py:17-280,
compression.py:18-156, compression_math.py:10-111, overlap.py:6-25, indexer.py:18-115, routing.py:12-85,
hyperconnection.py:13-79, rotary.py:9-100, normalization.py:8-38).

What makes the family:
  * several residual STREAMS per token (`hc_mult`): before each sub-layer a hyper-connection collapses them to one input
    (sigmoid read weights), after it the output is written back with per-stream gains and the streams are mixed by a
    doubly-normalised (Sinkhorn) matrix; a hyper-head collapses the streams before the final norm;
  * attention with ONE shared key/value head whose values are the keys: low-rank query (`q_a` -> norm -> `q_b`, an
    unweighted RMS norm per head), interleaved-pair rotary on the trailing `qk_rope_head_dim` channels, a learned sink
    logit per head, rotary UNDONE on the output at the query position, grouped low-rank output projection;
  * three layer types by what the keys are: "sliding_attention" (the last `sliding_window` tokens),
    "heavily_compressed_attention" (the window plus one entry per `rate` tokens: a softmax-gated pool of the window's
    projections) and "compressed_sparse_attention" (entries pooled over two overlapping windows, of which each query
    sees only the `index_topk` that a small indexer scores highest). An entry is visible once its window is complete;
  * MoE with a selection bias (top-k on scores + bias, weights from the plain scores, `routed_scaling_factor`), or, in
    "hash_moe" layers, experts looked up in a token-id table; clamped SwiGLU; one shared expert.

Rows are packed `[T, D]`, streams `[T, n, D]`; documents come from `AttnMeta.pieces`, so windows, entries and positions
restart at every document. Sequence parallelism (reference: llmtuner/parallel/context_parallel/compressor_attention.py:39-371,
compression_windows.py exchanges windows and runs a Ulysses exchange over the query heads) takes another route here: the
key/value stream is ONE head and the compressor inputs are a few head-widths per token, so they are gathered over the
sequence ranks (a few MB at 128k tokens) and every rank pools all windows itself; queries, the H-head products and
the hyper-connection streams stay local to the rank's span. The window/entry attention is evaluated densely in query
chunks (fp32 softmax); every projection is a `Linear` of this framework and therefore a tcgen05 GEMM on the device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from .common import Embedding, GatedMLP, Linear, RMSNorm
from .contracts import DecoderStructure
from .moe import MoE
from .qwen3 import ForwardContext, Qwen3Config, Qwen3ForCausalLM, Qwen3Model

ATTENTION_TYPES = ("sliding_attention", "compressed_sparse_attention", "heavily_compressed_attention")
MLP_TYPES = ("hash_moe", "moe")


@dataclass
class DeepseekV4Config(Qwen3Config):
    q_lora_rank: int = 32
    o_groups: int = 2
    o_lora_rank: int = 16
    qk_rope_head_dim: int = 8
    sliding_window: int = 16
    layer_types: list[str] = field(default_factory=list)          # per layer; default cycles sliding / CSA / HCA
    mlp_layer_types: list[str] = field(default_factory=list)      # per layer; default hash_moe for layer 0, then moe
    compress_rates: dict = field(default_factory=lambda: {"compressed_sparse_attention": 4, "heavily_compressed_attention": 8})
    index_n_heads: int = 2
    index_head_dim: int = 16
    index_topk: int = 4
    hc_mult: int = 2
    hc_sinkhorn_iters: int = 3
    hc_eps: float = 1e-6
    scoring_func: str = "sqrtsoftplus"
    routed_scaling_factor: float = 1.5
    swiglu_limit: float = 7.0
    compress_rope_theta: float = 160_000.0
    model_type: str = "deepseek_v4"

    def __post_init__(self):
        super().__post_init__()
        n = self.num_hidden_layers
        if not self.layer_types:
            self.layer_types = [ATTENTION_TYPES[i % 3] for i in range(n)]
        if not self.mlp_layer_types:
            self.mlp_layer_types = ["hash_moe" if i == 0 else "moe" for i in range(n)]
        validate_layer_schedule(self)
        for name in ("num_attention_heads", "head_dim", "o_groups", "o_lora_rank", "q_lora_rank"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError(f"DeepSeek-V4 {name} must be a positive integer")
        if self.num_attention_heads * self.head_dim % self.o_groups:
            raise ValueError("DeepSeek-V4 attention width must be divisible by o_groups")
        if self.qk_rope_head_dim % 2 or self.qk_rope_head_dim > min(self.head_dim, self.index_head_dim):
            raise ValueError("qk_rope_head_dim must be even and fit into head_dim and index_head_dim")
        if self.num_experts <= 0 or not 0 < self.num_experts_per_tok <= self.num_experts:
            raise ValueError("DeepSeek-V4 needs routed experts and 0 < top-k <= experts")
        self.router_score_fn = self.scoring_func
        self.route_scale = self.routed_scaling_factor

    def is_moe_layer(self, i: int) -> bool:
        return True


def validate_layer_schedule(cfg) -> None:
    for name, allowed in (("layer_types", ATTENTION_TYPES), ("mlp_layer_types", MLP_TYPES)):
        sched = getattr(cfg, name)
        if len(sched) != cfg.num_hidden_layers:
            raise ValueError(f"DeepSeek-V4 {name} must name every decoder layer ({len(sched)} for {cfg.num_hidden_layers})")
        for i, kind in enumerate(sched):
            if kind not in allowed:
                raise ValueError(f"DeepSeek-V4 {name}[{i}] = {kind!r} is not one of {allowed}")
    for kind in set(cfg.layer_types) - {"sliding_attention"}:
        rate = cfg.compress_rates.get(kind)
        if isinstance(rate, bool) or not isinstance(rate, int) or rate <= 0:
            raise ValueError(f"DeepSeek-V4 compress_rates[{kind!r}] must be a positive integer")


# --------------------------------------------------------------------------------------------------- small pieces
def unweighted_rms_norm(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + eps).to(x.dtype)


def rope_tables_interleaved(positions: torch.Tensor, dim: int, theta: float):
    """cos, sin [T, dim/2] in fp32: one frequency per interleaved channel pair."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=positions.device) / dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def rotate_trailing_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [T, ..., d]; the last 2*cos.shape[-1] channels rotate as interleaved pairs (even, odd), in fp32; the leading
    channels pass through. Passing -sin undoes the rotation."""
    w = 2 * cos.shape[-1]
    lead, rot = x[..., :-w], x[..., -w:]
    shape = [cos.shape[0]] + [1] * (x.dim() - 2) + [cos.shape[-1]]
    c, s = cos.view(shape), sin.view(shape)
    even, odd = rot[..., 0::2].float(), rot[..., 1::2].float()
    out = torch.stack((even * c - odd * s, odd * c + even * s), dim=-1).flatten(-2).to(x.dtype)
    return torch.cat((lead, out), dim=-1)


class GroupedLinear(nn.Module):
    """`n_groups` independent projections stored as one 2-D weight [out, in_per_group]; rows of the weight belong to
    groups in order."""

    def __init__(self, in_per_group: int, out_features: int, n_groups: int, dtype=None, device=None):
        super().__init__()
        if out_features % n_groups:
            raise ValueError("grouped projection: out_features must divide into n_groups")
        self.n_groups, self.in_per_group, self.out_features = n_groups, in_per_group, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_per_group, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [T, G, in] -> [T, G, out/G]."""
        if x.shape[-2:] != (self.n_groups, self.in_per_group):
            raise ValueError(f"grouped projection expects [..., {self.n_groups}, {self.in_per_group}], got {tuple(x.shape)}")
        w = self.weight.view(self.n_groups, -1, self.in_per_group).transpose(1, 2)        # [G, in, out/G]
        return torch.bmm(x.transpose(0, 1), w.to(x.dtype)).transpose(0, 1)


@dataclass
class V4Context(ForwardContext):
    positions: torch.Tensor | None = None
    rope: dict | None = None                 # "main" / "compress" -> (cos, sin) [T, rope/2]
    token_ids: torch.Tensor | None = None    # set by the model's forward for hash-routed blocks


def _cp(ctx):
    cp = getattr(ctx, "cp", None)
    return cp if cp is not None and getattr(cp, "size", 1) > 1 else None


def _docs(ctx) -> list[tuple[int, int]]:
    """(first row, length) of every document of the batch, in the row numbering of the gathered (whole-sequence) tensors:
    the local rows without sequence parallelism, the global rows with it."""
    cp = _cp(ctx)
    if cp is None:
        return [(int(p[0]), int(p[1])) for p in ctx.attn_meta.pieces]
    gcu = cp._mb["gcu"]
    return [(gcu[i], gcu[i + 1] - gcu[i]) for i in range(len(gcu) - 1)]


def _views(ctx) -> list[tuple[int, int, int, int]]:
    """What this rank's queries see: (first local query row, count, position of that row inside its document, index of the
    document in `_docs`). Without sequence parallelism every document is one view that starts at position 0."""
    cp = _cp(ctx)
    if cp is None:
        return [(int(p[0]), int(p[1]), 0, i) for i, p in enumerate(ctx.attn_meta.pieces)]
    import bisect
    gcu = cp._mb["gcu"]
    return [(int(q0), int(n), int(off), bisect.bisect_right(gcu, int(k0)) - 1) for q0, n, k0, _klen, off in cp._mb["meta"].pieces]


def _whole(ctx, t: torch.Tensor) -> torch.Tensor:
    """Per-token tensors that every rank needs for the whole sequence (one shared key/value head, compressor inputs) are
    small: under sequence parallelism they are gathered, and every rank pools the windows redundantly."""
    cp = _cp(ctx)
    return t if cp is None else cp.gather_rows(t)


# --------------------------------------------------------------------------------------------------- compressors
class _WindowPool(nn.Module):
    """Shared by the two compressors and the indexer: project, cut each document into windows of `rate` tokens, pool
    every window with a softmax gate (plus a learned per-slot bias), normalise, rotate at the window's first position."""

    def __init__(self, cfg: DeepseekV4Config, rate: int, width: int, overlap: bool, dtype=None, device=None):
        super().__init__()
        self.rate, self.width, self.overlap = rate, width, overlap
        m = 2 if overlap else 1
        self.kv_proj = Linear(cfg.hidden_size, m * width, dtype, device)
        self.gate_proj = Linear(cfg.hidden_size, m * width, dtype, device)
        self.position_bias = nn.Parameter(torch.empty(rate, m * width, dtype=dtype, device=device))
        self.kv_norm = RMSNorm(width, cfg.rms_norm_eps, dtype, device)
        self.rope_dim, self.theta = cfg.qk_rope_head_dim, cfg.compress_rope_theta

    def pool(self, x: torch.Tensor, ctx) -> list[torch.Tensor]:
        """Per document of `_docs`: entries [W, width] (W = complete windows of that document, possibly 0)."""
        kv_all, gate_all = _whole(ctx, self.kv_proj(x)), _whole(ctx, self.gate_proj(x))
        out = []
        d, r = self.width, self.rate
        for q0, L in _docs(ctx):
            W = L // r
            if W == 0:
                out.append(kv_all.new_zeros(0, d))
                continue
            kv = kv_all[q0:q0 + W * r].view(W, r, -1)
            gate = gate_all[q0:q0 + W * r].view(W, r, -1) + self.position_bias.to(gate_all.dtype)
            if self.overlap:
                # entry w pools the FIRST half of window w-1's features with the SECOND half of window w's; window 0 has
                # no predecessor: its first half is masked out
                prev_kv = torch.cat((kv.new_zeros(1, r, d), kv[:-1, :, :d]), 0)
                prev_gate = torch.cat((gate.new_full((1, r, d), float("-inf")), gate[:-1, :, :d]), 0)
                kv = torch.cat((prev_kv, kv[..., d:]), 1)
                gate = torch.cat((prev_gate, gate[..., d:]), 1)
            w = gate.softmax(dim=1, dtype=torch.float32).to(kv.dtype)
            e = self.kv_norm((kv * w).sum(1))
            pos = torch.arange(W, device=x.device) * r
            cos, sin = rope_tables_interleaved(pos, self.rope_dim, self.theta)
            out.append(rotate_trailing_pairs(e, cos, sin))
        return out


class Indexer(_WindowPool):
    """Scores compressed keys per query and keeps the `index_topk` best among those already complete. Selection is not
    differentiable (the reference runs it without gradient as well)."""

    def __init__(self, cfg: DeepseekV4Config, dtype=None, device=None):
        super().__init__(cfg, cfg.compress_rates["compressed_sparse_attention"], cfg.index_head_dim, True, dtype, device)
        self.heads, self.topk = cfg.index_n_heads, cfg.index_topk
        self.q_b_proj = Linear(cfg.q_lora_rank, self.heads * self.width, dtype, device)
        self.weights_proj = Linear(cfg.hidden_size, self.heads, dtype, device)
        self.score_scale, self.head_scale = self.width ** -0.5, self.heads ** -0.5

    @torch.no_grad()
    def select(self, x: torch.Tensor, q_residual: torch.Tensor, ctx) -> list[torch.Tensor]:
        """Per view of `_views`: [L, min(topk, W)] entry indices, -1 where fewer entries are visible."""
        if q_residual.shape != (x.shape[0], self.q_b_proj.weight.shape[1]):
            raise ValueError("indexer: q_residual does not match the rows")
        keys = self.pool(x, ctx)
        cos, sin = ctx.rope["compress"]
        q = rotate_trailing_pairs(self.q_b_proj(q_residual).view(x.shape[0], self.heads, self.width), cos, sin)
        hw = self.weights_proj(x).float() * self.head_scale
        out = []
        for q0, L, _first, doc in _views(ctx):
            k = keys[doc]
            W = k.shape[0]
            if W == 0:
                out.append(torch.full((L, 0), -1, dtype=torch.int64, device=x.device))
                continue
            s = torch.einsum("lhd,wd->lhw", q[q0:q0 + L].float(), k.float())
            s = (F.relu(s) * self.score_scale * hw[q0:q0 + L, :, None]).sum(1)                  # [L, W]
            thr = (ctx.positions[q0:q0 + L] + 1) // self.rate
            s = s.masked_fill(torch.arange(W, device=x.device)[None, :] >= thr[:, None], float("-inf"))
            sel = s.topk(min(self.topk, W), dim=-1).indices
            out.append(torch.where(sel >= thr[:, None], torch.full_like(sel, -1), sel))
        return out


class HCACompressor(_WindowPool):
    def __init__(self, cfg, dtype=None, device=None):
        super().__init__(cfg, cfg.compress_rates["heavily_compressed_attention"], cfg.head_dim, False, dtype, device)

    def forward(self, x, q_residual, ctx):
        """Per view: (entries [W, d], bias [L, W]: 0 where the entry's window is complete at the query, else -inf)."""
        out = []
        pooled = self.pool(x, ctx)
        for q0, L, _first, doc in _views(ctx):
            e = pooled[doc]
            thr = (ctx.positions[q0:q0 + L] + 1) // self.rate
            hidden = torch.arange(e.shape[0], device=x.device)[None, :] >= thr[:, None]
            out.append((e, torch.zeros(L, e.shape[0], device=x.device).masked_fill(hidden, float("-inf"))))
        return out


class CSACompressor(_WindowPool):
    def __init__(self, cfg, dtype=None, device=None):
        super().__init__(cfg, cfg.compress_rates["compressed_sparse_attention"], cfg.head_dim, True, dtype, device)
        self.indexer = Indexer(cfg, dtype, device)

    def forward(self, x, q_residual, ctx):
        out = []
        pooled = self.pool(x, ctx)
        for (q0, L, _first, doc), sel in zip(_views(ctx), self.indexer.select(x, q_residual, ctx)):
            e = pooled[doc]
            W = e.shape[0]
            bias = torch.full((L, W + 1), float("-inf"), device=x.device)
            bias.scatter_(1, torch.where(sel >= 0, sel, torch.full_like(sel, W)), 0.0)      # invalid picks go to a spare slot
            out.append((e, bias[:, :W]))
        return out


# --------------------------------------------------------------------------------------------------- attention
class V4Attention(nn.Module):
    def __init__(self, cfg: DeepseekV4Config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_type = cfg.layer_types[layer_idx]
        self.rope_kind = "main" if self.layer_type == "sliding_attention" else "compress"
        H, d = cfg.num_attention_heads, cfg.head_dim
        self.H, self.d, self.window, self.eps, self.groups = H, d, cfg.sliding_window, cfg.rms_norm_eps, cfg.o_groups
        self.scale = d ** -0.5
        self.q_a_proj = Linear(cfg.hidden_size, cfg.q_lora_rank, dtype, device)
        self.q_a_norm = RMSNorm(cfg.q_lora_rank, cfg.rms_norm_eps, dtype, device)
        self.q_b_proj = Linear(cfg.q_lora_rank, H * d, dtype, device)
        self.kv_proj = Linear(cfg.hidden_size, d, dtype, device)
        self.kv_norm = RMSNorm(d, cfg.rms_norm_eps, dtype, device)
        self.o_a_proj = GroupedLinear(H * d // cfg.o_groups, cfg.o_groups * cfg.o_lora_rank, cfg.o_groups, dtype, device)
        self.o_b_proj = Linear(cfg.o_groups * cfg.o_lora_rank, cfg.hidden_size, dtype, device)
        self.sinks = nn.Parameter(torch.empty(H, dtype=dtype, device=device))
        self.compressor = {"sliding_attention": None, "heavily_compressed_attention": HCACompressor,
                           "compressed_sparse_attention": CSACompressor}[self.layer_type]
        if self.compressor is not None:
            self.compressor = self.compressor(cfg, dtype, device)

    def _attend(self, q, kv, entries, bias, first: int = 0, chunk: int = 1024):
        """One view. q [L, H, d]: queries at positions first .. first + L of their document; kv [first + L, d]: the
        document's shared keys = values up to the last query; entries [W, d] with additive bias [L, W]. The query at
        position p sees rows (p - window, p] and the entries its bias admits; a per-head sink logit joins the softmax
        and is dropped afterwards."""
        L, H, d = q.shape
        W = entries.shape[0]
        sink = self.sinks.float().view(1, H, 1)
        outs = []
        for c0 in range(0, L, chunk):
            c1 = min(L, c0 + chunk)
            k0 = max(0, first + c0 - self.window + 1)
            keys = kv[k0:first + c1]
            s = torch.einsum("lhd,kd->lhk", q[c0:c1], keys).float() * self.scale
            qi = torch.arange(first + c0, first + c1, device=q.device)[:, None]
            kj = torch.arange(k0, first + c1, device=q.device)[None, :]
            s = s.masked_fill(((kj > qi) | (kj <= qi - self.window))[:, None, :], float("-inf"))
            parts = [s]
            if W:
                se = torch.einsum("lhd,wd->lhw", q[c0:c1], entries).float() * self.scale
                parts.append(se + bias[c0:c1, None, :])
            parts.append(sink.expand(c1 - c0, H, 1))
            p = torch.cat(parts, -1).softmax(-1)
            n = keys.shape[0]
            o = torch.einsum("lhk,kd->lhd", p[..., :n].to(kv.dtype), keys)
            if W:
                o = o + torch.einsum("lhw,wd->lhd", p[..., n:n + W].to(kv.dtype), entries)
            outs.append(o)
        return torch.cat(outs, 0)

    def forward(self, x: torch.Tensor, ctx: V4Context) -> torch.Tensor:
        T = x.shape[0]
        cos, sin = ctx.rope[self.rope_kind]
        q_res = self.q_a_norm(self.q_a_proj(x))
        q = unweighted_rms_norm(self.q_b_proj(q_res).view(T, self.H, self.d), self.eps)
        q = rotate_trailing_pairs(q, cos, sin)
        kv = _whole(ctx, rotate_trailing_pairs(self.kv_norm(self.kv_proj(x)), cos, sin))
        comp = self.compressor(x, q_res, ctx) if self.compressor is not None else None
        docs = _docs(ctx)
        outs = []
        for i, (q0, L, first, doc) in enumerate(_views(ctx)):
            if comp is None:
                e, b = kv.new_zeros(0, self.d), None
            else:
                e, b = comp[i]
            g0 = docs[doc][0]
            outs.append(self._attend(q[q0:q0 + L], kv[g0:g0 + first + L], e, b, first))
        o = torch.cat(outs, 0) if len(outs) > 1 else outs[0]
        o = rotate_trailing_pairs(o, cos, -sin)            # values carried the rotation of their own position: undo the query's
        g = self.o_a_proj(o.reshape(T, self.groups, -1)).reshape(T, -1)
        return self.o_b_proj(g)


# --------------------------------------------------------------------------------------------------- hyper-connections
class HyperConnection(nn.Module):
    """streams [T, n, D] -> (write gains [T, n], mixing matrix [T, n, n], collapsed input [T, D])."""

    def __init__(self, cfg: DeepseekV4Config, dtype=None, device=None):
        super().__init__()
        n = cfg.hc_mult
        self.n, self.iters, self.eps, self.norm_eps = n, cfg.hc_sinkhorn_iters, cfg.hc_eps, cfg.rms_norm_eps
        self.fn = nn.Parameter(torch.empty((2 + n) * n, n * cfg.hidden_size, dtype=dtype, device=device))
        self.base = nn.Parameter(torch.empty((2 + n) * n, dtype=dtype, device=device))
        self.scale = nn.Parameter(torch.empty(3, dtype=dtype, device=device))

    def forward(self, streams: torch.Tensor):
        n = self.n
        flat = unweighted_rms_norm(streams.flatten(1).float(), self.norm_eps)
        pre_w, post_w, comb_w = F.linear(flat, self.fn.float()).split([n, n, n * n], dim=-1)
        pre_b, post_b, comb_b = self.base.float().split([n, n, n * n])
        s_pre, s_post, s_comb = self.scale.float().unbind(0)
        pre = torch.sigmoid(pre_w * s_pre + pre_b) + self.eps
        post = 2 * torch.sigmoid(post_w * s_post + post_b)
        comb = torch.softmax(comb_w.view(-1, n, n) * s_comb + comb_b.view(n, n), dim=-1) + self.eps
        comb = comb / (comb.sum(-2, keepdim=True) + self.eps)                       # columns first
        for _ in range(self.iters - 1):
            comb = comb / (comb.sum(-1, keepdim=True) + self.eps)
            comb = comb / (comb.sum(-2, keepdim=True) + self.eps)
        collapsed = (pre.unsqueeze(-1) * streams).sum(1)
        return post, comb, collapsed.to(streams.dtype)


class HyperHead(nn.Module):
    def __init__(self, cfg: DeepseekV4Config, dtype=None, device=None):
        super().__init__()
        self.eps, self.norm_eps = cfg.hc_eps, cfg.rms_norm_eps
        self.hc_fn = nn.Parameter(torch.empty(cfg.hc_mult, cfg.hc_mult * cfg.hidden_size, dtype=dtype, device=device))
        self.hc_base = nn.Parameter(torch.empty(cfg.hc_mult, dtype=dtype, device=device))
        self.hc_scale = nn.Parameter(torch.empty(1, dtype=dtype, device=device))

    def forward(self, streams: torch.Tensor) -> torch.Tensor:
        flat = unweighted_rms_norm(streams.flatten(1).float(), self.norm_eps)
        pre = torch.sigmoid(F.linear(flat, self.hc_fn.float()) * self.hc_scale.float() + self.hc_base.float()) + self.eps
        return (pre.unsqueeze(-1) * streams).sum(1).to(streams.dtype)


def write_streams(post, comb, y, streams):
    """new[t, m] = post[t, m] * y[t] + sum_n comb[t, n, m] * streams[t, n]: the mixing consumes the matrix transposed."""
    dt = streams.dtype
    return post.to(dt).unsqueeze(-1) * y.unsqueeze(1) + torch.matmul(comb.to(dt).transpose(-1, -2), streams)


# --------------------------------------------------------------------------------------------------- layers, model
class ClampedGatedMLP(GatedMLP):
    def __init__(self, hidden, inter, limit, dtype=None, device=None):
        super().__init__(hidden, inter, dtype, device)
        self.limit = limit

    def forward(self, x):
        from .. import ops
        g = self.gate_proj(x).clamp(max=self.limit)
        u = self.up_proj(x).clamp(min=-self.limit, max=self.limit)
        return self.down_proj(ops.swiglu(g, u))


class V4DecoderLayer(nn.Module):
    def __init__(self, cfg: DeepseekV4Config, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.self_attn = V4Attention(cfg, layer_idx, dtype, device)
        self.is_hash = cfg.mlp_layer_types[layer_idx] == "hash_moe"
        self.mlp = MoE(cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size,
                       shared_inter=cfg.shared_expert_intermediate_size or cfg.moe_intermediate_size, score_fn=cfg.scoring_func,
                       norm_topk_prob=True, route_scale=cfg.routed_scaling_factor,
                       bias_update_coeff=0.0 if self.is_hash else cfg.router_bias_update_coeff,
                       aux_loss_coef=cfg.router_aux_loss_coef, experts_implementation=cfg.experts_implementation, dtype=dtype,
                       device=device, swiglu_limit=cfg.swiglu_limit, hash_vocab_size=cfg.vocab_size if self.is_hash else 0,
                       shared_mlp_factory=lambda inter: ClampedGatedMLP(cfg.hidden_size, inter, cfg.swiglu_limit, dtype, device))
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.attn_hc = HyperConnection(cfg, dtype, device)
        self.ffn_hc = HyperConnection(cfg, dtype, device)

    def forward(self, streams: torch.Tensor, ctx: V4Context) -> torch.Tensor:
        post, comb, x = self.attn_hc(streams)
        streams = write_streams(post, comb, self.self_attn(self.input_layernorm(x), ctx), streams)
        post, comb, x = self.ffn_hc(streams)
        h = self.post_attention_layernorm(x)
        y = self.mlp(h, token_ids=ctx.token_ids) if self.is_hash else self.mlp(h)
        return write_streams(post, comb, y, streams)


class DeepseekV4ForCausalLM(Qwen3ForCausalLM):
    decoder_structure = DecoderStructure()

    def __init__(self, cfg: DeepseekV4Config, dtype=None, device=None):
        nn.Module.__init__(self)
        self.config = cfg
        self.model = Qwen3Model.__new__(Qwen3Model)
        nn.Module.__init__(self.model)
        self.model.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, dtype, device)
        self.model.layers = nn.ModuleList(V4DecoderLayer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers))
        self.model.hc_head = HyperHead(cfg, dtype, device)
        self.model.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype, device)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.activation_checkpoint, self.ac_save_every, self.block_runner = "none", 2, None
        self.pp_first = self.pp_last = True

    @torch.no_grad()
    def initialize_parameters(self, seed: int | None = None) -> None:
        super().initialize_parameters(seed)
        for m in self.modules():
            if isinstance(m, V4Attention) and not m.sinks.is_meta:
                m.sinks.zero_()
            elif isinstance(m, HyperConnection) and not m.base.is_meta:
                m.base.zero_()
                m.scale.fill_(1.0)
            elif isinstance(m, HyperHead) and not m.hc_base.is_meta:
                m.hc_base.zero_()
                m.hc_scale.fill_(1.0)
            elif isinstance(m, _WindowPool) and not m.position_bias.is_meta:
                m.position_bias.zero_()
        for i, layer in enumerate(self.model.layers):
            if layer.is_hash and not layer.mlp.router.tid2eid.is_meta:
                layer.mlp.router.fill_table(seed=(seed or 0) * 131 + i)

    def tp_config(self) -> dict[str, str]:
        return {}

    def validate_parallel(self, tp: int = 1, cp_ulysses: int = 1, ep: int = 1) -> None:
        from ..errors import UnsupportedCombinationError
        if tp > 1 or cp_ulysses > 1:
            raise UnsupportedCombinationError("deepseek_v4: no tensor-parallel plan and no Ulysses exchange; use data, expert, FSDP and "
                                              "key/value-gathering sequence parallelism")
        if self.config.num_experts % ep:
            raise UnsupportedCombinationError(f"expert_parallel_size {ep} must divide num_experts {self.config.num_experts}")

    def build_context(self, positions: torch.Tensor, attn_meta, cp=None) -> V4Context:
        if cp is not None and getattr(cp, "size", 1) > 1 and (cp.strategy != "kv_allgather" or cp.load_balancer is not None):
            from ..errors import UnsupportedCombinationError
            raise UnsupportedCombinationError("deepseek_v4: sequence parallelism gathers the shared key/value head and the compressor "
                                              "inputs over contiguous spans: use context_parallel_kv_allgather_size without a load balancer")
        c = self.config
        rope = {"main": rope_tables_interleaved(positions, c.qk_rope_head_dim, c.rope_theta),
                "compress": rope_tables_interleaved(positions, c.qk_rope_head_dim, c.compress_rope_theta)}
        return V4Context(rope["main"][0], rope["main"][1], attn_meta, cp, positions=positions, rope=rope)

    def checkpoint_configuration(self) -> dict:
        """What a reader of a checkpoint must agree on before the tensors mean anything."""
        names = ("vocab_size", "hidden_size", "moe_intermediate_size", "num_hidden_layers", "num_attention_heads", "head_dim",
                 "q_lora_rank", "o_lora_rank", "o_groups", "qk_rope_head_dim", "swiglu_limit", "rms_norm_eps", "sliding_window",
                 "rope_theta", "compress_rope_theta", "layer_types", "mlp_layer_types", "compress_rates", "index_head_dim",
                 "index_n_heads", "index_topk", "hc_mult", "hc_eps", "hc_sinkhorn_iters", "num_experts", "num_experts_per_tok",
                 "scoring_func", "routed_scaling_factor", "tie_word_embeddings")
        return {n: getattr(self.config, n) for n in names}

    def forward(self, tokens, ctx: V4Context, skip_lm_head: bool = False, inputs_embeds=None):
        if any(l.is_hash for l in self.model.layers):
            if not self.pp_first and inputs_embeds is None:
                raise ValueError("hash-routed layers need token ids; they are only known on the first pipeline stage")
            ctx.token_ids = tokens
        x = inputs_embeds if inputs_embeds is not None else self.model.embed_tokens(tokens)
        streams = x.unsqueeze(1).expand(-1, self.config.hc_mult, -1).contiguous()
        for i, layer in enumerate(self.model.layers):
            streams = self.run_block(i, layer, streams, ctx)
        h = self.model.norm(self.model.hc_head(streams))
        return h if skip_lm_head else self.lm_head(h)


def build_deepseek_v4(model_config, dtype=None, device=None, **overrides) -> DeepseekV4ForCausalLM:
    kw = dict(vocab_size=model_config.vocab_size, hidden_size=model_config.hidden_size, intermediate_size=model_config.intermediate_size,
              num_hidden_layers=model_config.num_hidden_layers, num_attention_heads=model_config.num_attention_heads,
              num_key_value_heads=1, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
              shared_expert_intermediate_size=64, router_bias_update_coeff=1e-3,
              experts_implementation=model_config.experts_implementation)
    kw.update(model_config.arch_overrides or {})
    kw.update(overrides)
    kw["num_key_value_heads"] = 1
    names = set(DeepseekV4Config.__dataclass_fields__)
    return DeepseekV4ForCausalLM(DeepseekV4Config(**{k: v for k, v in kw.items() if k in names}), dtype=dtype, device=device)
