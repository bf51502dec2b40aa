"""A small Qwen3-MoE in plain PyTorch with its parallel cuts written out.

Every parameter carries `kind`:
  "dense"   replicated on every rank (embedding, head, norms, router): gradient summed over the data ranks (dp x ep)
  "tp"      a tensor-parallel shard of a dense weight (q/k/v by heads, o by input columns): summed over the data ranks
  "expert"  this rank's experts (ep) cut along the intermediate dimension (tp): summed over dp only, because the ranks of
            one ep group already sent all their tokens to the owner
The full model is built from the seed on every rank and then cut, so a parallel run starts from the same weights as a
single-rank run."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import MiniConfig
from .parallel import AllToAllRows, Mesh, copy_to_tp, reduce_from_tp, shard


def rms_norm(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def rope(x, theta):
    """x [B, S, H, d]: half-rotation rotary embedding at positions 0..S-1."""
    B, S, H, d = x.shape
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=x.device) / d))
    ang = torch.arange(S, dtype=torch.float32, device=x.device)[:, None] * inv[None]
    c, s = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    a, b = x[..., : d // 2], x[..., d // 2:]
    return torch.cat((a * c - b * s, b * c + a * s), -1)


def _param(t: torch.Tensor, kind: str) -> nn.Parameter:
    p = nn.Parameter(t)
    p.kind = kind
    return p


class Attention(nn.Module):
    def __init__(self, cfg: MiniConfig, mesh: Mesh, g: torch.Generator):
        super().__init__()
        D, d, H, Hk = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        init = lambda o, i: torch.randn(o, i, generator=g) * 0.02  # noqa: E731
        wq, wk, wv, wo = init(H * d, D), init(Hk * d, D), init(Hk * d, D), init(D, H * d)
        t, n = mesh.t, mesh.tp
        self.wq, self.wk, self.wv = (_param(shard(w, 0, t, n), "tp") for w in (wq, wk, wv))     # column-parallel: whole heads
        self.wo = _param(shard(wo, 1, t, n), "tp")                                              # row-parallel
        self.q_norm, self.k_norm = _param(torch.ones(d), "dense"), _param(torch.ones(d), "dense")
        self.cfg, self.mesh = cfg, mesh

    def forward(self, x):
        cfg, grp = self.cfg, self.mesh.tp_group
        B, S, _ = x.shape
        d = cfg.head_dim
        h = copy_to_tp(x, grp)
        q = F.linear(h, self.wq).view(B, S, -1, d)
        k = F.linear(h, self.wk).view(B, S, -1, d)
        v = F.linear(h, self.wv).view(B, S, -1, d)
        # the norm weights are replicated but each tp rank applies them to its own heads only: their gradient is partial
        q = rope(rms_norm(q, copy_to_tp(self.q_norm, grp), cfg.rms_eps), cfg.rope_theta)
        k = rope(rms_norm(k, copy_to_tp(self.k_norm, grp), cfg.rms_eps), cfg.rope_theta)
        rep = q.shape[2] // k.shape[2]
        k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        o = o.transpose(1, 2).reshape(B, S, -1)
        return reduce_from_tp(F.linear(o, self.wo), grp)


class MoE(nn.Module):
    def __init__(self, cfg: MiniConfig, mesh: Mesh, g: torch.Generator):
        super().__init__()
        E, D, Fi = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.router = _param(torch.randn(E, D, generator=g) * 0.02, "dense")
        w1, w3, w2 = (torch.randn(E, Fi, D, generator=g) * 0.02, torch.randn(E, Fi, D, generator=g) * 0.02,
                      torch.randn(E, D, Fi, generator=g) * 0.02)
        own = lambda w, dim: shard(shard(w, 0, mesh.e, mesh.ep), dim, mesh.t, mesh.tp)  # noqa: E731
        self.w1, self.w3, self.w2 = _param(own(w1, 1), "expert"), _param(own(w3, 1), "expert"), _param(own(w2, 2), "expert")
        self.cfg, self.mesh = cfg, mesh
        self.local = E // mesh.ep

    def experts(self, rows, counts):
        """rows sorted by local expert, `counts[i]` rows for local expert i."""
        out, at = [], 0
        for i, n in enumerate(counts):
            r = rows[at:at + n]
            out.append(F.linear(F.silu(F.linear(r, self.w1[i])) * F.linear(r, self.w3[i]), self.w2[i]))
            at += n
        return torch.cat(out) if out else rows.new_zeros(0, rows.shape[1])

    def forward(self, x):
        cfg, mesh = self.cfg, self.mesh
        B, S, D = x.shape
        flat = x.reshape(-1, D)
        scores = F.softmax(F.linear(flat.float(), self.router.float()), -1)
        w, idx = scores.topk(cfg.top_k, -1)
        w = (w / (w.sum(-1, keepdim=True) + 1e-20)).to(x.dtype)
        # one copy of the token per chosen expert, sorted by expert so that every destination rank gets one run
        order = idx.reshape(-1).argsort(stable=True)
        copies = copy_to_tp(flat, mesh.tp_group)[order // cfg.top_k]
        counts = torch.bincount(idx.reshape(-1), minlength=cfg.num_experts)
        if mesh.ep > 1:
            theirs = torch.empty_like(counts)
            torch.distributed.all_to_all_single(theirs, counts, group=mesh.ep_group)      # [source rank, local expert]
            send = counts.view(mesh.ep, -1).sum(1).tolist()
            recv = theirs.view(mesh.ep, -1).sum(1).tolist()
            rows = AllToAllRows.apply(copies, send, recv, mesh.ep_group)
            # received rows are (source rank, local expert)-major: regroup them by local expert
            owner = torch.repeat_interleave(torch.arange(self.local).repeat(mesh.ep), theirs)
            by_expert = owner.argsort(stable=True)
            y = self.experts(rows[by_expert], theirs.view(mesh.ep, -1).sum(0).tolist())
            back = torch.empty_like(y)
            back[by_expert] = y
            y = AllToAllRows.apply(back, recv, send, mesh.ep_group)
        else:
            y = self.experts(copies, counts.tolist())
        out = torch.zeros_like(y)
        out[order] = y                                                                     # back to (token, k) order
        # the expert outputs are partial sums over tp; the scores multiply them before the reduction, so the scores'
        # gradient is partial too
        mixed = (out.view(-1, cfg.top_k, D) * copy_to_tp(w, mesh.tp_group)[..., None]).sum(1)
        return reduce_from_tp(mixed, mesh.tp_group).view(B, S, D)


class Block(nn.Module):
    def __init__(self, cfg, mesh, g):
        super().__init__()
        self.n1, self.n2 = _param(torch.ones(cfg.hidden_size), "dense"), _param(torch.ones(cfg.hidden_size), "dense")
        self.attn, self.moe, self.eps = Attention(cfg, mesh, g), MoE(cfg, mesh, g), cfg.rms_eps

    def forward(self, x):
        x = x + self.attn(rms_norm(x, self.n1, self.eps))
        return x + self.moe(rms_norm(x, self.n2, self.eps))


class MiniQwen3Moe(nn.Module):
    def __init__(self, cfg: MiniConfig, mesh: Mesh):
        super().__init__()
        g = torch.Generator().manual_seed(cfg.seed)
        self.embed = _param(torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.02, "dense")
        self.blocks = nn.ModuleList(Block(cfg, mesh, g) for _ in range(cfg.num_layers))
        self.norm = _param(torch.ones(cfg.hidden_size), "dense")
        self.head = _param(torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.02, "dense")
        self.cfg = cfg

    def forward(self, tokens):
        x = F.embedding(tokens, self.embed)
        for b in self.blocks:
            x = b(x)
        return F.linear(rms_norm(x, self.norm, self.cfg.rms_eps), self.head)
