"""MoonViT: the vision tower of Kimi-K3 (reference: llmtuner/models/kimi/kimi_k3/multimodal.py:146-914).

Differences from the Qwen-style tower of `models/vision.py`:
  * the patch embedding has a bias and adds a LEARNED 2-D position table [H0, W0, D], resampled bicubically to each
    item's grid, plus a fixed sine / cosine code of the frame index for clips;
  * rotary positions inside the blocks use interleaved channel pairs that alternate between the patch's column (even
    pairs) and its row (odd pairs), both with the frequencies theta^(-4i/d);
  * blocks are LayerNorm -> packed QKV attention over all patches of one item (every frame of a clip attends every
    other) -> LayerNorm -> GELU MLP, projections with biases; a final LayerNorm;
  * clips are POOLED OVER TIME (mean over frames) before each `m x m` neighbourhood is folded into one row, so an item
    contributes (gh / m) * (gw / m) rows however many frames it has;
  * the projector is LayerNorm over the patch width -> Linear -> GELU -> Linear to the text width.
Matrix products go through `ops.linear` (tcgen05 GEMM on the device), attention through the packed-row kernel with one
non-causal piece per item.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..errors import ConfigError
from ..ops.attn_meta import AttnMeta


@dataclass
class MoonViTConfig:
    patch_size: int = 14
    in_channels: int = 3
    hidden_size: int = 128
    intermediate_size: int = 256
    depth: int = 2
    num_heads: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 128
    pos_emb_height: int = 8
    pos_emb_width: int = 8
    pos_emb_time: int = 4
    rope_theta: float = 10_000.0
    ln_eps: float = 1e-5
    temporal_pool: bool = True            # read by the data pipeline: rows per item do not grow with the frame count

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.patch_size * self.patch_size


class BiasLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))

    def forward(self, x):
        return ops.linear(x, self.weight) + self.bias.to(x.dtype)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        return F.layer_norm(x.float(), (x.shape[-1],), self.weight.float(), self.bias.float(), self.eps).to(x.dtype)


def time_code(dim: int, frames: int) -> torch.Tensor:
    """[frames, dim]: sin of frame * 10000^(-j / (dim/2)) for the first half of the channels, cos for the second."""
    omega = 1.0 / 10000 ** (torch.arange(dim // 2, dtype=torch.float32) / (dim / 2.0))
    ang = torch.arange(frames, dtype=torch.float32)[:, None] * omega[None, :]
    return torch.cat((ang.sin(), ang.cos()), 1)


def grid_pair_angles(grids, head_dim: int, theta: float, device=None) -> torch.Tensor:
    """[N, head_dim/2] rotation angle of every interleaved channel pair: pair 2i follows the column, pair 2i+1 the row."""
    if head_dim % 4:
        raise ConfigError("vision rotary head_dim must be divisible by 4")
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 4, dtype=torch.float32, device=device) / head_dim))
    out = []
    for t, gh, gw in grids:
        col = torch.arange(gw, device=device).repeat(gh).float()
        row = torch.arange(gh, device=device).repeat_interleave(gw).float()
        ang = torch.stack((col[:, None] * freqs, row[:, None] * freqs), -1).flatten(1)      # [gh*gw, d/2]
        out.append(ang.repeat(t, 1))
    return torch.cat(out)


def rotate_pairs(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """x [N, H, d], interleaved pairs (2j, 2j+1) rotate by ang[:, j]."""
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2).to(x.dtype)


class MoonViTBlock(nn.Module):
    def __init__(self, cfg: MoonViTConfig, dtype=None, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.heads, self.head_dim = cfg.num_heads, cfg.head_dim
        self.norm0, self.norm1 = LayerNorm(D, cfg.ln_eps, dtype, device), LayerNorm(D, cfg.ln_eps, dtype, device)
        self.wqkv, self.wo = BiasLinear(D, 3 * D, dtype, device), BiasLinear(D, D, dtype, device)
        self.fc0, self.fc1 = BiasLinear(D, cfg.intermediate_size, dtype, device), BiasLinear(cfg.intermediate_size, D, dtype, device)
        self.scale = 1.0 / math.sqrt(self.head_dim)

    def forward(self, x, ang, meta: AttnMeta):
        N = x.shape[0]
        q, k, v = self.wqkv(self.norm0(x)).view(N, 3, self.heads, self.head_dim).unbind(1)
        q, k = rotate_pairs(q, ang), rotate_pairs(k, ang)
        o = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), meta, self.scale)   # width 72 runs padded to 128
        x = x + self.wo(o.reshape(N, -1))
        return x + self.fc1(F.gelu(self.fc0(self.norm1(x))))


class MoonViTTower(nn.Module):
    def __init__(self, cfg: MoonViTConfig, dtype=None, device=None):
        super().__init__()
        if cfg.hidden_size % cfg.num_heads or cfg.hidden_size % 2:
            raise ConfigError("vision hidden_size must be even and a multiple of num_heads")
        self.config = cfg
        self.padded_patch_dim = -(-cfg.patch_dim // 64) * 64
        self.patch_embed = BiasLinear(self.padded_patch_dim, cfg.hidden_size, dtype, device)
        self.pos_emb = nn.Parameter(torch.empty(cfg.pos_emb_height, cfg.pos_emb_width, cfg.hidden_size, dtype=dtype, device=device))
        self.register_buffer("time_weight", time_code(cfg.hidden_size, cfg.pos_emb_time), persistent=False)
        self.blocks = nn.ModuleList(MoonViTBlock(cfg, dtype, device) for _ in range(cfg.depth))
        self.final_layernorm = LayerNorm(cfg.hidden_size, cfg.ln_eps, dtype, device)
        wide = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.pre_norm = LayerNorm(cfg.hidden_size, cfg.ln_eps, dtype, device)
        self.proj0, self.proj1 = BiasLinear(wide, wide, dtype, device), BiasLinear(wide, cfg.out_hidden_size, dtype, device)

    def initialize_parameters(self, seed: int | None = None, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu")
        if seed is not None:
            g.manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.is_meta:
                    continue
                if name.endswith("bias"):
                    p.zero_()
                elif p.dim() == 1:
                    p.fill_(1.0)
                elif name == "pos_emb":
                    p.copy_(torch.randn(p.shape, generator=g).to(p.dtype))
                else:
                    p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))

    def position_table(self, grids, dtype) -> torch.Tensor:
        cfg, out = self.config, []
        table = self.pos_emb.float()
        for t, gh, gw in grids:
            if t > cfg.pos_emb_time:
                raise ConfigError(f"a clip of {t} temporal steps exceeds pos_emb_time {cfg.pos_emb_time}")
            p = table.flatten(0, 1) if (gh, gw) == tuple(table.shape[:2]) else \
                F.interpolate(table.permute(2, 0, 1)[None], size=(gh, gw), mode="bicubic")[0].permute(1, 2, 0).flatten(0, 1)
            if t > 1:
                p = (p[None] + self.time_weight[:t, None, :].to(p.device)).flatten(0, 1)
            out.append(p)
        return torch.cat(out).to(dtype)

    def merge(self, x: torch.Tensor, grids) -> torch.Tensor:
        """Mean over an item's frames, then every m x m neighbourhood -> [rows, m*m, D] in row-major order of the merged grid."""
        m, D, out, at = self.config.spatial_merge_size, x.shape[1], [], 0
        for t, gh, gw in grids:
            n = t * gh * gw
            g = x[at:at + n].view(t, gh // m, m, gw // m, m, D).permute(0, 1, 3, 2, 4, 5).mean(0)
            out.append(g.reshape((gh // m) * (gw // m), m * m, D))
            at += n
        return torch.cat(out)

    def forward(self, patches: torch.Tensor, grids) -> torch.Tensor:
        cfg, m = self.config, self.config.spatial_merge_size
        counts = [t * gh * gw for t, gh, gw in grids]
        if sum(counts) != patches.shape[0] or patches.shape[1] != cfg.patch_dim:
            raise ConfigError(f"patches {tuple(patches.shape)} do not match grids {list(grids)} with patch_dim {cfg.patch_dim}")
        if any(gh % m or gw % m for _, gh, gw in grids):
            raise ConfigError(f"every grid side must be a multiple of the merge size {m}: {list(grids)}")
        w = self.patch_embed.weight
        x = self.patch_embed(F.pad(patches.to(w.dtype), (0, self.padded_patch_dim - cfg.patch_dim)))
        x = x + self.position_table(grids, x.dtype)
        ang = grid_pair_angles(grids, cfg.head_dim, cfg.rope_theta, device=x.device)
        cu = torch.tensor([0] + counts, dtype=torch.int64).cumsum(0)
        meta = AttnMeta.build(cu, causal=False, device=x.device)
        for blk in self.blocks:
            x = blk(x, ang, meta)
        x = self.merge(self.pre_norm(self.final_layernorm(x)), grids)
        return self.proj1(F.gelu(self.proj0(x.flatten(1))))
