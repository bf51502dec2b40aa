"""The vision tower of Qwen3.5's published vision-language checkpoints, weight for weight
(reference: llmtuner/models/qwen/qwen3_5/multimodal.py:47-290 wraps the Hugging Face tower; what the tower computes is
pinned here against `transformers.models.qwen3_5.modeling_qwen3_5.Qwen3_5VisionModel` in
`tests/test_cpu_hf_interop.py`).

  patches       one row per patch: channels x temporal_patch_size x patch x patch values (an image repeats its frame over
                the temporal axis; a row that carries only channels x patch x patch values is repeated here)
  patch_embed   a linear map with bias (a 3-D convolution whose stride equals its kernel is exactly that)
  pos_embed     a learned table over a square grid, read by bilinear interpolation at the patch's place in ITS grid
  blocks        LayerNorm -> attention inside one frame (queries, keys rotated by a 2-D rotary embedding: half of the
                frequencies turn with the row, half with the column) -> LayerNorm -> two-layer GELU(tanh) MLP, all with bias
  merger        LayerNorm, then every merge x merge neighbourhood concatenated into one row, two-layer GELU MLP to the
                text width

Inside the tower rows run in merge-block order (frame, block row, block column, row in block, column in block), the
order Hugging Face processors emit; `patch_order="row_major"` (this framework's data pipeline) is permuted on entry. Either
way one output row per merged cell comes out in (frame, block row, block column) order, the order of the placeholder tokens.

Every projection is `ops.linear` (the sm_100a GEMM on the device), attention is `ops.attention` with one non-causal piece
per frame (head width 72 of the published tower runs zero-padded to 128)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..errors import ConfigError
from ..ops.attn_meta import AttnMeta
from .moonvit import BiasLinear, LayerNorm


@dataclass
class QwenViTConfig:
    depth: int = 2
    hidden_size: int = 128
    intermediate_size: int = 256
    num_heads: int = 2
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    out_hidden_size: int = 128
    num_position_embeddings: int = 64          # a square number: the side of the learned grid is its root
    rope_theta: float = 10_000.0
    ln_eps: float = 1e-6
    patch_order: str = "row_major"             # row_major (this framework's data pipeline) | merge_blocks (HF processors)

    def __post_init__(self):
        side = math.isqrt(self.num_position_embeddings)
        if side * side != self.num_position_embeddings:
            raise ConfigError(f"num_position_embeddings {self.num_position_embeddings} is not a square number")
        if self.hidden_size % self.num_heads or (self.hidden_size // self.num_heads) % 4:
            raise ConfigError("vision hidden_size / num_heads must be a whole number divisible by 4")
        if self.patch_order not in ("row_major", "merge_blocks"):
            raise ConfigError(f"patch_order {self.patch_order!r} is not 'row_major' or 'merge_blocks'")

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:                 # one frame of a patch: what the data pipeline cuts out of an image
        return self.in_channels * self.patch_size * self.patch_size

    @property
    def full_patch_dim(self) -> int:
        return self.patch_dim * self.temporal_patch_size


def merge_block_order(grids, m: int, device=None) -> torch.Tensor:
    """Index that takes row-major patches (frame, row, column) to merge-block order (frame, block row, block column,
    row in block, column in block), over all items of `grids`."""
    out, at = [], 0
    for t, gh, gw in grids:
        idx = torch.arange(t * gh * gw, device=device).view(t, gh // m, m, gw // m, m).permute(0, 1, 3, 2, 4)
        out.append(idx.reshape(-1) + at)
        at += t * gh * gw
    return torch.cat(out)


def block_order_coordinates(grids, m: int, device=None):
    """(row, column) of every patch inside its frame, in merge-block order."""
    rows, cols = [], []
    for t, gh, gw in grids:
        r = torch.arange(gh, device=device)[:, None].expand(gh, gw)
        c = torch.arange(gw, device=device)[None, :].expand(gh, gw)
        perm = lambda g: g.reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).reshape(-1).repeat(t)  # noqa: E731
        rows.append(perm(r))
        cols.append(perm(c))
    return torch.cat(rows), torch.cat(cols)


def interpolated_positions(table: torch.Tensor, grids, m: int) -> torch.Tensor:
    """The learned [side*side, D] table read bilinearly at every patch of every grid (a grid of h x w patches spans the
    whole table: patch i of h sits at i * (side - 1) / (h - 1)), in merge-block order, repeated over the frames."""
    side = math.isqrt(table.shape[0])
    out = []
    for t, gh, gw in grids:
        y = torch.linspace(0, side - 1, gh, device=table.device)
        x = torch.linspace(0, side - 1, gw, device=table.device)
        y0, x0 = y.floor().long(), x.floor().long()
        y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
        fy, fx = (y - y0).to(table.dtype)[:, None, None], (x - x0).to(table.dtype)[None, :, None]
        at = lambda a, b: table[(a[:, None] * side + b[None, :])]                   # noqa: E731  [gh, gw, D]
        grid = (at(y0, x0) * (1 - fy) * (1 - fx) + at(y0, x1) * (1 - fy) * fx + at(y1, x0) * fy * (1 - fx) + at(y1, x1) * fy * fx)
        D = grid.shape[-1]
        grid = grid.view(gh // m, m, gw // m, m, D).permute(0, 2, 1, 3, 4).reshape(gh * gw, D)
        out.append(grid.repeat(t, 1))
    return torch.cat(out)


def rotate_halves(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [N, H, d]; channel j pairs with channel j + d/2."""
    xf = x.float()
    a, b = xf[..., :x.shape[-1] // 2], xf[..., x.shape[-1] // 2:]
    return (xf * cos[:, None, :] + torch.cat((-b, a), -1) * sin[:, None, :]).to(x.dtype)


class _Weight(nn.Module):
    """A bare parameter under the name `<module>.weight` (the position table is an embedding in published files)."""

    def __init__(self, *shape, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))


class PatchProjection(nn.Module):
    """`proj.weight` keeps the published 5-D shape [D, channels, temporal, patch, patch]; the product runs on its 2-D
    view. Where a row is not a whole number of 64-element GEMM tiles (toy sizes; the published 1536 is), rows and weight
    are zero-padded for the call."""

    def __init__(self, cfg: "QwenViTConfig", dtype=None, device=None):
        super().__init__()
        self.proj = nn.Module()
        self.proj.weight = nn.Parameter(torch.empty(cfg.hidden_size, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size,
                                                    dtype=dtype, device=device))
        self.proj.bias = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=dtype, device=device))
        self.pad = (-cfg.full_patch_dim) % 64

    def forward(self, x):
        w = self.proj.weight.view(self.proj.weight.shape[0], -1)
        if self.pad:
            x, w = F.pad(x, (0, self.pad)), F.pad(w, (0, self.pad))
        return ops.linear(x, w) + self.proj.bias.to(x.dtype)


class QwenViTAttention(nn.Module):
    def __init__(self, cfg: QwenViTConfig, dtype=None, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.heads, self.head_dim, self.scale = cfg.num_heads, cfg.head_dim, cfg.head_dim ** -0.5
        self.qkv, self.proj = BiasLinear(D, 3 * D, dtype, device), BiasLinear(D, D, dtype, device)

    def forward(self, x, cos, sin, meta: AttnMeta):
        N = x.shape[0]
        q, k, v = self.qkv(x).view(N, 3, self.heads, self.head_dim).unbind(1)
        q, k = rotate_halves(q, cos, sin), rotate_halves(k, cos, sin)
        o = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), meta, self.scale)
        return self.proj(o.reshape(N, -1))


class QwenViTMLP(nn.Module):
    def __init__(self, cfg: QwenViTConfig, dtype=None, device=None):
        super().__init__()
        self.linear_fc1 = BiasLinear(cfg.hidden_size, cfg.intermediate_size, dtype, device)
        self.linear_fc2 = BiasLinear(cfg.intermediate_size, cfg.hidden_size, dtype, device)

    def forward(self, x):
        return self.linear_fc2(F.gelu(self.linear_fc1(x), approximate="tanh"))


class QwenViTBlock(nn.Module):
    def __init__(self, cfg: QwenViTConfig, dtype=None, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.norm1, self.norm2 = LayerNorm(D, cfg.ln_eps, dtype, device), LayerNorm(D, cfg.ln_eps, dtype, device)
        self.attn, self.mlp = QwenViTAttention(cfg, dtype, device), QwenViTMLP(cfg, dtype, device)

    def forward(self, x, cos, sin, meta: AttnMeta):
        x = x + self.attn(self.norm1(x), cos, sin, meta)
        return x + self.mlp(self.norm2(x))


class QwenViTMerger(nn.Module):
    def __init__(self, cfg: QwenViTConfig, dtype=None, device=None):
        super().__init__()
        self.wide = cfg.hidden_size * cfg.spatial_merge_size ** 2
        self.norm = LayerNorm(cfg.hidden_size, cfg.ln_eps, dtype, device)
        self.linear_fc1, self.linear_fc2 = BiasLinear(self.wide, self.wide, dtype, device), BiasLinear(self.wide, cfg.out_hidden_size, dtype, device)

    def forward(self, x):                      # rows already in merge-block order: a block is m*m consecutive rows
        return self.linear_fc2(F.gelu(self.linear_fc1(self.norm(x).view(-1, self.wide))))


class QwenViTTower(nn.Module):
    """Parameter names are those of the published files under `model.visual.`."""

    def __init__(self, cfg: QwenViTConfig, dtype=None, device=None):
        super().__init__()
        self.config = cfg
        self.patch_embed = PatchProjection(cfg, dtype, device)
        self.pos_embed = _Weight(cfg.num_position_embeddings, cfg.hidden_size, dtype=dtype, device=device)
        self.blocks = nn.ModuleList(QwenViTBlock(cfg, dtype, device) for _ in range(cfg.depth))
        self.merger = QwenViTMerger(cfg, dtype, device)

    def initialize_parameters(self, seed: int | None = None, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu")
        if seed is not None:
            g.manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("bias"):
                    p.zero_()
                elif p.dim() == 1:
                    p.fill_(1.0)
                else:
                    p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(p.dtype))

    def rotary_tables(self, grids, device):
        cfg = self.config
        freqs = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim // 2, 2, dtype=torch.float32, device=device) / (cfg.head_dim // 2)))
        row, col = block_order_coordinates(grids, cfg.spatial_merge_size, device)
        ang = torch.cat((row[:, None].float() * freqs, col[:, None].float() * freqs), -1)      # [N, head_dim / 2]
        ang = torch.cat((ang, ang), -1)
        return ang.cos(), ang.sin()

    def forward(self, patches: torch.Tensor, grids) -> torch.Tensor:
        """patches [N, patch_dim or full_patch_dim] in `config.patch_order`, `grids` [(frames, rows, columns), ...]
        -> [N / merge^2, out_hidden_size]."""
        cfg, m = self.config, self.config.spatial_merge_size
        grids = [tuple(int(v) for v in g) for g in grids]
        if sum(t * gh * gw for t, gh, gw in grids) != patches.shape[0] or patches.shape[1] not in (cfg.patch_dim, cfg.full_patch_dim):
            raise ConfigError(f"patches {tuple(patches.shape)} do not match grids {grids} with patch widths {cfg.patch_dim} / {cfg.full_patch_dim}")
        if any(gh % m or gw % m for _, gh, gw in grids):
            raise ConfigError(f"every grid side must be a multiple of the merge size {m}: {grids}")
        x = patches.to(self.patch_embed.proj.weight.dtype)
        if x.shape[1] == cfg.patch_dim and cfg.temporal_patch_size > 1:                  # one frame: repeated over the temporal axis
            x = x.view(-1, cfg.in_channels, 1, cfg.patch_size * cfg.patch_size).expand(-1, -1, cfg.temporal_patch_size, -1).reshape(x.shape[0], -1)
        if cfg.patch_order == "row_major":
            x = x[merge_block_order(grids, m, x.device)]
        x = self.patch_embed(x)
        x = x + interpolated_positions(self.pos_embed.weight, grids, m).to(x.dtype)
        cos, sin = self.rotary_tables(grids, x.device)
        cu = torch.tensor([0] + [gh * gw for t, gh, gw in grids for _ in range(t)], dtype=torch.int64).cumsum(0)
        meta = AttnMeta.build(cu, causal=False, device=x.device)
        for blk in self.blocks:
            x = blk(x, cos, sin, meta)
        return self.merger(x)
