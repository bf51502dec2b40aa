"""Vision tower, multi-axis rotary positions and the vision-language wrapper of the multimodal families
(reference: llmtuner/models/qwen/qwen3_5/multimodal.py:47-290, llmtuner/models/qwen/qwen3_5_moe/multimodal.py:80-823,
llmtuner/models/qwen/qwen3_5_moe/rotary.py, llmtuner/models/kimi/kimi_k3/multimodal.py:77-1572).

  VisionTower            flattened image patches -> patch embedding -> pre-norm transformer blocks (bidirectional
                         attention inside one image, 2-D rotary positions over the patch grid, SwiGLU MLP) -> a merger that
                         folds every `merge x merge` neighbourhood into one row of the text width
  mrope_tables           cos / sin tables for 3-axis (temporal, height, width) positions: the rotary frequencies are split
                         into sections, each section turns with one axis; with equal axes it is the ordinary table
  VisionLanguageModel    text decoder + tower: image rows replace the embeddings of the placeholder tokens, the decoder
                         runs on the mixed rows with the 3-axis positions

Every projection is the sm_100a GEMM, attention is the packed-row kernel with one non-causal piece per image, the norms
and the rotary step are the fused elementwise kernels; on CPU the same calls resolve to the fp32 statements.
The wrapper exposes the same contracts as a text decoder (decoder structure, `prepare_inputs`, `build_context`, the
block-runner and checkpointing switches pass through to the text model), so the trainer shards its decoder blocks as
usual and keeps the tower in the unit of parameters that no block owns.
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
from .common import GatedMLP, Linear, RMSNorm
from .contracts import DecoderStructure
from .qwen3 import ForwardContext


@dataclass
class VisionConfig:
    patch_size: int = 14
    in_channels: int = 3
    hidden_size: int = 256
    intermediate_size: int = 512
    depth: int = 2
    num_heads: int = 2                 # head_dim = hidden_size / num_heads, 64 or 128 for the CUDA attention kernel
    spatial_merge_size: int = 2
    out_hidden_size: int = 256         # the text decoder's width
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10_000.0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.patch_size * self.patch_size


def grid_rope_tables(grids, head_dim: int, theta: float, device=None):
    """cos / sin [N, head_dim/2] for row-major patches of the grids `(t, gh, gw)`: the first half of the frequencies
    turns with the patch's row, the second half with its column."""
    q = head_dim // 4
    if q * 4 != head_dim:
        raise ConfigError(f"2-D rotary positions need head_dim % 4 == 0, got {head_dim}")
    inv = 1.0 / (theta ** (torch.arange(0, q, dtype=torch.float32, device=device) / q))
    hh, ww = [], []
    for t, gh, gw in grids:
        hh.append(torch.arange(gh, device=device).repeat_interleave(gw).repeat(t))
        ww.append(torch.arange(gw, device=device).repeat(gh * t))
    h, w = torch.cat(hh).float(), torch.cat(ww).float()
    ang = torch.cat((h[:, None] * inv[None], w[:, None] * inv[None]), dim=1)
    return ang.cos(), ang.sin()


def mrope_tables(positions: torch.Tensor, head_dim: int, theta: float, sections=None):
    """positions [3, T] (temporal, height, width) or [T]; `sections` = how many of the head_dim/2 frequencies follow each
    axis (default: an even three-way split, remainder to the temporal axis). Returns cos, sin [T, head_dim/2]."""
    if positions.dim() == 1:
        return ops.rope_tables(positions, head_dim, theta)
    half = head_dim // 2
    if sections is None:
        s = half // 3
        sections = [half - 2 * s, s, s]
    if sum(sections) != half or len(sections) != 3:
        raise ConfigError(f"mrope sections {sections} must be three numbers that sum to head_dim/2 = {half}")
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    axis = torch.repeat_interleave(torch.arange(3, device=positions.device), torch.tensor(sections, device=positions.device))
    pos = positions.float()[axis]                              # [half, T]: the axis each frequency follows
    ang = (pos.t() * inv[None, :]).contiguous()       # the rotary kernel wants dense fp32 tables
    return ang.cos(), ang.sin()


class VisionAttention(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype=None, device=None):
        super().__init__()
        self.heads, self.head_dim, self.eps = cfg.num_heads, cfg.head_dim, cfg.rms_norm_eps
        self.qkv = Linear(cfg.hidden_size, 3 * cfg.hidden_size, dtype, device)
        self.proj = Linear(cfg.hidden_size, cfg.hidden_size, dtype, device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim)

    def forward(self, x, cos, sin, meta: AttnMeta):
        N = x.shape[0]
        q, k, v = self.qkv(x).view(N, 3, self.heads, self.head_dim).unbind(1)
        q, k = ops.qk_norm_rope(q.contiguous(), k.contiguous(), None, None, cos, sin, self.eps)
        o = ops.attention(q, k, v.contiguous(), meta, self.scale)
        return self.proj(o.reshape(N, -1))


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype=None, device=None):
        super().__init__()
        self.norm1 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.attn = VisionAttention(cfg, dtype, device)
        self.norm2 = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.mlp = GatedMLP(cfg.hidden_size, cfg.intermediate_size, dtype, device)

    def forward(self, x, cos, sin, meta):
        x = x + self.attn(self.norm1(x), cos, sin, meta)
        return x + self.mlp(self.norm2(x))


class PatchMerger(nn.Module):
    """Every `m x m` neighbourhood of the patch grid becomes one row: norm, concatenate, two-layer MLP to the text width.
    Output rows are row-major over the merged grid, the order in which the placeholder tokens are laid out."""

    def __init__(self, cfg: VisionConfig, dtype=None, device=None):
        super().__init__()
        self.m = cfg.spatial_merge_size
        wide = cfg.hidden_size * self.m * self.m
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.fc1 = Linear(wide, wide, dtype, device)
        self.fc2 = Linear(wide, cfg.out_hidden_size, dtype, device)

    def regroup(self, x, grids):
        m, D, out, at = self.m, x.shape[1], [], 0
        for t, gh, gw in grids:
            n = t * gh * gw
            g = x[at:at + n].view(t, gh // m, m, gw // m, m, D).permute(0, 1, 3, 2, 4, 5)
            out.append(g.reshape(t * (gh // m) * (gw // m), m * m * D))
            at += n
        return torch.cat(out)

    def forward(self, x, grids):
        x = self.regroup(self.norm(x), grids)
        return self.fc2(F.gelu(self.fc1(x)))


class VisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype=None, device=None):
        super().__init__()
        if cfg.hidden_size % cfg.num_heads:
            raise ConfigError("vision hidden_size must be a multiple of num_heads")
        self.config = cfg
        self.padded_patch_dim = -(-cfg.patch_dim // 64) * 64     # GEMM rows start on 16-byte boundaries
        self.patch_embed = Linear(self.padded_patch_dim, cfg.hidden_size, dtype, device)
        self.blocks = nn.ModuleList(VisionBlock(cfg, dtype, device) for _ in range(cfg.depth))
        self.merger = PatchMerger(cfg, dtype, device)

    def initialize_parameters(self, seed: int | None = None, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu")
        if seed is not None:
            g.manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() == 1:
                    p.fill_(1.0)
                else:
                    p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(p.dtype))

    def forward(self, patches: torch.Tensor, grids) -> torch.Tensor:
        """patches [N, C*p*p], row-major per image in the order of `grids` [(t, gh, gw), ...] -> [N / m^2, out_hidden]."""
        cfg, m = self.config, self.config.spatial_merge_size
        counts = [t * gh * gw for t, gh, gw in grids]
        if sum(counts) != patches.shape[0] or patches.shape[1] != cfg.patch_dim:
            raise ConfigError(f"patches {tuple(patches.shape)} do not match grids {list(grids)} with patch_dim {cfg.patch_dim}")
        if any(gh % m or gw % m for _, gh, gw in grids):
            raise ConfigError(f"every grid side must be a multiple of the merge size {m}: {list(grids)}")
        w = self.patch_embed.weight
        x = F.pad(patches.to(w.dtype), (0, self.padded_patch_dim - cfg.patch_dim))
        x = self.patch_embed(x)
        cos, sin = grid_rope_tables(grids, cfg.head_dim, cfg.rope_theta, device=x.device)
        cu = torch.tensor([0] + counts, dtype=torch.int64).cumsum(0)
        meta = AttnMeta.build(cu, causal=False, device=x.device)
        for blk in self.blocks:
            x = blk(x, cos, sin, meta)
        return self.merger(x, grids)


class VisionLanguageModel(nn.Module):
    """`text` is any decoder of the registry (its `forward(tokens, ctx, skip_lm_head, inputs_embeds=...)` runs on given
    rows); `image_token_id` marks the rows that the tower's output replaces."""

    decoder_structure = DecoderStructure(decoder="text.model", embedding="text.model.embed_tokens", blocks="text.model.layers",
                                         final_norm="text.model.norm", head="text.lm_head")
    # switches that the parallel stages set on "the model" and the text decoder reads on itself
    _PASS = ("block_runner", "activation_checkpoint", "ac_save_every", "ac_block_mask", "pp_first", "pp_last", "activation_swap")

    def __init__(self, text: nn.Module, vision, image_token_id: int, mrope_sections=None, dtype=None, device=None, tower=None):
        """`tower`: the tower class for `vision` (default: the Qwen-style `VisionTower`; `models/moonvit.py::MoonViTTower`
        for Kimi)."""
        super().__init__()
        if vision.out_hidden_size != text.config.hidden_size:
            raise ConfigError(f"vision out_hidden_size {vision.out_hidden_size} != text hidden_size {text.config.hidden_size}")
        self.text, self.visual = text, (tower or VisionTower)(vision, dtype, device)
        self.image_token_id, self.mrope_sections = image_token_id, mrope_sections
        self.config = text.config

    def __setattr__(self, name, value):
        if name in self._PASS and "text" in self.__dict__.get("_modules", {}):
            setattr(self._modules["text"], name, value)
            return
        super().__setattr__(name, value)

    def __getattr__(self, name):
        if name in VisionLanguageModel._PASS:
            return getattr(self._modules["text"], name)
        return super().__getattr__(name)

    @property
    def lm_head(self):
        return self.text.lm_head

    def initialize_parameters(self, seed: int | None = None) -> None:
        self.text.initialize_parameters(seed)
        self.visual.initialize_parameters(None if seed is None else seed + 1)

    def tp_config(self) -> dict:
        return {}

    def validate_parallel(self, tp: int = 1, cp_ulysses: int = 1, ep: int = 1) -> None:
        from ..errors import UnsupportedCombinationError
        if tp > 1 or cp_ulysses > 1:
            raise UnsupportedCombinationError("vision-language models run data-, FSDP- and expert-parallel; the tower is not cut by "
                                              "heads and image rows are not split across sequence shards")
        self.text.validate_parallel(1, 1, ep)

    def flops_per_token(self, seq_len: int) -> float:
        return self.text.flops_per_token(seq_len)

    def prepare_inputs(self, batch: dict, device=None, parallel_dims=None) -> dict:
        """Batch dict of the multimodal collator (`input`, `labels`, `positions` [3, B, S] or [B, S], `cu_seqlens`,
        `patches`, `grids`) -> packed model inputs; patches and grids travel under `model_kwargs`."""
        if parallel_dims is not None and (parallel_dims.get("cp", 1) > 1 or parallel_dims.get("tp", 1) > 1):
            raise ConfigError("vision-language inputs are not split across context- or tensor-parallel ranks")
        ids, labels = batch["input"], batch["labels"]
        B, S = ids.shape
        positions = batch.get("positions")
        if positions is None:
            positions = torch.arange(S, dtype=torch.int64).repeat(B, 1)
        positions = positions.reshape(3, -1) if positions.dim() == 3 else positions.reshape(-1)
        cu = batch.get("cu_seqlens")
        if cu is None:
            cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32)
        dev = device if device is not None else next(self.parameters()).device
        patches = batch.get("patches")
        out = {"tokens": ids.reshape(-1).to(dev, non_blocking=True), "targets": labels.reshape(-1).to(dev, non_blocking=True),
               "positions": positions.to(dev, non_blocking=True), "cu_seqlens": cu, "batch": B, "seq": S,
               "attn_meta": AttnMeta.build(cu, causal=True, device=dev),
               "model_kwargs": {"patches": None if patches is None else patches.to(dev, non_blocking=True), "grids": batch.get("grids")}}
        return out

    def build_context(self, positions: torch.Tensor, attn_meta: AttnMeta, cp=None) -> ForwardContext:
        if getattr(self.text, "accepts_three_axis_positions", False) or positions.dim() == 1:
            return self.text.build_context(positions, attn_meta, cp)
        if getattr(self.text, "positions_are_document_indices", False):      # no rotary in the text model: only restarts matter
            doc = torch.cat([torch.arange(int(p[1]), device=positions.device) for p in attn_meta.pieces])
            return self.text.build_context(doc, attn_meta, cp)
        cos, sin = mrope_tables(positions, self.config.head_dim, self.config.rope_theta, self.mrope_sections)
        return ForwardContext(cos, sin, attn_meta, cp)

    def embed(self, tokens: torch.Tensor, patches=None, grids=None) -> torch.Tensor:
        x = self.text.model.embed_tokens(tokens)
        where = (tokens == self.image_token_id).nonzero().squeeze(1)
        if patches is None:
            if where.numel():
                raise ConfigError(f"{where.numel()} image placeholder tokens but no image patches")
            return x
        rows = self.visual(patches, grids)
        if rows.shape[0] != where.numel():
            raise ConfigError(f"the images give {rows.shape[0]} rows but the text holds {where.numel()} placeholder tokens")
        return x.index_copy(0, where, rows.to(x.dtype))

    def forward(self, tokens, ctx, skip_lm_head: bool = False, patches=None, grids=None):
        return self.text(tokens, ctx, skip_lm_head=skip_lm_head, inputs_embeds=self.embed(tokens, patches, grids))
