"""Multimodal samples -> packed trainer batches (reference: llmtuner/datasets/multimodal/image.py:1-472, video.py:1-174,
mrope.py:1-231, packing.py:1-140, collator.py:1-220, processors.py:1-273, recipes.py:1-53).

A sample is text with image and video placeholders plus the pixel tensors themselves. The pipeline
  1. turns every image / clip into flattened patches and a grid `(t, gh, gw)` within a pixel budget (video: frames are
     sampled at a target rate within a frame budget, and `temporal_patch_size` consecutive frames form one temporal step);
  2. expands each placeholder to the number of merged patches of its item, masks those tokens (and anything the recipe
     marks as prompt) in the labels, and builds the three-axis rotary positions (text advances all axes, an item keeps
     time per temporal step and walks its grid, the text after it continues past the largest position used);
  3. packs samples into rows of `seq_len` tokens, never cutting inside a sample (first fit over open rows; a sample longer
     than a row is dropped and counted), with document boundaries, per-document positions and the patches of a row in
     the order of its placeholders;
  4. collates rows into one batch dict: `input`, `labels` (already shifted), `positions` [3, B, S], `cu_seqlens`,
     `patches` [N, C*p*p], `grids`, `num_valid_tokens`.
`SyntheticMultimodalLoader` feeds the pipeline with deterministic random samples (no files, no network) and is resumable
by its step cursor, which makes the whole path testable and benchmarkable offline.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .contracts import BaseDataLoader, IGNORE_INDEX, require_same_dp_degree, validate_dp_coordinates
from .multimodal import build_mrope_positions, calculate_vision_tokens, smart_resize, vision_to_patches


@dataclass
class VisionSpec:
    patch_size: int = 14
    merge_size: int = 2
    temporal_patch_size: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 14 * 14 * 4 * 256
    video_fps: float = 2.0
    video_min_frames: int = 4
    video_max_frames: int = 32
    temporal_pool: bool = False        # the tower averages a clip's frames: rows per item do not grow with the frame count
    # The tower's patch embedding has a temporal axis (`models/qwen_vit.py`): every row carries channels x
    # temporal_patch_size x patch x patch values, the frames of a temporal step side by side (an image repeats its one
    # frame), instead of one frame-sized patch per step with the step's frames averaged.
    full_temporal: bool = False

    @property
    def factor(self) -> int:
        return self.patch_size * self.merge_size

    def rows_of(self, grid) -> int:
        t, gh, gw = grid
        return calculate_vision_tokens((1 if self.temporal_pool else t, gh, gw), self.merge_size)

    def position_grid(self, grid):
        return (1, grid[1], grid[2]) if self.temporal_pool else tuple(grid)


# --------------------------------------------------------------------------------------------------- items
def image_to_patches(img: torch.Tensor, spec: VisionSpec):
    """img [C, H, W] in [0, 1] -> (patches [gh*gw, C*p*p], (1, gh, gw))."""
    c, h, w = img.shape
    nh, nw = smart_resize(h, w, factor=spec.factor, min_pixels=spec.min_pixels, max_pixels=spec.max_pixels)
    img = F.interpolate(img[None], size=(nh, nw), mode="bilinear", align_corners=False)[0]
    rows = vision_to_patches(img, spec.patch_size)
    if spec.full_temporal:
        rows = temporal_rows([rows] * spec.temporal_patch_size, c)
    return rows, (1, nh // spec.patch_size, nw // spec.patch_size)


def temporal_rows(frames_rows: list[torch.Tensor], channels: int) -> torch.Tensor:
    """Per-frame patch rows [N, C*p*p] of one temporal step -> [N, C * len(frames) * p*p], laid out channel-major then
    frame, the order of a [C, temporal, patch, patch] convolution kernel."""
    n = frames_rows[0].shape[0]
    return torch.stack([r.view(n, channels, -1) for r in frames_rows], 2).reshape(n, -1)


def sample_frame_indices(num_frames: int, source_fps: float, spec: VisionSpec) -> list[int]:
    """Evenly spaced frame indices at about `video_fps`, clamped to the frame budget and rounded down to a multiple of
    the temporal patch size (never below it)."""
    if num_frames <= 0 or source_fps <= 0:
        raise ValueError("a clip needs frames and a positive frame rate")
    want = num_frames / source_fps * spec.video_fps
    n = int(min(max(want, spec.video_min_frames), spec.video_max_frames, num_frames))
    n = max(spec.temporal_patch_size, n // spec.temporal_patch_size * spec.temporal_patch_size)
    if n > num_frames:
        raise ValueError(f"a clip of {num_frames} frames cannot fill one temporal patch of {spec.temporal_patch_size}")
    return [min(num_frames - 1, int(round(i * (num_frames - 1) / max(1, n - 1)))) for i in range(n)]


def video_to_patches(frames: torch.Tensor, source_fps: float, spec: VisionSpec):
    """frames [F, C, H, W] -> (patches [t*gh*gw, C*p*p], (t, gh, gw)). Each temporal step averages its
    `temporal_patch_size` frames (the tower's patch embedding sees one frame-sized patch per step), or with
    `spec.full_temporal` keeps them side by side in rows of C*temporal_patch_size*p*p values; the pixel budget is shared by
    the steps."""
    idx = sample_frame_indices(frames.shape[0], source_fps, spec)
    clip = frames[idx]
    t = len(idx) // spec.temporal_patch_size
    _, c, h, w = clip.shape
    nh, nw = smart_resize(h, w, factor=spec.factor, min_pixels=spec.min_pixels, max_pixels=max(spec.min_pixels, spec.max_pixels // t))
    clip = F.interpolate(clip, size=(nh, nw), mode="bilinear", align_corners=False)
    steps = clip.view(t, spec.temporal_patch_size, c, nh, nw)
    if spec.full_temporal:
        patches = torch.cat([temporal_rows([vision_to_patches(f, spec.patch_size) for f in step], c) for step in steps])
    else:
        patches = torch.cat([vision_to_patches(s, spec.patch_size) for s in steps.mean(1)])
    return patches, (t, nh // spec.patch_size, nw // spec.patch_size)


# --------------------------------------------------------------------------------------------------- samples
@dataclass
class MultimodalSample:
    tokens: list[int]                  # placeholders already expanded
    labels: list[int]                  # unshifted; IGNORE_INDEX on vision tokens and prompt tokens
    positions: torch.Tensor            # [3, L]
    patches: torch.Tensor              # [N, C*p*p]
    grids: list[tuple[int, int, int]]

    def __len__(self) -> int:
        return len(self.tokens)


def build_sample(ids: list[int], items: list[tuple[torch.Tensor, tuple[int, int, int]]], *, placeholder_id: int, spec: VisionSpec,
                 start_id: int | None = None, end_id: int | None = None, prompt_len: int = 0) -> MultimodalSample:
    """`ids` holds one `placeholder_id` per item, in order; `prompt_len` leading tokens of `ids` carry no loss."""
    grids = [g for _, g in items]
    if sum(t == placeholder_id for t in ids) != len(items):
        raise ValueError(f"{len(items)} vision items but {sum(t == placeholder_id for t in ids)} placeholders")
    tokens, labels, gi = [], [], 0
    for i, t in enumerate(ids):
        if t == placeholder_id:
            n = spec.rows_of(grids[gi])
            gi += 1
            block = ([start_id] if start_id is not None else []) + [placeholder_id] * n + ([end_id] if end_id is not None else [])
            tokens += block
            labels += [IGNORE_INDEX] * len(block)
        else:
            tokens.append(t)
            labels.append(IGNORE_INDEX if i < prompt_len else t)
    positions = build_mrope_positions(tokens, placeholder_id, [spec.position_grid(g) for g in grids], spec.merge_size)
    patches = torch.cat([p for p, _ in items]) if items else torch.zeros(0, 0)
    return MultimodalSample(tokens, labels, positions, patches, grids)


# --------------------------------------------------------------------------------------------------- packing
@dataclass
class PackedRow:
    samples: list[MultimodalSample] = field(default_factory=list)
    used: int = 0


def pack_samples(samples: list[MultimodalSample], seq_len: int, rows: int):
    """First fit into `rows` rows of `seq_len` tokens, samples kept whole and in arrival order inside a row. Returns
    (rows, leftovers that did not fit, number dropped because a single sample exceeds a row)."""
    out = [PackedRow() for _ in range(rows)]
    left, dropped = [], 0
    for s in samples:
        if len(s) > seq_len:
            dropped += 1
            continue
        for r in out:
            if r.used + len(s) <= seq_len:
                r.samples.append(s)
                r.used += len(s)
                break
        else:
            left.append(s)
    return out, left, dropped


def collate_rows(rows: list[PackedRow], seq_len: int, pad_id: int) -> dict:
    """Padding is one extra document per row (no loss, positions from 0), so that the document table always covers
    every token."""
    B = len(rows)
    ids = torch.full((B, seq_len), pad_id, dtype=torch.int64)
    raw = torch.full((B, seq_len), IGNORE_INDEX, dtype=torch.int64)
    pos = torch.zeros(3, B, seq_len, dtype=torch.int64)
    cu, patches, grids = [0], [], []
    for b, row in enumerate(rows):
        at = 0
        for s in row.samples:
            n = len(s)
            ids[b, at:at + n] = torch.tensor(s.tokens)
            raw[b, at:at + n] = torch.tensor(s.labels)
            pos[:, b, at:at + n] = s.positions
            at += n
            cu.append(b * seq_len + at)
            if s.grids:
                patches.append(s.patches)
                grids += s.grids
        if at < seq_len:
            pos[:, b, at:] = torch.arange(seq_len - at)
            cu.append((b + 1) * seq_len)
    labels = torch.full_like(raw, IGNORE_INDEX)
    labels[:, :-1] = raw[:, 1:]                         # position t predicts token t + 1 ...
    cuts = torch.tensor(cu[1:], dtype=torch.int64) - 1
    labels.view(-1)[cuts] = IGNORE_INDEX                # ... but never across a document boundary
    return {"input": ids, "labels": labels, "positions": pos, "cu_seqlens": torch.tensor(cu, dtype=torch.int32),
            "patches": torch.cat(patches) if patches else None, "grids": grids, "num_valid_tokens": int((labels != IGNORE_INDEX).sum())}


# --------------------------------------------------------------------------------------------------- synthetic loader
class SyntheticMultimodalLoader(BaseDataLoader):
    """Deterministic random documents: a prompt, one to `max_items` images or short clips, a response. Every row of every
    step is a function of (seed, step, global row), so ranks draw disjoint rows and a resumed run sees the same data."""

    def __init__(self, *, vocab_size: int, image_token_id: int, global_batch: int, seq_len: int, seed: int, dp_rank: int, dp_degree: int,
                 rows_per_rank: int, spec: VisionSpec | None = None, max_items: int = 2, video_fraction: float = 0.25,
                 image_side: tuple[int, int] = (56, 168), pin_memory: bool = False):
        validate_dp_coordinates(dp_rank, dp_degree)
        if rows_per_rank * dp_degree > global_batch:
            raise ValueError(f"{rows_per_rank} rows x {dp_degree} ranks exceed the global batch {global_batch}")
        if not 0 <= image_token_id < vocab_size:
            raise ValueError("image_token_id must be a token of the vocabulary")
        self.vocab, self.image_id, self.global_batch, self.seq_len, self.seed = vocab_size, image_token_id, global_batch, seq_len, seed
        self.dp_rank, self.dp_degree, self.rows = dp_rank, dp_degree, rows_per_rank
        self.spec = spec or VisionSpec()
        self.max_items, self.video_fraction, self.image_side, self.pin_memory = max_items, video_fraction, image_side, pin_memory
        self.cursor = 0
        self.mb_per_step = global_batch // (rows_per_rank * dp_degree)
        self.dropped = 0

    def _text(self, g, n: int) -> list[int]:
        t = torch.randint(0, self.vocab - 1, (n,), generator=g)
        t = torch.where(t >= self.image_id, t + 1, t)              # never the placeholder itself
        return t.tolist()

    def _sample(self, g) -> MultimodalSample:
        spec = self.spec
        k = int(torch.randint(1, self.max_items + 1, (), generator=g))
        ids, items = self._text(g, int(torch.randint(4, 17, (), generator=g))), []
        prompt_len = len(ids)
        for _ in range(k):
            h, w = (int(torch.randint(self.image_side[0], self.image_side[1] + 1, (), generator=g)) for _ in range(2))
            if torch.rand((), generator=g).item() < self.video_fraction:
                frames = torch.rand(int(torch.randint(4, 13, (), generator=g)), 3, h, w, generator=g)
                items.append(video_to_patches(frames, 4.0, spec))
            else:
                items.append(image_to_patches(torch.rand(3, h, w, generator=g), spec))
            ids.append(self.image_id)
            ids += self._text(g, int(torch.randint(2, 9, (), generator=g)))
            prompt_len = len(ids)
        ids += self._text(g, int(torch.randint(8, 33, (), generator=g)))
        return build_sample(ids, items, placeholder_id=self.image_id, spec=spec, prompt_len=prompt_len)

    def _row(self, step: int, row: int) -> PackedRow:
        g = torch.Generator(device="cpu").manual_seed(((self.seed * 100003 + step) * 1009 + row) % (2 ** 63))
        out = PackedRow()
        while True:
            s = self._sample(g)
            if len(s) > self.seq_len:
                self.dropped += 1
                if not out.samples and self.dropped > 64:
                    raise ValueError(f"no synthetic sample fits max_seq_len {self.seq_len}; raise it or shrink the images")
                continue
            if out.used + len(s) > self.seq_len:
                return out
            out.samples.append(s)
            out.used += len(s)

    def __next__(self) -> dict:
        step, mb = divmod(self.cursor, self.mb_per_step)
        r0 = mb * self.rows * self.dp_degree + self.dp_rank * self.rows
        batch = collate_rows([self._row(step, r0 + i) for i in range(self.rows)], self.seq_len, pad_id=0 if self.image_id != 0 else 1)
        if self.pin_memory:
            for k in ("input", "labels", "positions", "patches"):
                if isinstance(batch.get(k), torch.Tensor):
                    batch[k] = batch[k].pin_memory()
        self.cursor += 1
        return batch

    def state_dict(self) -> dict:
        return {"cursor": self.cursor, "dp_degree": self.dp_degree, "rows": self.rows, "global_batch": self.global_batch,
                "seq_len": self.seq_len, "seed": self.seed}

    def load_state_dict(self, sd: dict) -> None:
        require_same_dp_degree(int(sd["dp_degree"]), self.dp_degree)
        for k, cur in (("rows", self.rows), ("global_batch", self.global_batch), ("seq_len", self.seq_len)):
            if int(sd[k]) != cur:
                raise ValueError(f"data layout changed: saved {k}={sd[k]}, now {cur}")
        self.cursor = int(sd["cursor"])
