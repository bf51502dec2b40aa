"""Multimodal sample preparation for vision-language text decoders (reference: llmtuner/datasets/multimodal/image.py,
mrope.py, placeholders.py, processors.py): resize an image to a patch grid within a pixel budget, cut it into
flattened patches, splice the right number of placeholder tokens into the text, and build the 3-axis (temporal, height,
width) rotary positions that such models use. Decoding of image/video files is left to the caller (a tensor comes in);
no dataset download is attempted."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """Closest (h, w), both multiples of `factor`, keeping the aspect ratio and the pixel budget."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("absolute aspect ratio must be below 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def process_image(img: torch.Tensor, patch: int = 14, merge: int = 2, **budget):
    """img [C, H, W] float in [0, 1] -> (patches [gh*gw, C*patch*patch], (1, gh, gw))."""
    c, h, w = img.shape
    nh, nw = smart_resize(h, w, factor=patch * merge, **budget)
    img = F.interpolate(img[None], size=(nh, nw), mode="bilinear", align_corners=False)[0]
    return vision_to_patches(img, patch), (1, nh // patch, nw // patch)


def vision_to_patches(img: torch.Tensor, patch: int = 14) -> torch.Tensor:
    c, h, w = img.shape
    gh, gw = h // patch, w // patch
    x = img[:, :gh * patch, :gw * patch].reshape(c, gh, patch, gw, patch).permute(1, 3, 0, 2, 4)
    return x.reshape(gh * gw, c * patch * patch)


def calculate_vision_tokens(grid, merge: int = 2) -> int:
    t, gh, gw = grid
    return t * (gh // merge) * (gw // merge)


def insert_vision_placeholders(ids: list[int], image_id: int, grids, merge: int = 2, start_id=None, end_id=None) -> list[int]:
    """Every single `image_id` in `ids` is expanded to the number of merged patches of the matching image."""
    out, gi = [], 0
    for t in ids:
        if t == image_id:
            n = calculate_vision_tokens(grids[gi], merge)
            gi += 1
            out += ([start_id] if start_id is not None else []) + [image_id] * n + ([end_id] if end_id is not None else [])
        else:
            out.append(t)
    if gi != len(grids):
        raise ValueError(f"{len(grids)} images but {gi} placeholders")
    return out


def build_mrope_positions(ids: list[int], image_id: int, grids, merge: int = 2) -> torch.Tensor:
    """[3, T] positions: text tokens advance all three axes together; an image block keeps the temporal axis fixed and
    walks its (height, width) grid; the text after it continues from the largest position used so far + 1."""
    pos = torch.zeros(3, len(ids), dtype=torch.int64)
    nxt, i, gi = 0, 0, 0
    while i < len(ids):
        if ids[i] == image_id:
            t, gh, gw = grids[gi]
            gi += 1
            gh, gw = gh // merge, gw // merge
            n = t * gh * gw
            tt = torch.arange(t).repeat_interleave(gh * gw)
            hh = torch.arange(gh).repeat_interleave(gw).repeat(t)
            ww = torch.arange(gw).repeat(gh * t)
            pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            nxt += max(t, gh, gw)
            i += n
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos
