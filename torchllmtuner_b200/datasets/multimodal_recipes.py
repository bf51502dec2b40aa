"""Multimodal recipes over local files (reference: llmtuner/datasets/multimodal/recipes.py:1-53, processors.py:1-273; its
`obelics`, `cc12m` and `cc12m-test` recipes stream from the hub, which this platform cannot reach, so the same three
record shapes are read from local JSONL files whose image fields are paths).

  local_captions      {"image": "a.png", "caption": "..."}                       cc12m shape: one image, then its caption
  local_interleaved   {"texts": ["...", null, "..."], "images": [null, "b.png", null]}   obelics shape: aligned lists,
                      exactly one of texts[i] / images[i] is set
  local_multimodal    {"text": "... <|image_pad|> ... <|video_pad|> ...", "images": [...], "videos": [[frame, ...], ...]}

A record becomes a `MultimodalSample` (patches, grids, expanded placeholders, masked labels, three-axis positions). The
loader shuffles by epoch, shards by data-parallel rank, packs whole samples first-fit into rows, collates, and is
resumable by the number of batches delivered (the stream is a pure function of data, seed and rank)."""
from __future__ import annotations

import os

import torch

from ..errors import ConfigError
from .composition import DatasetIterationPolicy, epoch_order
from .contracts import BaseDataLoader, DataloaderExhaustedError, require_same_dp_degree
from .multimodal_pipeline import PackedRow, VisionSpec, build_sample, collate_rows, image_to_patches, video_to_patches

RECIPES = ("local_captions", "local_interleaved", "local_multimodal")


def load_image(path: str) -> torch.Tensor:
    """[3, H, W] float in [0, 1]."""
    from PIL import Image
    import numpy as np
    with Image.open(path) as im:
        arr = np.asarray(im.convert("RGB"), dtype=np.float32) / 255.0
    return torch.from_numpy(arr).permute(2, 0, 1).contiguous()


class MultimodalProcessor:
    """Record -> `MultimodalSample`. `tokenizer` is a `MultimodalTokenizer` (text tokenizer + placeholder ids)."""

    def __init__(self, tokenizer, recipe: str, spec: VisionSpec, root: str = "", image_token: str = "<|image_pad|>",
                 video_token: str = "<|video_pad|>", video_fps: float = 4.0, add_eos: bool = True):
        if recipe not in RECIPES:
            raise ConfigError(f"unknown multimodal recipe {recipe!r}; expected one of {RECIPES}")
        if tokenizer.image_id is None:
            raise ConfigError(f"the tokenizer has no id for the image placeholder {image_token!r}")
        self.tok, self.recipe, self.spec, self.root = tokenizer, recipe, spec, root
        self.image_token, self.video_token, self.video_fps, self.add_eos = image_token, video_token, video_fps, add_eos

    def _path(self, p: str) -> str:
        return p if os.path.isabs(p) else os.path.join(self.root, p)

    def _segments(self, rec: dict):
        """[(kind, payload)] with kind in text / image / video, in reading order."""
        if self.recipe == "local_captions":
            return [("image", rec["image"]), ("text", rec["caption"])]
        if self.recipe == "local_interleaved":
            texts, images = rec["texts"], rec["images"]
            if len(texts) != len(images) or any((t is None) == (i is None) for t, i in zip(texts, images)):
                raise ConfigError("interleaved record: texts and images must be aligned lists with exactly one entry set per slot")
            return [("text", t) if t is not None else ("image", i) for t, i in zip(texts, images)]
        segs, images, videos = [], list(rec.get("images") or []), list(rec.get("videos") or [])
        rest = rec["text"]
        while rest:
            cut = [(rest.find(tok), kind, tok) for kind, tok in (("image", self.image_token), ("video", self.video_token)) if tok in rest]
            if not cut:
                segs.append(("text", rest))
                break
            at, kind, tok = min(cut)
            if at:
                segs.append(("text", rest[:at]))
            pool = images if kind == "image" else videos
            if not pool:
                raise ConfigError(f"record names more {kind} placeholders than {kind}s")
            segs.append((kind, pool.pop(0)))
            rest = rest[at + len(tok):]
        if images or videos:
            raise ConfigError("record holds images or videos without a placeholder in its text")
        return segs

    def __call__(self, rec: dict):
        ids, items = [], []
        for kind, payload in self._segments(rec):
            if kind == "text":
                ids += [t for t in self.tok.encode(payload) if t != self.tok.image_id]
            elif kind == "image":
                items.append(image_to_patches(load_image(self._path(payload)), self.spec))
                ids.append(self.tok.image_id)
            else:
                frames = torch.stack([load_image(self._path(p)) for p in payload])
                items.append(video_to_patches(frames, self.video_fps, self.spec))
                ids.append(self.tok.image_id)          # clips use the same placeholder rows as images
        eos = getattr(self.tok, "eos_id", None)
        if self.add_eos and eos is not None:
            ids.append(eos)
        return build_sample(ids, items, placeholder_id=self.tok.image_id, spec=self.spec, start_id=self.tok.vision_start_id,
                            end_id=self.tok.vision_end_id)


class MultimodalDataLoader(BaseDataLoader):
    def __init__(self, source, processor, *, seq_len: int, rows_per_rank: int, dp_rank: int, dp_degree: int, policy: DatasetIterationPolicy,
                 pad_id: int = 0, identity: str = "", pin_memory: bool = False):
        self.source, self.proc = source, processor
        self.seq_len, self.rows, self.dp_rank, self.dp_degree = seq_len, rows_per_rank, dp_rank, dp_degree
        self.policy, self.pad_id, self.identity, self.pin = policy, pad_id, identity, pin_memory
        self.delivered, self.dropped = 0, 0
        self._gen = None

    def _samples(self):
        epoch = 0
        while True:
            order = epoch_order(len(self.source), epoch, self.policy, self.dp_rank, self.dp_degree)
            if not order:
                return
            for i in order:
                yield self.proc(self.source[i])
            epoch += 1
            if not self.policy.repeat:
                return

    def _batches(self):
        """Rows are filled in arrival order; a sample that does not fit the open row closes it (samples stay whole)."""
        rows, cur = [], PackedRow()
        for s in self._samples():
            if len(s) > self.seq_len:
                self.dropped += 1
                continue
            if cur.used + len(s) > self.seq_len:
                rows.append(cur)
                cur = PackedRow()
                if len(rows) == self.rows:
                    yield collate_rows(rows, self.seq_len, self.pad_id)
                    rows = []
            cur.samples.append(s)
            cur.used += len(s)
        if cur.samples:
            rows.append(cur)
        if len(rows) == self.rows:
            yield collate_rows(rows, self.seq_len, self.pad_id)

    def __next__(self) -> dict:
        if self._gen is None:
            self._gen = self._batches()
            for _ in range(self.delivered):
                next(self._gen, None)
        b = next(self._gen, None)
        if b is None:
            raise DataloaderExhaustedError("multimodal data exhausted")
        if self.pin:
            for k in ("input", "labels", "positions", "patches"):
                if isinstance(b.get(k), torch.Tensor):
                    b[k] = b[k].pin_memory()
        self.delivered += 1
        return b

    def state_dict(self) -> dict:
        return {"delivered": self.delivered, "dp_degree": self.dp_degree, "rows": self.rows, "seq_len": self.seq_len, "identity": self.identity}

    def load_state_dict(self, sd: dict) -> None:
        require_same_dp_degree(int(sd["dp_degree"]), self.dp_degree)
        if sd.get("identity") != self.identity:
            raise ConfigError("the data cursor belongs to a different corpus / tokenizer / packing setup")
        if int(sd["rows"]) != self.rows or int(sd["seq_len"]) != self.seq_len:
            raise ConfigError("batch layout changed since the data cursor was saved")
        self.delivered, self._gen = int(sd["delivered"]), None


def build_multimodal_dataloader(data_cfg, *, model, vocab_size: int, seq_len: int, seed: int, dp_rank: int, dp_degree: int,
                                rows_per_rank: int, pin_memory: bool = False, split: str = "train") -> MultimodalDataLoader:
    from ..components.tokenizer.huggingface import MultimodalTokenizer, build_tokenizer
    from .corpus_identity import corpus_data_identity
    from .sources import IndexedJsonlSource
    if model is None or not hasattr(model, "image_token_id"):
        raise ConfigError(f"dataset {data_cfg.dataset!r} needs a vision-language model")
    if not data_cfg.dataset_path:
        raise ConfigError(f"dataset {data_cfg.dataset!r} needs dataset_path")
    tok = MultimodalTokenizer(build_tokenizer(data_cfg), data_cfg)
    if tok.vocab_size > vocab_size:
        raise ConfigError(f"tokenizer vocabulary {tok.vocab_size} exceeds the model vocabulary {vocab_size}")
    if tok.image_id != model.image_token_id:
        raise ConfigError(f"the tokenizer maps {data_cfg.mm_image_token!r} to {tok.image_id}, the model expects image_token_id "
                          f"{model.image_token_id}")
    vc = model.visual.config
    spec = VisionSpec(patch_size=vc.patch_size, merge_size=vc.spatial_merge_size, max_pixels=data_cfg.mm_max_pixels,
                      min_pixels=min(data_cfg.mm_max_pixels, (vc.patch_size * vc.spatial_merge_size * 2) ** 2),
                      temporal_pool=getattr(vc, "temporal_pool", False), video_max_frames=2 * getattr(vc, "pos_emb_time", 16),
                      temporal_patch_size=getattr(vc, "temporal_patch_size", 2), full_temporal=hasattr(vc, "full_patch_dim"))
    src = IndexedJsonlSource(data_cfg.dataset_path)
    root = os.path.dirname(src.paths[0]) if getattr(src, "paths", None) else ""
    proc = MultimodalProcessor(tok, data_cfg.dataset, spec, root=root, image_token=data_cfg.mm_image_token, video_token=data_cfg.mm_video_token)
    ident = corpus_data_identity(data_cfg, tok.identity(), getattr(src, "paths", ()))
    policy = DatasetIterationPolicy(shuffle=data_cfg.shuffle, seed=seed, repeat=split == "train")
    return MultimodalDataLoader(src, proc, seq_len=seq_len, rows_per_rank=rows_per_rank, dp_rank=dp_rank, dp_degree=dp_degree, policy=policy,
                                pad_id=tok.pad_id or 0, identity=ident, pin_memory=pin_memory)
