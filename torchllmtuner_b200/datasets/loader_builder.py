"""`build_dataloader`: synthetic path, or recipe + tokenizer + packing + collator + prefetching loader
(reference: llmtuner/datasets/loader_builder.py:154-317)."""
from __future__ import annotations

from ..errors import ConfigError
from .synthetic import RandomPackedSource, RandomTokenDataLoader, RandomTokenSource


def build_dataloader(data_cfg, *, vocab_size: int, global_batch: int, seq_len: int, seed: int, dp_rank: int, dp_degree: int,
                     rows_per_rank: int, pin_memory: bool = False, split: str = "train", model=None):
    name = data_cfg.dataset
    if name == "random_multimodal":
        # image-and-text documents for a vision-language model: the model says which token marks an image and how its
        # tower cuts pixels into patches
        from .multimodal_pipeline import SyntheticMultimodalLoader, VisionSpec
        if model is None or not hasattr(model, "image_token_id"):
            raise ConfigError("dataset 'random_multimodal' needs a vision-language model (one that names an image_token_id)")
        vc = model.visual.config
        spec = VisionSpec(patch_size=vc.patch_size, merge_size=vc.spatial_merge_size, max_pixels=data_cfg.mm_max_pixels,
                          temporal_pool=getattr(vc, "temporal_pool", False), video_max_frames=2 * getattr(vc, "pos_emb_time", 16),
                      temporal_patch_size=getattr(vc, "temporal_patch_size", 2), full_temporal=hasattr(vc, "full_patch_dim"),
                          min_pixels=min(data_cfg.mm_max_pixels, (vc.patch_size * vc.spatial_merge_size * 2) ** 2))
        return SyntheticMultimodalLoader(vocab_size=vocab_size, image_token_id=model.image_token_id, global_batch=global_batch,
                                         seq_len=seq_len, seed=seed, dp_rank=dp_rank, dp_degree=dp_degree, rows_per_rank=rows_per_rank,
                                         spec=spec, max_items=data_cfg.mm_max_items, video_fraction=data_cfg.mm_video_fraction,
                                         pin_memory=pin_memory)
    if name == "random":
        return RandomTokenDataLoader(RandomTokenSource(vocab_size, global_batch, seq_len, seed), dp_rank, dp_degree,
                                     rows_per_rank, pin_memory)
    if name == "random_packed":
        src = RandomPackedSource(vocab_size, global_batch, seq_len, seed, data_cfg.packed_min_doc_len, data_cfg.packed_max_doc_len)
        return RandomTokenDataLoader(src, dp_rank, dp_degree, rows_per_rank, pin_memory)
    if name in ("local_captions", "local_interleaved", "local_multimodal"):
        from .multimodal_recipes import build_multimodal_dataloader
        return build_multimodal_dataloader(data_cfg, model=model, vocab_size=vocab_size, seq_len=seq_len, seed=seed, dp_rank=dp_rank,
                                           dp_degree=dp_degree, rows_per_rank=rows_per_rank, pin_memory=pin_memory, split=split)
    try:
        from .text import build_text_dataloader
    except ImportError as e:  # pragma: no cover
        raise ConfigError(f"dataset {name!r} needs the text pipeline: {e}") from e
    return build_text_dataloader(data_cfg, vocab_size=vocab_size, seq_len=seq_len, seed=seed, dp_rank=dp_rank,
                                 dp_degree=dp_degree, rows_per_rank=rows_per_rank, pin_memory=pin_memory, split=split)
