"""Dataloader config group (reference: llmtuner/config/data_config.py:13-257)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .utils import require_choice, require_integer_at_least


@dataclass
class DataloaderConfig:
    dataset: str = "random"                      # random | random_packed | local_jsonl | local_jsonl_sft | recipe key
    tokenizer_path: str | None = None
    tokenizer_backend: str = "huggingface"
    dataset_path: str | None = None
    data_identity: str | None = None
    prompt_field: str = "prompt"
    response_field: str = "response"
    text_field: str = "text"
    chat_template: str | None = None
    chat_template_kwargs: dict[str, Any] = field(default_factory=dict)
    chat_renderer: str | None = None
    messages_field: str = "messages"
    shuffle: bool = True
    global_context_rows: bool = False
    streaming_shuffle_buffer_size: int = 1000
    num_prefetch_batches: int = 2
    packing: str = "concat_then_split"           # concat_then_split | first_fit
    num_packing_bins: int = 8
    max_num_documents: int | None = None
    packed_min_doc_len: int = 512                # random_packed: log-uniform document lengths
    packed_max_doc_len: int = 32768
    mm_image_token: str = "<|image_pad|>"
    mm_video_token: str = "<|video_pad|>"
    mm_vision_start_token: str = "<|vision_start|>"
    mm_vision_end_token: str = "<|vision_end|>"
    mm_pad_token: str = "<|endoftext|>"
    mm_max_pixels: int = 14 * 14 * 4 * 64        # random_multimodal: pixel budget per image / clip
    mm_max_items: int = 2                        # random_multimodal: images or clips per document
    mm_video_fraction: float = 0.25              # random_multimodal: share of items that are short clips

    def __post_init__(self):
        require_choice("tokenizer_backend", self.tokenizer_backend, ("huggingface", "kimi_k3", "whitespace"))
        require_choice("packing", self.packing, ("concat_then_split", "first_fit"))
        require_integer_at_least("num_prefetch_batches", self.num_prefetch_batches, 0)
        require_integer_at_least("num_packing_bins", self.num_packing_bins, 1)

    def attention_mask_type(self) -> str:
        """`block_causal` when rows hold several documents, else `causal`
        (reference: config/data_config.py:149-159)."""
        if self.dataset == "random":
            return "causal"
        if self.dataset == "random_packed":
            return "block_causal"
        return "block_causal" if self.max_num_documents != 1 else "causal"
