"""Tokenizers (reference: llmtuner/components/tokenizer/*.py): a small base contract, a Hugging Face `tokenizers`
back end with BOS/EOS inference and chat templates, a whitespace tokenizer for tests and offline fixtures, and thin
Kimi / multimodal adapters."""
from .base import BaseTokenizer  # noqa: F401
from .huggingface import HuggingFaceTokenizer, build_tokenizer  # noqa: F401
from .whitespace import WhitespaceTokenizer  # noqa: F401
