"""Hugging Face `tokenizers` back end (reference: llmtuner/components/tokenizer/huggingface.py:19-445): loads
`tokenizer.json`, infers BOS/EOS from `tokenizer_config.json` / `special_tokens_map.json` / `config.json`, renders chat
templates with jinja when the folder ships one."""
from __future__ import annotations

import hashlib
import json
import os

from ...errors import ConfigError
from .base import BaseTokenizer


class HuggingFaceTokenizer(BaseTokenizer):
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        tj = os.path.join(path, "tokenizer.json") if os.path.isdir(path) else path
        if not os.path.exists(tj):
            raise ConfigError(f"no tokenizer.json under {path}")
        self.path = os.path.dirname(tj)
        self.tok = Tokenizer.from_file(tj)
        self._cfg = self._read("tokenizer_config.json")
        smap = self._read("special_tokens_map.json")
        mcfg = self._read("config.json")
        self.bos_token = self._special(self._cfg.get("bos_token") or smap.get("bos_token"))
        self.eos_token = self._special(self._cfg.get("eos_token") or smap.get("eos_token"))
        self.pad_token = self._special(self._cfg.get("pad_token") or smap.get("pad_token"))
        self.bos_id = self.tok.token_to_id(self.bos_token) if self.bos_token else mcfg.get("bos_token_id")
        self.eos_id = self.tok.token_to_id(self.eos_token) if self.eos_token else mcfg.get("eos_token_id")
        self.pad_id = self.tok.token_to_id(self.pad_token) if self.pad_token else self.eos_id
        self.chat_template = self._cfg.get("chat_template")
        with open(tj, "rb") as f:
            self._hash = hashlib.sha256(f.read()).hexdigest()[:16]

    def _read(self, name: str) -> dict:
        p = os.path.join(self.path, name)
        if os.path.exists(p):
            with open(p) as f:
                return json.load(f)
        return {}

    @staticmethod
    def _special(v):
        return v.get("content") if isinstance(v, dict) else v

    def encode(self, text, add_bos=False, add_eos=False):
        ids = self.tok.encode(text, add_special_tokens=False).ids
        if add_bos and self.bos_id is not None:
            ids = [self.bos_id] + ids
        if add_eos and self.eos_id is not None:
            ids = ids + [self.eos_id]
        return ids

    def decode(self, ids):
        return self.tok.decode(list(ids))

    @property
    def vocab_size(self):
        return self.tok.get_vocab_size()

    def apply_chat_template(self, messages, add_generation_prompt=False, **kw):
        if not self.chat_template:
            return super().apply_chat_template(messages, add_generation_prompt, **kw)
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(message):                     # templates call this for malformed conversations
            raise ConfigError(f"chat template: {message}")
        # the environment published templates are written for: sandboxed, loop controls, `tojson` that keeps unicode
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
        env.globals["raise_exception"] = raise_exception
        env.filters["tojson"] = lambda v, indent=None: json.dumps(v, ensure_ascii=False, indent=indent)
        del jinja2
        return env.from_string(self.chat_template).render(messages=messages, add_generation_prompt=add_generation_prompt,
                                                          bos_token=self.bos_token or "", eos_token=self.eos_token or "", **kw)

    def identity(self):
        return "hf:" + self._hash


class KimiK3Tokenizer(HuggingFaceTokenizer):
    """Kimi ships a tiktoken-style vocabulary; when a converted `tokenizer.json` is present it is used as is."""


class MultimodalTokenizer:
    """Wraps a text tokenizer and knows the ids of the vision placeholder tokens."""

    def __init__(self, inner: BaseTokenizer, data_cfg):
        self.inner = inner
        enc = lambda t: (inner.encode(t) or [None])[0]  # noqa: E731
        self.image_id, self.video_id = enc(data_cfg.mm_image_token), enc(data_cfg.mm_video_token)
        self.vision_start_id, self.vision_end_id = enc(data_cfg.mm_vision_start_token), enc(data_cfg.mm_vision_end_token)

    def __getattr__(self, name):
        return getattr(self.inner, name)


def build_tokenizer(data_cfg) -> BaseTokenizer:
    from .whitespace import WhitespaceTokenizer
    if data_cfg.tokenizer_backend == "whitespace":
        if not data_cfg.tokenizer_path:
            raise ConfigError("tokenizer_backend='whitespace' needs tokenizer_path (a vocabulary json)")
        return WhitespaceTokenizer.from_file(data_cfg.tokenizer_path)
    if not data_cfg.tokenizer_path:
        raise ConfigError(f"dataset {data_cfg.dataset!r} needs tokenizer_path")
    cls = KimiK3Tokenizer if data_cfg.tokenizer_backend == "kimi_k3" else HuggingFaceTokenizer
    return cls(data_cfg.tokenizer_path)
