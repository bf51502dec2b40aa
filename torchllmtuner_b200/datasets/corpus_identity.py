"""Stable identity of a corpus + tokenizer + packing setup (reference: llmtuner/datasets/corpus_identity.py:18-102);
stored with the data cursor so that a resume against different data is refused."""
from __future__ import annotations

import hashlib
import os


def corpus_data_identity(data_cfg, tokenizer_identity: str, paths=()) -> str:
    if data_cfg.data_identity:
        return data_cfg.data_identity
    h = hashlib.sha256()
    for k in ("dataset", "packing", "num_packing_bins", "max_num_documents", "prompt_field", "response_field", "text_field",
              "messages_field", "chat_template"):
        h.update(f"{k}={getattr(data_cfg, k, None)};".encode())
    h.update(tokenizer_identity.encode())
    for p in sorted(paths):
        st = os.stat(p)
        h.update(f"{os.path.basename(p)}:{st.st_size};".encode())
        with open(p, "rb") as f:
            h.update(f.read(1 << 20))
    return h.hexdigest()[:24]
