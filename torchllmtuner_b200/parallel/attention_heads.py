"""Head-count checks shared by the stages that cut attention by heads
(reference: llmtuner/parallel/attention_heads.py:34-80)."""
from __future__ import annotations

from ..errors import UnsupportedCombinationError


def head_counts(model) -> list[tuple[str, int]]:
    """(config field, count) for query and key/value heads of `model.config`; a configuration that does not name its
    key/value heads has one per query head. Empty when the model has no head counts at all."""
    cfg = getattr(model, "config", None)
    n = getattr(cfg, "num_attention_heads", None)
    if n is None:
        return []
    kv = getattr(cfg, "num_key_value_heads", None)
    out = [("num_attention_heads", n), ("num_key_value_heads", n if kv is None else kv)]
    for name, c in out:
        if isinstance(c, bool) or not isinstance(c, int) or c < 1:
            raise ValueError(f"{name} must be a positive integer, got {c!r}")
    return out


def require_heads_divisible_by(model, *, size: int, axis: str, why: str) -> None:
    """Raises unless `size` divides every head count. `axis` names the degree (`tp`, `tp*cp_ulysses`), `why` says in one
    line why that axis cuts heads, so each caller's message carries its own reason. A size of 1 is never checked."""
    if type(size) is not int or size < 1:
        raise ValueError(f"{axis} degree must be a positive integer, got {size!r}")
    if size == 1:
        return
    for name, c in head_counts(model):
        if c % size:
            raise UnsupportedCombinationError(f"{name} ({c}) must be divisible by {axis} ({size}): {why}")
