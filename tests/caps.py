"""Capability gates for tests (the reference's `tests/caps.py:78-154` plays the same role): a test names what it needs,
and where that is absent it is skipped with a message that says what is missing. `pytest -rs` then doubles as the report of
what this environment could not check."""
import importlib.util

import pytest

_PACKAGES = {"fsspec": "fsspec", "safetensors": "safetensors", "tokenizers": "tokenizers", "datasets": "datasets",
             "tensorboard": "tensorboard", "jinja2": "jinja2", "yaml": "yaml", "transformers": "transformers"}


def available(name: str) -> bool:
    """A package from `_PACKAGES` or a capability of `torchllmtuner_b200.accelerator.capabilities`."""
    if name in _PACKAGES:
        return importlib.util.find_spec(_PACKAGES[name]) is not None
    from torchllmtuner_b200.accelerator import capabilities
    return capabilities.has(name)


def missing(*names: str) -> list[str]:
    return [n for n in names if not available(n)]


def require_env(*names: str) -> None:
    """Module level: skip the whole module unless everything named is there."""
    lack = missing(*names)
    if lack:
        pytest.skip(f"[env] missing: {', '.join(lack)}", allow_module_level=True)


def skip_without(*names: str):
    """Decorator for one test."""
    lack = missing(*names)
    return pytest.mark.skipif(bool(lack), reason=f"[env] missing: {', '.join(lack)}")
