"""torchllmtuner_b200: a B200-native hybrid-parallel LLM training framework.

Public surface (lazy): `LLMTunerConfig`, `Trainer`; `python -m torchllmtuner_b200 --flag value ...` runs the CLI."""
__version__ = "0.1.0"

_EXPORTS = {"LLMTunerConfig": ".config", "Trainer": ".trainer"}


def __getattr__(name):
    if name in _EXPORTS:
        import importlib
        return getattr(importlib.import_module(_EXPORTS[name], __name__), name)
    raise AttributeError(name)


__all__ = sorted(_EXPORTS)
