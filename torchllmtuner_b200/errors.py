"""Framework error taxonomy.

Three user-facing classes under one root, mirroring the reference's taxonomy
(reference: llmtuner/errors.py:41-54): a bad value (`ConfigError`), a valid value
whose combination with another feature is not supported (`UnsupportedCombinationError`)
and a missing capability of the machine (`EnvironmentUnsupportedError`).
"""
from __future__ import annotations


class LLMTunerError(Exception):
    """Root of every error raised on purpose by this framework."""


class ConfigError(LLMTunerError, ValueError):
    """A configuration value is invalid on its own or against another group."""


class UnsupportedCombinationError(LLMTunerError, NotImplementedError):
    """Two features are individually valid but cannot be combined."""


class EnvironmentUnsupportedError(LLMTunerError, RuntimeError):
    """The machine (device, library, driver) lacks what the request needs."""


class KernelStatusError(LLMTunerError, RuntimeError):
    """A device kernel returned a non-zero status word (bounded wait expired,
    capacity overflow, bad argument detected on the device)."""

    def __init__(self, kernel: str, code: int, detail: str = ""):
        self.kernel, self.code, self.detail = kernel, code, detail
        super().__init__(f"kernel {kernel!r} reported status {code}: {detail}")
