"""Peak-FLOPS table used for MFU (reference: llmtuner/utils/monitoring.py:146-236).

The table value for B200 is the nominal dense bf16 figure (2.25e15). A second denominator, the
cuBLAS bf16 throughput measured on the machine, can be supplied through the
`LLMT_MEASURED_PEAK_TFLOPS` environment variable or a `MEASURED_PEAKS.json` beside the package.
"""
from __future__ import annotations

import json
import os

_TABLE = (
    ("GB200", 2.5e15), ("GB300", 2.5e15), ("B200", 2.25e15), ("B300", 2.25e15), ("B100", 1.8e15),
    ("H200", 989e12), ("H100 PCIe", 756e12), ("H100 NVL", 835e12), ("H100", 989e12), ("H800", 989e12),
    ("A100", 312e12), ("A800", 312e12), ("L40S", 362e12), ("MI300X", 1300e12), ("910", 376e12),
)


def get_peak_flops(device_name: str | None = None) -> float:
    """Peak dense bf16 FLOP/s by device name; 0.0 means unknown (MFU is then suppressed)."""
    if device_name is None:
        import torch
        if not torch.cuda.is_available():
            return 0.0
        device_name = torch.cuda.get_device_name()
    for key, val in _TABLE:
        if key.lower() in device_name.lower():
            return val
    return 0.0


def get_measured_peak_flops() -> float:
    """Sustained cuBLAS bf16 FLOP/s measured on this machine, 0.0 when no record exists."""
    env = os.environ.get("LLMT_MEASURED_PEAK_TFLOPS")
    if env:
        return float(env) * 1e12
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                return float(json.load(f).get("bf16_tflops_sustained", 0.0)) * 1e12
        except (OSError, ValueError):
            return 0.0
    return 0.0
