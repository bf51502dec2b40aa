"""Model building blocks shared by every family: Linear / RMSNorm over the kernel layer, gated MLP, target helpers
(reference: llmtuner/models/common/linear.py, activation.py, targets.py)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops

IGNORE_INDEX = ops.IGNORE_INDEX


def next_token_targets(labels: torch.Tensor) -> torch.Tensor:
    """Unshifted labels [B, S] -> targets [B, S] where position t predicts token t+1 and the last position is ignored."""
    t = torch.full_like(labels, IGNORE_INDEX)
    t[..., :-1] = labels[..., 1:]
    return t


class Linear(nn.Module):
    """Bias-free linear over `ops.linear` (tcgen05 GEMM on CUDA bf16)."""

    def __init__(self, in_features: int, out_features: int, dtype=None, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))

    def forward(self, x):
        return ops.linear(x, self.weight)

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}"


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, dtype=None, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x, residual=None):
        if residual is None:
            return ops.rms_norm(x, self.weight, self.eps)
        return ops.add_rms_norm(x, residual, self.weight, self.eps)


class GatedMLP(nn.Module):
    """down(silu(gate(x)) * up(x))"""

    def __init__(self, hidden: int, inter: int, dtype=None, device=None):
        super().__init__()
        self.gate_proj = Linear(hidden, inter, dtype, device)
        self.up_proj = Linear(hidden, inter, dtype, device)
        self.down_proj = Linear(inter, hidden, dtype, device)

    accepts_sharded_rows = True     # `x` may be a row-sharded handle whose `linears` gathers inside the first GEMM

    def forward(self, x):
        if hasattr(x, "linears"):
            g, u = x.linears(self.gate_proj.weight, self.up_proj.weight)
            return self.down_proj(ops.swiglu(g, u))
        g, u = ops.linears(x, self.gate_proj.weight, self.up_proj.weight)
        return self.down_proj(ops.swiglu(g, u))


class Embedding(nn.Module):
    def __init__(self, vocab: int, dim: int, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim, dtype=dtype, device=device))

    def forward(self, ids):
        return torch.nn.functional.embedding(ids, self.weight)
