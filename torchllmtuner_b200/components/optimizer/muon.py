"""Distributed Muon over flat shards (reference: llmtuner/components/optimizer/flex_shard/dist_muon.py:181-2088,
_optimizer_reshard_runtime.py:108-879, optimizer_reshard.py).

Matrices (2-D parameters of the decoder blocks) take the Muon update: momentum 0.95 (Nesterov), five Newton-Schulz
iterations in bf16 with coefficients (3.4445, -4.7750, 2.0315), decoupled weight decay. Every other parameter
(embedding, head, norms, routers, packed experts) takes AdamW. Storage stays the flat fp32 shard layout of the FSDP
units. Newton-Schulz needs whole matrices, so per unit the momentum-updated gradient shards are gathered once
(storage -> compute), each matrix is orthogonalised by exactly one owner rank (owners balanced by matrix size, the same
plan on every rank, checked by a plan hash), and the owners' results are summed back so that every rank can update the
slice it stores (compute -> storage). The products run on the tcgen05 GEMM on CUDA."""
from __future__ import annotations

import hashlib
import re

import torch
import torch.distributed as dist

from ... import ops
from .sharded import ShardedAdamW

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Orthogonalise a matrix: X <- aX + (bA + cA^2)X with A = XX^T, on the shorter side, in bf16."""
    a, b, c = NS_COEFFS
    x = g.to(torch.bfloat16)
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t().contiguous()
    x = x / (x.float().norm() + eps).to(x.dtype)
    use_kernel = x.is_cuda and x.shape[0] % 8 == 0 and x.shape[1] % 8 == 0
    for _ in range(steps):
        if use_kernel:
            A = ops.gemm(x, x)                               # X X^T
            B = (b * A.float() + c * ops.gemm(A, A).float()).to(torch.bfloat16)
            x = (a * x.float() + ops.gemm(B, x, b_mn=True).float()).to(torch.bfloat16)
        else:
            xf = x.float()
            A = xf @ xf.t()
            x = (a * xf + (b * A + c * (A @ A)) @ xf).to(torch.bfloat16)
    return x.t().contiguous() if transposed else x


def adjusted_lr(lr: float, shape, mode: str) -> float:
    m, n = shape
    if mode == "original":
        return lr * max(1.0, m / n) ** 0.5
    if mode == "match_rms_adamw":
        return lr * 0.2 * max(m, n) ** 0.5
    if mode == "spectral_unclamped":
        return lr * (m / n) ** 0.5
    raise ValueError(mode)


class DistMuon:
    def __init__(self, rt, *, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5, eps: float = 1e-7, betas=(0.9, 0.999), adjust_lr: str = "original", adamw_lr: float | None = None,
                 muon_pattern: str = r"layers\.\d+\..*(proj|gate_proj|up_proj|down_proj)\.weight$", param_group_rules=None):
        self.rt, self.units = rt, list(rt.units)
        self.momentum, self.nesterov, self.ns_steps, self.eps, self.adjust = momentum, nesterov, ns_steps, eps, adjust_lr
        self.param_groups = [dict(lr=lr, weight_decay=weight_decay, name="muon", param_names=[])]
        self.pattern = re.compile(muon_pattern)
        self.step_count = 0
        self.state: dict[str, dict[str, torch.Tensor]] = {}
        # matrices per unit: (fqn, offset, shape) ; everything else is AdamW (same flat shards, masked by ranges)
        self.matrices: dict[str, list[tuple[str, int, tuple]]] = {}
        plan = []
        for u in self.units:
            ms = [(s.fqn, s.offset, tuple(s.shape)) for s in u.slots if len(s.shape) == 2 and self.pattern.search(s.fqn) and not u.is_expert]
            self.matrices[u.name] = ms
            self.state[u.name] = {"momentum_buffer": torch.zeros(u.shard_numel, dtype=torch.float32, device=u.master.device)}
            self.param_groups[0]["param_names"] += [m[0] for m in ms]
            plan += [f"{u.name}:{m[0]}:{m[2]}" for m in ms]
        self.plan_hash = hashlib.sha256("|".join(plan).encode()).hexdigest()[:16]
        if dist.is_initialized() and rt.world > 1:
            hashes = [None] * dist.get_world_size(rt.group)
            dist.all_gather_object(hashes, self.plan_hash, group=rt.group)
            if len(set(hashes)) != 1:
                raise RuntimeError(f"ranks disagree on the Muon compute plan: {hashes}")
        self.adamw = ShardedAdamW(self.units, lr=adamw_lr or lr, betas=betas, eps=1e-8, weight_decay=0.0, param_group_rules=param_group_rules)
        self.param_groups += self.adamw.param_groups
        for u in self.units:
            self.state[u.name].update(self.adamw.state[u.name])

    def zero_grad(self) -> None:
        for u in self.units:
            u.has_grad = False

    def _owner(self, idx: int, world: int) -> int:
        return idx % world

    @torch.no_grad()
    def step(self, clip_coef=None) -> None:
        self.step_count += 1
        g0 = self.param_groups[0]
        coef = 1.0 if clip_coef is None else clip_coef
        # AdamW part first: it updates every element; Muon ranges are then overwritten from a snapshot of the
        # pre-update master values, so the two never mix on one element.
        snap = {u.name: u.master.clone() for u in self.units if self.matrices[u.name] and u.has_grad}
        self.adamw.step(clip_coef)
        for u in self.units:
            ms = self.matrices[u.name]
            if not ms or not u.has_grad:
                continue
            buf = self.state[u.name]["momentum_buffer"]
            g = u.grad_shard.float() * coef
            buf.mul_(self.momentum).add_(g)
            upd = g.add(buf, alpha=self.momentum) if self.nesterov else buf.clone()
            if u.world > 1:
                full = torch.empty(u.padded, dtype=torch.float32, device=upd.device)
                dist.all_gather_into_tensor(full, upd, group=u.group)
            else:
                full = upd
            out = torch.zeros_like(full)
            for i, (fqn, off, shape) in enumerate(ms):
                if self._owner(i, u.world) != u.rank:
                    continue
                n = shape[0] * shape[1]
                o = newton_schulz(full[off:off + n].view(shape), self.ns_steps, self.eps).float()
                out[off:off + n] = (o * (adjusted_lr(g0["lr"], shape, self.adjust) / max(g0["lr"], 1e-30))).reshape(-1)
            if u.world > 1:
                mine = torch.empty(u.shard_numel, dtype=torch.float32, device=out.device)
                dist.reduce_scatter_tensor(mine, out, group=u.group)
            else:
                mine = out
            a, _ = u.my_range()
            pre = snap[u.name]
            for fqn, off, shape in ms:
                lo, hi = max(a, off), min(a + u.shard_numel, off + shape[0] * shape[1])
                if hi <= lo:
                    continue
                sl = slice(lo - a, hi - a)
                u.master[sl] = pre[sl] * (1.0 - g0["lr"] * g0["weight_decay"]) - g0["lr"] * mine[sl]
            if u.separate_master:
                u.shard_lowp.copy_(u.master)
