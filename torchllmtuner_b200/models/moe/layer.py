"""Sparse MoE block with aux-loss-free bias balancing (reference: llmtuner/models/common/moe/layer.py:88-309,
bias_update.py:36-291, auxiliary_loss.py:31-168).

Persistent fp32 buffers `expert_bias_E` and `tokens_per_expert_E`. Once per optimizer step the token counts are
all-reduced over the data ranks and `bias += delta - mean(delta)` with `delta = coeff * sign(mean(counts) - counts)`.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .experts import GroupedExperts, RoutedExperts
from .routing import HashRouter, QuantileBalancedTopKRouter, TokenChoiceTopKRouter


class MoE(nn.Module):
    always_bias = False     # True: the selection bias is applied even when it is not being updated (loaded from a checkpoint)

    def __init__(self, hidden: int, num_experts: int, top_k: int, moe_inter: int, *, shared_inter: int = 0,
                 score_fn: str = "softmax", norm_topk_prob: bool = True, route_scale: float = 1.0,
                 bias_update_coeff: float = 0.0, aux_loss_coef: float = 0.0, quantile_balancing: bool = False,
                 fixed_router: bool = False, experts_implementation: str = "native", dtype=None, device=None,
                 shared_mlp_factory=None, swiglu_limit: float | None = None, hash_vocab_size: int = 0, num_groups: int = 1,
                 topk_groups: int = 1, expert_width: int | None = None, glu_fn=None, shared_gate: bool = False):
        super().__init__()
        if hash_vocab_size:
            self.router = HashRouter(hidden, num_experts, top_k, hash_vocab_size, score_fn, norm_topk_prob, route_scale, dtype=dtype,
                                     device=device)
        else:
            rcls = QuantileBalancedTopKRouter if quantile_balancing else TokenChoiceTopKRouter
            kw = {} if quantile_balancing else dict(num_groups=num_groups, topk_groups=topk_groups)
            self.router = rcls(hidden, num_experts, top_k, score_fn, norm_topk_prob, route_scale, fixed=fixed_router, dtype=dtype,
                               device=device, **kw)
        self.hash_routed = bool(hash_vocab_size)
        # `expert_width`: the experts work in a narrower latent space; the block projects into and out of it
        self.routed = RoutedExperts(GroupedExperts(num_experts, expert_width or hidden, moe_inter, dtype=dtype, device=device,
                                                   implementation=experts_implementation, swiglu_limit=swiglu_limit, glu_fn=glu_fn))
        self.shared_experts = shared_mlp_factory(shared_inter) if (shared_inter and shared_mlp_factory) else None
        # Qwen3.5: the shared expert's output is scaled per token by sigmoid(w_g . x)
        self.shared_expert_gate = None
        if shared_gate and self.shared_experts is not None:
            from ..common import Linear
            self.shared_expert_gate = Linear(hidden, 1, dtype, device)
        self.num_experts, self.top_k = num_experts, top_k
        self.bias_update_coeff, self.aux_loss_coef = bias_update_coeff, aux_loss_coef
        self.register_buffer("expert_bias_E", torch.zeros(num_experts, dtype=torch.float32, device=device), persistent=True)
        self.register_buffer("tokens_per_expert_E", torch.zeros(num_experts, dtype=torch.float32, device=device), persistent=True)
        self.aux_loss: torch.Tensor | None = None
        self.router.need_scores = aux_loss_coef > 0      # the balance loss needs the full score matrix
        self.dispatch_timer = None

    @property
    def gate(self):          # HF-style name of the router projection
        return self.router.gate

    @property
    def experts(self):
        return self.routed.experts

    def forward(self, x: torch.Tensor, token_ids: torch.Tensor | None = None) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        bias = self.expert_bias_E if (self.bias_update_coeff > 0 or self.always_bias) else None
        w, idx, counts, scores = self.router(x2, bias, token_ids=token_ids) if self.hash_routed else self.router(x2, bias)
        if self.training and torch.is_grad_enabled():
            with torch.no_grad():
                self.tokens_per_expert_E.add_(counts)
        if self.aux_loss_coef > 0 and self.training:
            self.aux_loss = self.aux_loss_coef * self.balance_loss_sum(counts, scores)
        out = self.routed_output(self.routed(self.routed_input(x2), w, idx))
        if self.shared_experts is not None:
            sh = self.shared_experts(x2)
            if self.shared_expert_gate is not None:
                sh = sh * torch.sigmoid(self.shared_expert_gate(x2))
            out = out + sh
        return out.reshape(shape)

    def routed_input(self, x2: torch.Tensor) -> torch.Tensor:
        """What the routed experts consume; the router and the shared expert always see the block's input."""
        return x2

    def routed_output(self, y: torch.Tensor) -> torch.Tensor:
        return y

    def balance_loss_sum(self, counts: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
        """Micro-batch load-balance loss in its token-sum form, T * L_bal (reference:
        llmtuner/models/common/moe/auxiliary_loss.py:31-168; DeepSeek-V3 eqs. 17-20).

        f_i = E * counts_i / sum_j counts_j (not differentiable), P_i = sum_t s'_{t,i} with s' the scores L1-normalised
        per token, value sum_i f_i * P_i. It is a sum over this forward's tokens, so the caller divides it by the global
        valid-token count exactly like the token loss: the injected weight is then `coef * L_bal` per token stream whatever
        the data-parallel degree or the number of accumulation steps. Counts and score sums are partial over the ranks that
        hold pieces of ONE token stream (`self.stream_groups`: the context-parallel group, and the tensor-parallel group
        when the experts are expert-parallel); they are all-reduced forward with an identity backward. Data-parallel ranks
        own independent streams and are not reduced."""
        from ...accelerator.collectives import PartialToInvariantAllReduce
        probs = scores / scores.sum(-1, keepdim=True).clamp_min(1e-12)
        p_sum = probs.sum(0)
        counts = counts.detach().to(p_sum.dtype)
        for grp in getattr(self, "stream_groups", ()) or ():
            counts = PartialToInvariantAllReduce.apply(counts, grp)
            p_sum = PartialToInvariantAllReduce.apply(p_sum, grp)
        f = counts / counts.sum().clamp_min(1.0) * self.num_experts
        return (f.detach() * p_sum).sum()

    @torch.no_grad()
    def update_expert_bias(self, reduce_fn=None) -> None:
        """`reduce_fn(counts)` all-reduces the counts over the data ranks (identity on one rank)."""
        counts = self.tokens_per_expert_E
        if reduce_fn is not None:
            counts = reduce_fn(counts)
        if self.bias_update_coeff > 0:
            delta = self.bias_update_coeff * torch.sign(counts.mean() - counts)
            self.expert_bias_E.add_(delta - delta.mean())
        self.tokens_per_expert_E.zero_()


def moe_blocks(model: nn.Module):
    return [m for m in model.modules() if isinstance(m, MoE)]


def collect_aux_loss(model: nn.Module):
    total = None
    for m in moe_blocks(model):
        if m.aux_loss is not None:
            total = m.aux_loss if total is None else total + m.aux_loss
            m.aux_loss = None
    return total


def routing_load_metrics(model: nn.Module) -> dict[str, float]:
    out = {}
    for i, m in enumerate(moe_blocks(model)):
        c = m.tokens_per_expert_E
        if c.sum() > 0:
            out[f"moe/layer{i}/max_over_mean"] = float(c.max() / c.mean().clamp_min(1e-9))
    return out
