"""Token-choice top-k routers (reference: llmtuner/models/common/moe/routing.py:31-345,
llmtuner/models/qwen/routing.py:20-78).

scores = f(fp32 logits) with f in {softmax, sigmoid, sqrtsoftplus}; the load-balancing bias enters the selection only,
never the combine weights; optional node-limited groups; renormalisation with +1e-20; `route_scale`; a fixed
round-robin router for debugging; a quantile-balanced variant that shifts logits by running per-expert quantiles.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...ops import reference as ref


class RouterGateLinear(nn.Module):
    """Router projection with fp32 output (reference: llmtuner/models/common/linear.py:104-183)."""

    def __init__(self, hidden: int, num_experts: int, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, hidden, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and x.dtype == torch.bfloat16:
            return _RouterGate.apply(x, self.weight)
        return torch.mm(x.float(), self.weight.float().t())


class _RouterGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return ops.gemm(x, w, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dl):
        x, w = ctx.saved_tensors
        d16 = dl.to(torch.bfloat16)
        dx = ops.gemm(d16, w, b_mn=True)
        dw = ops.gemm(d16, x, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


class _RouterTopK(torch.autograd.Function):
    """Fused score / biased top-k / renormalise / histogram kernel with its hand-written backward."""

    @staticmethod
    def forward(ctx, logits, bias, k, score_fn, renorm, route_scale):
        from ...ops.cuda_ext import load
        fn = 0 if score_fn == "softmax" else 1
        w, idx, counts, denom = load().router_topk(logits.contiguous(), bias, k, fn, renorm, route_scale)
        ctx.save_for_backward(logits, idx, denom)
        ctx.cfg = (fn, renorm, route_scale)
        ctx.mark_non_differentiable(idx, counts)
        return w, idx, counts

    @staticmethod
    def backward(ctx, dw, _di, _dc):
        from ...ops.cuda_ext import load
        logits, idx, denom = ctx.saved_tensors
        fn, renorm, scale = ctx.cfg
        return load().router_topk_bwd(logits.contiguous(), dw.float(), idx, denom, fn, renorm, scale), None, None, None, None, None


class TokenChoiceTopKRouter(nn.Module):
    def __init__(self, hidden: int, num_experts: int, top_k: int, score_fn: str = "softmax", norm_topk_prob: bool = True,
                 route_scale: float = 1.0, num_groups: int = 1, topk_groups: int = 1, fixed: bool = False, dtype=None,
                 device=None):
        super().__init__()
        self.gate = RouterGateLinear(hidden, num_experts, dtype=dtype, device=device)
        self.num_experts, self.top_k, self.score_fn = num_experts, top_k, score_fn
        self.norm_topk_prob, self.route_scale = norm_topk_prob, route_scale
        self.num_groups, self.topk_groups, self.fixed = num_groups, topk_groups, fixed

    @property
    def weight(self):
        return self.gate.weight

    def forward(self, x: torch.Tensor, expert_bias: torch.Tensor | None = None):
        """x [T, D] -> (weights [T,k] fp32, indices [T,k] int64, counts [E] fp32, scores [T,E] fp32)."""
        logits = self.gate(x)
        if (logits.is_cuda and not self.fixed and self.num_groups == 1 and self.score_fn in ("softmax", "sigmoid")
                and self.num_experts <= 512 and self.top_k <= 16):
            bias = expert_bias.float().contiguous() if expert_bias is not None else None
            w, idx, counts = _RouterTopK.apply(logits, bias, self.top_k, self.score_fn, self.norm_topk_prob, self.route_scale)
            return w, idx, counts, (ref.router_scores(logits, self.score_fn) if self.training and getattr(self, "need_scores", False) else None)
        scores = ref.router_scores(logits, self.score_fn)
        if self.fixed:
            T = x.shape[0]
            idx = (torch.arange(T, device=x.device)[:, None] * self.top_k + torch.arange(self.top_k, device=x.device)[None, :]) % self.num_experts
        else:
            sel = scores if expert_bias is None else scores + expert_bias.float()[None, :]
            if self.num_groups > 1:
                T = sel.shape[0]
                grp = sel.view(T, self.num_groups, -1)
                gscore = grp.topk(min(2, grp.shape[-1]), dim=-1).values.sum(-1) if expert_bias is not None else grp.amax(-1)
                keep = gscore.topk(self.topk_groups, dim=-1).indices
                mask = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, keep, True)
                sel = grp.masked_fill(~mask[..., None], float("-inf")).view(T, -1)
            idx = torch.topk(sel.detach(), self.top_k, dim=-1, sorted=True).indices
        w = scores.gather(-1, idx)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * self.route_scale
        counts = torch.zeros(self.num_experts, dtype=torch.float32, device=x.device)
        counts.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x.device))
        return w, idx, counts, scores


class HashRouter(TokenChoiceTopKRouter):
    """Experts come from a persistent token-id table `tid2eid` [vocab, k] instead of a top-k; the learned projection
    still scores them, so the combine weights (and the projection's gradient) are those of the looked-up experts
    (reference: llmtuner/models/deepseek/deepseek_v4/routing.py:60-85). The caller passes the token ids of the rows."""

    def __init__(self, hidden: int, num_experts: int, top_k: int, vocab_size: int, score_fn: str = "sqrtsoftplus",
                 norm_topk_prob: bool = True, route_scale: float = 1.0, dtype=None, device=None):
        super().__init__(hidden, num_experts, top_k, score_fn, norm_topk_prob, route_scale, dtype=dtype, device=device)
        self.register_buffer("tid2eid", torch.zeros(vocab_size, top_k, dtype=torch.int64, device=device), persistent=True)

    @torch.no_grad()
    def fill_table(self, seed: int = 0) -> None:
        """A fixed pseudo-random table with k distinct experts per token id (pre-trained checkpoints bring their own)."""
        g = torch.Generator().manual_seed(seed)
        V, k = self.tid2eid.shape
        self.tid2eid.copy_(torch.rand(V, self.num_experts, generator=g).topk(k, dim=-1).indices.to(self.tid2eid.device))

    def forward(self, x: torch.Tensor, expert_bias=None, token_ids: torch.Tensor | None = None):
        if token_ids is None:
            raise ValueError("a hash-routed block needs the token ids of its rows")
        scores = ref.router_scores(self.gate(x), self.score_fn)
        idx = self.tid2eid[token_ids.reshape(-1)]
        w = scores.gather(-1, idx)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        counts = torch.zeros(self.num_experts, dtype=torch.float32, device=x.device)
        counts.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x.device))
        return w * self.route_scale, idx, counts, scores


class QuantileBalancer(nn.Module):
    """Running per-expert logit quantiles from a 1000-bin histogram (reference: routing.py:491)."""

    def __init__(self, num_experts: int, top_k: int, bins: int = 1000, lo: float = -20.0, hi: float = 20.0, momentum: float = 0.9):
        super().__init__()
        self.bins, self.lo, self.hi, self.momentum = bins, lo, hi, momentum
        self.target = 1.0 - top_k / num_experts
        self.register_buffer("threshold_E", torch.zeros(num_experts, dtype=torch.float32))

    @torch.no_grad()
    def update(self, logits: torch.Tensor) -> None:
        E = logits.shape[1]
        width = (self.hi - self.lo) / self.bins
        b = ((logits.float() - self.lo) / width).clamp_(0, self.bins - 1).long()
        hist = torch.zeros(E, self.bins, device=logits.device)
        hist.scatter_add_(1, b.t().contiguous(), torch.ones_like(b.t(), dtype=torch.float32))
        cdf = hist.cumsum(1) / max(1, logits.shape[0])
        q = (cdf < self.target).sum(1).float() * width + self.lo
        self.threshold_E.mul_(self.momentum).add_(q, alpha=1 - self.momentum)


class QuantileBalancedTopKRouter(TokenChoiceTopKRouter):
    """Selection on logits shifted by each expert's running quantile, so every expert fires at about the same rate."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.balancer = QuantileBalancer(self.num_experts, self.top_k)

    def forward(self, x, expert_bias=None):
        logits = self.gate(x)
        if self.training:
            self.balancer.update(logits.detach())
        scores = ref.router_scores(logits, self.score_fn)
        sel = logits.detach().float() - self.balancer.threshold_E[None, :]
        idx = torch.topk(sel, self.top_k, dim=-1, sorted=True).indices
        w = scores.gather(-1, idx)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        counts = torch.zeros(self.num_experts, dtype=torch.float32, device=x.device)
        counts.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x.device))
        return w * self.route_scale, idx, counts, scores
