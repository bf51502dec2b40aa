"""Grouped experts and token dispatch on one rank (reference: llmtuner/models/common/moe/experts.py:73-343,
llmtuner/parallel/expert_parallel/token_dispatch.py:127-275).

Weights are kept in the native packed layout `w1_EFD` (gate), `w3_EFD` (up), `w2_EDF` (down). Token copies are
sorted by expert into 128-row aligned segments (padding rows are zero), which lets the grouped tcgen05 GEMM tile
without ever crossing an expert boundary in M (forward, dgrad) or in K (wgrad).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ... import ops
from ...ops import reference as ref
from ...ops.cuda_ext import load as _ext

SEG_ALIGN = 128


def padded_capacity(num_copies: int, num_experts: int) -> int:
    """Static upper bound of padded rows: every expert wastes at most SEG_ALIGN-1 rows."""
    cap = num_copies + num_experts * (SEG_ALIGN - 1)
    return -(-cap // SEG_ALIGN) * SEG_ALIGN


def plan_segments(flat_expert: torch.Tensor, num_experts: int):
    """From the expert id of each token copy: (dest_row [n] int64 in the padded layout, seg_offsets [E+1] int32,
    counts [E] int64). Pure device ops, no host synchronisation."""
    counts = torch.bincount(flat_expert, minlength=num_experts)
    padded = (counts + (SEG_ALIGN - 1)) // SEG_ALIGN * SEG_ALIGN
    zero = counts.new_zeros(1)
    seg = torch.cat([zero, padded.cumsum(0)])
    start = torch.cat([zero, counts.cumsum(0)])[:-1]
    order = torch.argsort(flat_expert, stable=True)
    rank = torch.empty_like(order)
    rank[order] = torch.arange(order.numel(), device=order.device)
    dest = rank - start[flat_expert] + seg[:-1][flat_expert]
    return dest, seg.to(torch.int32), counts


class _GroupedLinear(torch.autograd.Function):
    """y[seg g] = x[seg g] @ w[g]^T over 128-aligned row segments."""

    @staticmethod
    def forward(ctx, x, w, seg):
        y = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        _ext().grouped_gemm(x, w, y, seg, False)
        ctx.save_for_backward(x, w, seg)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, seg = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _ext().grouped_gemm(dy, w, dx, seg, True)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)
            _ext().grouped_wgrad(dy, x, dw, seg, False)
        return dx, dw, None


def grouped_linear(x, w, seg_offsets, counts=None):
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _GroupedLinear.apply(x, w, seg_offsets)
    # CPU statement over the padded layout
    outs = x.new_zeros(x.shape[0], w.shape[1])
    seg = seg_offsets.tolist()
    for e in range(w.shape[0]):
        s, t = seg[e], seg[e + 1]
        if t > s:
            outs[s:t] = torch.nn.functional.linear(x[s:t], w[e])
    return outs


class _PermuteRows(torch.autograd.Function):
    """rows[dest[c]] = x[c // k] into a zeroed padded buffer; backward sums the k copies of every token."""

    @staticmethod
    def forward(ctx, x, dest, cap, k):
        rows = torch.zeros(cap, x.shape[1], dtype=x.dtype, device=x.device)
        _ext().permute_rows(x.contiguous(), dest, rows, k)
        ctx.save_for_backward(dest)
        ctx.k, ctx.T = k, x.shape[0]
        return rows

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        return _ext().combine_rows(g.contiguous(), dest, None, ctx.T, ctx.k), None, None, None


class _CombineRows(torch.autograd.Function):
    """out[t] = sum_j w[t, j] * y[dest[t * k + j]] in fp32."""

    @staticmethod
    def forward(ctx, y, weights, dest, T, k):
        w = weights.float().contiguous()
        ctx.save_for_backward(y, w, dest)
        ctx.k = k
        return _ext().combine_rows(y.contiguous(), dest, w, T, k)

    @staticmethod
    def backward(ctx, g):
        y, w, dest = ctx.saved_tensors
        dy, dw = _ext().combine_bwd(g, y.contiguous(), dest, w.reshape(-1), ctx.k)
        return dy, dw.view_as(w), None, None, None


class GroupedExperts(nn.Module):
    def __init__(self, num_experts: int, hidden: int, inter: int, dtype=None, device=None, implementation: str = "native",
                 swiglu_limit: float | None = None, glu_fn=None):
        super().__init__()
        # `glu_fn(gate, up) -> hidden` replaces silu(gate) * up (Kimi's bounded SituGLU); None keeps the fused kernel
        self.glu_fn = glu_fn
        self.num_experts, self.hidden, self.inter, self.implementation = num_experts, hidden, inter, implementation
        # asymmetric clamp before the gated activation: gate <= limit, |up| <= limit
        # (reference: llmtuner/models/deepseek/deepseek_v4/modeling.py:164-169)
        self.swiglu_limit = swiglu_limit
        self.w1_EFD = nn.Parameter(torch.empty(num_experts, inter, hidden, dtype=dtype, device=device))
        self.w3_EFD = nn.Parameter(torch.empty(num_experts, inter, hidden, dtype=dtype, device=device))
        self.w2_EDF = nn.Parameter(torch.empty(num_experts, hidden, inter, dtype=dtype, device=device))
        for p in (self.w1_EFD, self.w3_EFD, self.w2_EDF):
            p.is_expert = True

    def _clamp(self, g, u):
        if self.swiglu_limit is None:
            return g, u
        return g.clamp(max=self.swiglu_limit), u.clamp(min=-self.swiglu_limit, max=self.swiglu_limit)

    def forward(self, rows: torch.Tensor, seg_offsets: torch.Tensor) -> torch.Tensor:
        """rows: padded expert-major rows [R, D]; returns [R, D]."""
        if rows.shape[0] == 0:
            return rows.new_zeros(0, self.hidden) + 0.0 * (self.w1_EFD.sum() + self.w3_EFD.sum() + self.w2_EDF.sum())
        if self.implementation == "eager":
            seg = seg_offsets.tolist()
            out = rows.new_zeros(rows.shape[0], self.hidden)
            for e in range(self.w1_EFD.shape[0]):
                s, t = seg[e], seg[e + 1]
                if t > s:
                    g_, u_ = self._clamp(ops.linear(rows[s:t], self.w1_EFD[e]), ops.linear(rows[s:t], self.w3_EFD[e]))
                    h = ops.swiglu(g_, u_) if self.glu_fn is None else self.glu_fn(g_, u_)
                    out[s:t] = ops.linear(h, self.w2_EDF[e])
            return out
        g, u = self._clamp(grouped_linear(rows, self.w1_EFD, seg_offsets), grouped_linear(rows, self.w3_EFD, seg_offsets))
        # rows past the last segment of a statically sized receive buffer hold nothing: the kernels skip them
        limit = seg_offsets[-1:] if rows.is_cuda and seg_offsets.dtype == torch.int32 else None
        h = ops.swiglu(g, u, limit) if self.glu_fn is None else self.glu_fn(g, u)
        return grouped_linear(h, self.w2_EDF, seg_offsets)


class LocalTokenDispatcher:
    """All experts live on this rank: stable sort of the copies by expert, zero-padded 128-aligned segments,
    score-weighted fp32 combine."""

    def __init__(self, num_experts: int):
        self.num_experts = num_experts

    def dispatch(self, x: torch.Tensor, indices: torch.Tensor):
        T, k = indices.shape
        flat = indices.reshape(-1)
        dest, seg, counts = plan_segments(flat, self.num_experts)
        cap = padded_capacity(T * k, self.num_experts)
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
            rows = _PermuteRows.apply(x, dest, cap, k)
        else:
            tok = torch.arange(T * k, device=x.device) // k
            rows = x.new_zeros(cap, x.shape[1]).index_copy(0, dest, x.index_select(0, tok))
        return rows, seg, {"dest": dest, "T": T, "k": k}

    def combine(self, y: torch.Tensor, weights: torch.Tensor, state) -> torch.Tensor:
        T, k = state["T"], state["k"]
        if y.is_cuda and y.dtype == torch.bfloat16 and y.shape[1] % 8 == 0:
            return _CombineRows.apply(y, weights, state["dest"], T, k)
        g = y.index_select(0, state["dest"]).view(T, k, -1)
        return (g.float() * weights.float().unsqueeze(-1)).sum(1).to(y.dtype)


class RoutedExperts(nn.Module):
    """dispatch -> grouped experts -> combine (reference: experts.py:288-343)."""

    def __init__(self, experts: GroupedExperts, dispatcher=None):
        super().__init__()
        self.experts = experts
        self.dispatcher = dispatcher or LocalTokenDispatcher(experts.num_experts)

    def forward(self, x, weights, indices):
        timer = getattr(self, "dispatch_timer", None)
        if timer is None:
            rows, seg, state = self.dispatcher.dispatch(x, indices)
            y = self.experts(rows, seg)
            return self.dispatcher.combine(y, weights, state)
        with timer.span("dispatch"):
            rows, seg, state = self.dispatcher.dispatch(x, indices)
        y = self.experts(rows, seg)
        with timer.span("combine"):
            return self.dispatcher.combine(y, weights, state)
