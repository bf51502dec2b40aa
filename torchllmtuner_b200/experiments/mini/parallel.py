"""The `(dp, ep, tp)` mesh and the collectives of the teaching framework as autograd functions: every function says
what it does forward and what the matching backward collective is."""
from __future__ import annotations

import torch
import torch.distributed as dist


class Mesh:
    """rank = (d * ep + e) * tp + t. Every rank creates every group, in the same order."""

    def __init__(self, dp: int, ep: int, tp: int):
        self.dp, self.ep, self.tp = dp, ep, tp
        self.world = dp * ep * tp
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.d, rest = divmod(self.rank, ep * tp)
        self.e, self.t = divmod(rest, tp)
        self.tp_group = self.ep_group = self.dp_group = self.data_group = None
        if self.world == 1:
            return
        rk = lambda d, e, t: (d * ep + e) * tp + t  # noqa: E731
        for d in range(dp):
            for e in range(ep):
                g = dist.new_group([rk(d, e, t) for t in range(tp)]) if tp > 1 else None
                if (d, e) == (self.d, self.e):
                    self.tp_group = g
        for d in range(dp):
            for t in range(tp):
                g = dist.new_group([rk(d, e, t) for e in range(ep)]) if ep > 1 else None
                if (d, t) == (self.d, self.t):
                    self.ep_group = g
        for e in range(ep):
            for t in range(tp):
                g = dist.new_group([rk(d, e, t) for d in range(dp)]) if dp > 1 else None
                if (e, t) == (self.e, self.t):
                    self.dp_group = g
        for t in range(tp):                                   # ranks that see different data: dp x ep at one tp coordinate
            g = dist.new_group([rk(d, e, t) for d in range(dp) for e in range(ep)]) if dp * ep > 1 else None
            if t == self.t:
                self.data_group = g

    @property
    def data_rank(self) -> int:
        return self.d * self.ep + self.e

    @property
    def data_ranks(self) -> int:
        return self.dp * self.ep


def all_reduce_(t: torch.Tensor, group) -> torch.Tensor:
    if group is not None:
        dist.all_reduce(t, group=group)
    return t


class CopyToTP(torch.autograd.Function):
    """Forward: identity (the input is the same on every tp rank). Backward: all-reduce, because every tp rank used the
    value with its own shard of the weights and holds only its part of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_(g.contiguous().clone(), ctx.group), None


class ReduceFromTP(torch.autograd.Function):
    """Forward: all-reduce of the partial sums of a row-parallel product. Backward: identity."""

    @staticmethod
    def forward(ctx, x, group):
        return all_reduce_(x.contiguous().clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class AllToAllRows(torch.autograd.Function):
    """Forward: send `in_splits[r]` rows to rank r, receive `out_splits[r]` rows from it. Backward: the same exchange
    with the split lists swapped."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.cfg = (in_splits, out_splits, group)
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        in_splits, out_splits, group = ctx.cfg
        back = g.new_empty((sum(in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(back, g.contiguous(), in_splits, out_splits, group=group)
        return back, None, None, None


def copy_to_tp(x, group):
    return x if group is None else CopyToTP.apply(x, group)


def reduce_from_tp(x, group):
    return x if group is None else ReduceFromTP.apply(x, group)


def shard(full: torch.Tensor, dim: int, index: int, parts: int) -> torch.Tensor:
    """The `index`-th of `parts` equal slices of `full` along `dim` (a private copy)."""
    n = full.shape[dim] // parts
    return full.narrow(dim, index * n, n).clone()
