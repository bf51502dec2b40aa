"""Context parallelism for standard attention: Ulysses head<->sequence all-to-all and key/value all-gather with
optional head-tail load balancing, both with packed (multi-document) rows
(reference: llmtuner/parallel/context_parallel/context_parallel.py:18-55, attention.py:12-87, input_sharding.py:109-232;
the reference removed the standard-attention kernels, plan.py:27-34, and rejects packed rows under CP,
models/common/input_preparation.py:144-149; here both are supported by carrying the global document cuts to every rank).

The driver is installed as `ForwardContext.cp`; `Qwen3Attention` calls `cp.attention(q, k, v, meta, scale)` with local
rows `[T/cp, H, d]`.
  ulysses       a2a turns [T/cp, H, d] into [T, H/cp, d] for q, k, v; attention over complete rows and the global
                document table; a2a back for the output.
  kv_allgather  queries stay local; K and V are all-gathered into global row order; each local query span of each
                document attends that document's keys up to its own position (explicit query offsets).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..ops.attn_meta import AttnMeta
from .input_sharding import contiguous_chunk, headtail_chunks


class _SeqToHead(torch.autograd.Function):
    """[T/R, H, d] -> [T, H/R, d] (rows in global order of the rank chunks); backward is the inverse."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        R = dist.get_world_size(group)
        t, H, d = x.shape
        send = x.view(t, R, H // R, d).permute(1, 0, 2, 3).contiguous()         # [R, t, H/R, d]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.view(R * t, H // R, d)

    @staticmethod
    def backward(ctx, g):
        return _HeadToSeq.apply(g, ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        R = dist.get_world_size(group)
        T, h, d = x.shape
        send = x.contiguous().view(R, T // R, h, d)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 0, 2, 3).reshape(T // R, R * h, d)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHead.apply(g, ctx.group), None


def cp_all_to_all(x, group, to_heads: bool):
    return _SeqToHead.apply(x, group) if to_heads else _HeadToSeq.apply(x, group)


class _AllGatherRowsCP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, perm):
        ctx.group, ctx.perm = group, perm
        R = dist.get_world_size(group)
        out = x.new_empty((x.shape[0] * R, *x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out if perm is None else out.index_select(0, perm[0])

    @staticmethod
    def backward(ctx, g):
        R = dist.get_world_size(ctx.group)
        if ctx.perm is not None:
            g = g.index_select(0, ctx.perm[1])
        out = g.new_empty((g.shape[0] // R, *g.shape[1:]))
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None, None


class ContextParallelDriver:
    def __init__(self, topo, cp_config):
        self.topo = topo
        self.strategy = "ulysses" if topo.cp_ulysses > 1 else "kv_allgather"
        if topo.cp_ulysses > 1 and topo.cp_kv > 1:
            self.strategy = "hybrid"
        self.load_balancer = cp_config.context_parallel_load_balancer if topo.cp_kv > 1 else None
        self.group = topo.get_group("cp")
        self.size, self.rank = topo.cp, topo.coord("cp")
        if self.strategy == "hybrid":
            # key/value axis outside, ulysses axis inside: heads are exchanged among the ulysses ranks first, which
            # turns their rows into the rows of the key/value level; keys and values are then gathered over that axis
            self.group_ul, self.group_kv = topo.get_group("cp_ulysses"), topo.get_group("cp_kv")
            self.size_kv, self.rank_kv = topo.cp_kv, topo.coord("cp_kv")
        else:
            self.group_ul = self.group_kv = self.group
            self.size_kv, self.rank_kv = self.size, self.rank
        self._mb = None

    # ------------------------------------------------------------------ per micro-batch tables
    def begin_microbatch(self, inputs: dict) -> None:
        """Builds the attention tables of this rank from the global document cuts."""
        dev = inputs["tokens"].device
        B, S = inputs["batch"], inputs["seq"]
        gcu = inputs.get("global_cu_seqlens", inputs["cu_seqlens"]).tolist()
        mb = {"B": B, "S": S, "gcu": [int(c) for c in gcu]}
        if self.strategy == "ulysses":
            mb["meta"] = AttnMeta.build(gcu, causal=True, device=dev)
        else:
            # local spans of every sequence, in local row order (of the key/value level in the hybrid strategy)
            R, r = self.size_kv, self.rank_kv
            spans = headtail_chunks(S, R, r) if self.load_balancer == "headtail" else [contiguous_chunk(S, R, r)]
            pieces, local = [], 0
            for b in range(B):
                for a, e in spans:
                    ga, ge = b * S + a, b * S + e                      # global rows of this local span
                    for i in range(len(gcu) - 1):
                        ds, de = gcu[i], gcu[i + 1]
                        lo, hi = max(ga, ds), min(ge, de)
                        if hi > lo:
                            pieces.append((local + (lo - ga), hi - lo, ds, hi - ds, lo - ds))   # q0, qlen, k0, klen, off
                    local += e - a
            mb["meta"] = AttnMeta.from_pieces(pieces, total_q=local, total_k=B * S, causal=True, device=dev)
            if self.load_balancer == "headtail":
                # gathered rows arrive rank-major (each rank: head chunk, tail chunk); map to global order and back
                c = S // (2 * R)
                src = []
                for b in range(B):
                    for chunk in range(2 * R):
                        owner = chunk if chunk < R else 2 * R - 1 - chunk
                        half = 0 if chunk < R else 1
                        base = owner * (B * 2 * c) + b * 2 * c + half * c
                        src.append(torch.arange(base, base + c))
                fwd = torch.cat(src).to(dev)
                inv = torch.empty_like(fwd)
                inv[fwd] = torch.arange(fwd.numel(), device=dev)
                mb["perm"] = (fwd, inv)
            elif B > 1:
                t = S // R
                src = [torch.arange(rk * B * t + b * t, rk * B * t + (b + 1) * t) for b in range(B) for rk in range(R)]
                fwd = torch.cat(src).to(dev)
                inv = torch.empty_like(fwd)
                inv[fwd] = torch.arange(fwd.numel(), device=dev)
                mb["perm"] = (fwd, inv)
            else:
                mb["perm"] = None
        self._mb = mb

    # ------------------------------------------------------------------ attention
    def attention(self, q, k, v, meta, scale):
        mb = self._mb
        if self.strategy == "ulysses":
            B, S, R = mb["B"], mb["S"], self.size
            # local rows are [b][s/R]; after the exchange rows are [rank][b][s/R]: restore [b][s] order
            qh, kh, vh = (cp_all_to_all(t, self.group, True) for t in (q, k, v))
            if B > 1:
                t = S // R
                idx = torch.arange(R * B * t, device=q.device).view(R, B, t).permute(1, 0, 2).reshape(-1)
                inv = torch.empty_like(idx)
                inv[idx] = torch.arange(idx.numel(), device=q.device)
                qh, kh, vh = qh.index_select(0, idx), kh.index_select(0, idx), vh.index_select(0, idx)
            o = ops.attention(qh, kh, vh, mb["meta"], scale)
            if B > 1:
                o = o.index_select(0, inv)
            return cp_all_to_all(o, self.group, False)
        if self.strategy == "hybrid":
            q, k, v = (cp_all_to_all(t, self.group_ul, True) for t in (q, k, v))
        kg = _AllGatherRowsCP.apply(k, self.group_kv, mb["perm"])
        vg = _AllGatherRowsCP.apply(v, self.group_kv, mb["perm"])
        o = ops.attention(q, kg, vg, mb["meta"], scale)
        return cp_all_to_all(o, self.group_ul, False) if self.strategy == "hybrid" else o


    # ------------------------------------------------------------------ delta rule (recurrent state across ranks)
    def prev_rows(self, x: torch.Tensor, n: int) -> torch.Tensor:
        """x [B*t, C]: this rank's contiguous span of each of the B sequences. Returns [B, n, C]: the last n rows of the
        span before it (zeros on the first rank): the history a causal convolution of width n + 1 needs at the left
        edge (reference: llmtuner/models/kimi/kimi_k3/delta_attention.py:237-262 hands the same rows to its convolution
        kernel through the context-parallel context). Every rank keeps the gather in its graph."""
        from ..errors import UnsupportedCombinationError
        if self.strategy != "kv_allgather" or self.load_balancer is not None:
            raise UnsupportedCombinationError("convolution history needs contiguous sequence spans: use context_parallel_kcp_size or "
                                              "context_parallel_kv_allgather_size without a load balancer")
        B = self._mb["B"]
        t = x.shape[0] // B
        if t < n:
            raise UnsupportedCombinationError(f"a local span of {t} rows is shorter than the convolution history of {n}")
        tail = x.view(B, t, -1)[:, t - n:].contiguous().unsqueeze(0)
        every = _AllGatherRowsCP.apply(tail, self.group, None)                # [R, B, n, C]
        if self.rank == 0:
            return every[0] * 0.0
        return every[self.rank - 1] + 0.0 * every[self.rank].sum()

    def gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's rows [B*t, ...] -> every rank's rows in global order [B*S, ...] (differentiable: the backward is a
        reduce-scatter). For small per-token tensors that every rank needs whole: a shared single-head key/value stream,
        the inputs of window compressors."""
        from ..errors import UnsupportedCombinationError
        if self.strategy != "kv_allgather":
            raise UnsupportedCombinationError("gathering rows over the sequence axis needs context_parallel_kv_allgather_size (or kcp)")
        return _AllGatherRowsCP.apply(x, self.group_kv, self._mb["perm"])

    def delta_rule(self, q, k, v, beta, log_decay, chunk: int):
        """Sequence-parallel gated delta rule (reference: llmtuner/parallel/context_parallel/kcp.py:30-335). Every rank
        owns one contiguous span of each sequence. The recurrence is linear in the state, and its value columns evolve
        independently, so one pass over the local span with dk extra value columns that start as an identity yields the
        span's outputs from a zero state, its end state Sigma and its transition matrix Phi (end = Phi start + Sigma).
        (Phi, Sigma) of all ranks are gathered, every rank folds those of the ranks before it into its incoming state,
        and adds the incoming state's contribution to the outputs of the document that continues across its left
        edge. A document that starts inside a span cuts the chain: Phi = 0 for that rank."""
        from ..errors import UnsupportedCombinationError
        from ..models.families import chunked_delta_rule
        mb = self._mb
        if self.strategy != "kv_allgather" or self.load_balancer is not None:
            raise UnsupportedCombinationError("the delta-rule layers need contiguous sequence spans: use context_parallel_kcp_size or "
                                              "context_parallel_kv_allgather_size without a load balancer")
        B, S, R, r = mb["B"], mb["S"], self.size, self.rank
        gcu = mb["gcu"]
        t = S // R
        H, dk, dv = q.shape[1], q.shape[2], v.shape[2]
        eye = torch.eye(dk, dtype=q.dtype, device=q.device).expand(H, dk, dk)
        outs, exports, firsts = [], [], []
        for b in range(B):
            lo, hi = b * S + r * t, b * S + (r + 1) * t                       # global rows of this local span
            starts = [c for c in gcu if lo < c < hi]
            cuts = [lo] + starts + [hi]
            continues = r > 0 and lo not in gcu                                # a document crosses the left edge
            seg_out = []
            for i, (a, e) in enumerate(zip(cuts[:-1], cuts[1:])):
                sl = slice(b * t + a - lo, b * t + e - lo)
                last = i == len(cuts) - 2
                if last:                                                       # the segment whose end state leaves this rank
                    carry = continues and len(cuts) == 2
                    vx = torch.cat((v[sl], v.new_zeros(e - a, H, dk)), -1) if carry else v[sl]
                    s0 = torch.cat((v.new_zeros(H, dk, dv), eye), -1) if carry else None
                    o, st = chunked_delta_rule(q[sl], k[sl], vx, beta[sl], log_decay[sl], chunk, s0, True)
                    phi = st[..., dv:] if carry else st.new_zeros(H, dk, dk)
                    exports.append(torch.cat((st[..., :dv], phi), -1))        # [H, dk, dv + dk]
                    o = o[..., :dv]
                else:
                    o = chunked_delta_rule(q[sl], k[sl], v[sl], beta[sl], log_decay[sl], chunk)
                seg_out.append(o)
            firsts.append((slice(b * t, b * t + cuts[1] - lo), continues))
            outs.append(seg_out)
        mine = torch.stack(exports).unsqueeze(0)                              # [1, B, H, dk, dv + dk]
        every = _AllGatherRowsCP.apply(mine, self.group, None)                # [R, B, H, dk, dv + dk]
        result = []
        for b in range(B):
            sl, continues = firsts[b]
            if continues and r > 0:
                state = every[0, b, ..., :dv]
                for p in range(1, r):
                    state = every[p, b, ..., dv:] @ state + every[p, b, ..., :dv]
                # contribution of the incoming state to the first segment: the same recurrence without new values
                corr = chunked_delta_rule(q[sl], k[sl], torch.zeros_like(v[sl]), beta[sl], log_decay[sl], chunk, state)
                outs[b][0] = outs[b][0] + corr
            result.extend(outs[b])
        # every rank keeps the gathered tensor in its graph, so that all of them enter its backward collective
        result[0] = result[0] + 0.0 * every.sum()
        return torch.cat(result)


def build_cp_plan(model, topo, cp_config):
    """Which attention modules will run under context parallelism, and along which axes. Ulysses exchanges heads, so its
    degree has to divide the key/value heads left after tensor parallelism; checked here, before any stage runs."""
    from ..models.contracts import BoundDecoder
    from .plan import ParallelPlan, PlanTarget
    from ..errors import UnsupportedCombinationError
    bound = BoundDecoder(model.decoder_structure, model)
    st = model.decoder_structure
    targets = []
    for key, block in bound.block_items():
        attn = bound.attention_of(block)
        if topo.cp_ulysses > 1:
            for name in ("num_heads", "num_kv_heads"):
                h = getattr(attn, name, None)
                if h is not None and (h // max(1, topo.tp)) % topo.cp_ulysses:
                    raise UnsupportedCombinationError(f"context_parallel_ulysses_size {topo.cp_ulysses} does not divide "
                                                      f"{type(attn).__name__}.{name} = {h} (after tensor parallelism {topo.tp})")
        targets.append(PlanTarget(f"{st.blocks}.{key}.{st.attention}", "attention", "context", attn))
    axes = "+".join(n for n, d in (("kv_allgather", topo.cp_kv), ("ulysses", topo.cp_ulysses), ("kcp", getattr(topo, "kcp", 1))) if d > 1)
    return ParallelPlan("cp", topo.cp, axes or "none", tuple(targets), binds=("modules",),
                        notes=(f"load balancer: {cp_config.context_parallel_load_balancer}",))


def apply_cp(model, topo, cp_config) -> ContextParallelDriver:
    """`kcp` is the sequence axis of delta-attention models: softmax / latent attention layers gather keys and values
    over it, delta-rule layers hand their recurrent state from rank to rank (`ContextParallelDriver.delta_rule`)."""
    return ContextParallelDriver(topo, cp_config)
