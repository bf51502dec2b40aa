"""Expert-parallel token dispatch and combine over NVLink peer memory
(replaces the NCCL all-to-all dispatcher, reference: llmtuner/parallel/expert_parallel/token_dispatch.py:319-678).

No host synchronisation and no NCCL on the data path:
  * the per-expert counts are exchanged by `ep_exchange` (P2P stores into every rank's count table, bounded flag wait),
    which also derives the padded segment layout of the local experts and the offsets of this rank's rows in every
    owner's buffer, all on the device;
  * `ep_push_rows` writes every token copy straight into its final expert-major row of the owner's receive buffer;
  * after the grouped expert GEMMs the sources read their rows back with `ep_pull_rows`, which applies the router
    scores and accumulates in fp32 (fixed order, deterministic);
  * backward mirrors it: output gradients are pushed score-scaled (the same kernel also produces the router-weight
    gradients), input gradients are pulled.
Every rank owns four fixed-capacity row buffers in one symmetric arena (expert inputs, expert outputs and their two
gradients); `ready` / `free` epoch flags per buffer order producers and consumers. The buffers are sized for the worst
routing skew by default (every copy of every rank lands on one rank), as the reference's exact split sizes are
(token_dispatch.py:327-395); with a smaller `ep_capacity_factor` a run that does not fit raises the CapacityOverflow device
status instead of writing out of bounds. Sizes are agreed across the group when the arena is built.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..errors import ConfigError
from ..models.moe.experts import SEG_ALIGN
from .symm import canary_intact, write_canary

BUF_X, BUF_Y, BUF_DY, BUF_DX = 0, 1, 2, 3


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


class PeerExchange:
    """Arena + flags of one EP group, sized for `max_copies` token copies per rank and rows of `hidden` bf16."""

    def __init__(self, group, device, num_experts: int, max_copies: int, hidden: int, capacity_factor: float | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops.cuda_ext import load
        self.ext = load()
        self.group, self.device = group, device
        self.R, self.me = dist.get_world_size(group), dist.get_rank(group)
        self.E, self.El, self.D = num_experts, num_experts // self.R, hidden
        # Every offset below is added to PEER base addresses, so the layout has to be the same on every rank: the sizes
        # are agreed with one MAX all-reduce over the group (ranks may see different token counts on their first call)
        # and checked for equality.
        agreed = torch.tensor([max_copies, hidden, num_experts, -hidden, -num_experts], dtype=torch.int64, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=group)
        mx, hmax, emax, hmin, emin = (int(v) for v in agreed.tolist())
        if (hmax, emax) != (hidden, num_experts) or (-hmin, -emin) != (hidden, num_experts):
            raise ConfigError(f"expert-parallel ranks disagree on the exchange shape: hidden {hidden} (group max {hmax}), "
                              f"experts {num_experts} (group max {emax})")
        self.max_copies = max_copies = mx
        # Dropless by default: a rank can receive at most every copy of every rank (R * max_copies rows); each local expert
        # adds up to SEG_ALIGN - 1 rows of segment padding.
        factor = float(self.R) if capacity_factor is None else min(float(self.R), float(capacity_factor))
        self.dropless = factor >= float(self.R)
        cap = int(max_copies * factor) + self.El * (SEG_ALIGN - 1)
        self.cap = -(-cap // SEG_ALIGN) * SEG_ALIGN
        buf_b = _align(self.cap * hidden * 2)
        tab_b = _align(2 * self.R * self.E * 4)
        flag_b = _align(self.R * 4)
        self.off_buf = [i * buf_b for i in range(4)]
        self.off_tab = 4 * buf_b
        self.off_cflag = self.off_tab + tab_b
        base = self.off_cflag + flag_b
        self.off_flag = {(b, w): base + (2 * b + w) * flag_b for b in range(4) for w in (0, 1)}     # w: 0 ready, 1 free
        total = base + 8 * flag_b + 256
        self.arena = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.arena.zero_()
        write_canary(self.arena)
        self.hdl = symm_mem.rendezvous(self.arena, group)
        self.peer_base = [int(p) for p in self.hdl.buffer_ptrs]
        self.base = self.peer_base[self.me]
        self.epoch = [0, 0, 0, 0]
        self.count_epoch = 0
        self.stats = {"dispatches": 0, "combines": 0}
        torch.cuda.synchronize(device)
        self.hdl.barrier()

    def check_canaries(self) -> bool:
        return canary_intact(self.arena)

    def fits(self, copies: int, hidden: int, num_experts: int) -> bool:
        return copies <= self.max_copies and hidden == self.D and num_experts == self.E

    # ------------------------------------------------------------------ flag helpers
    def _ptrs(self, off: int) -> list[int]:
        return [b + off for b in self.peer_base]

    def signal(self, buf: int, which: int, value: int) -> None:
        self.ext.signal_peers(self._ptrs(self.off_flag[(buf, which)]), self.me, value)

    def wait(self, buf: int, which: int, value: int) -> None:
        if value > 0:
            self.ext.wait_flags(self.base + self.off_flag[(buf, which)], self.R, value, 8300 + 10 * buf + which)

    def local_buf(self, buf: int) -> torch.Tensor:
        o = self.off_buf[buf]
        return self.arena[o: o + self.cap * self.D * 2].view(torch.bfloat16).view(self.cap, self.D)

    # ------------------------------------------------------------------ phases
    def plan(self, indices: torch.Tensor):
        """Device-only routing plan of one MoE call: destination (rank, row) of every token copy and this rank's
        segment layout."""
        flat = indices.reshape(-1).contiguous()
        self.count_epoch += 1
        seg, totals, send_off = self.ext.ep_exchange(flat, self.E, self.me, self._ptrs(self.off_tab), self._ptrs(self.off_cflag),
                                                     self.count_epoch, self.cap)
        if self.E <= 256 and os.environ.get("LLMT_EP_FUSED_PLAN", "1") == "1":
            drank, drow = self.ext.ep_plan(flat, self.E, self.R, send_off)
        else:
            counts = torch.bincount(flat, minlength=self.E)
            start = counts.cumsum(0) - counts
            order = torch.argsort(flat, stable=True)
            rank = torch.empty_like(order)
            rank[order] = torch.arange(order.numel(), device=order.device)
            pos = rank - start[flat]                                         # stable position inside this rank's run
            drow = (send_off.long()[flat] + pos).to(torch.int32)
            drank = (flat // self.El).to(torch.int32)
        return {"seg": seg, "totals": totals, "drank": drank, "drow": drow, "T": indices.shape[0], "k": indices.shape[1]}

    def push(self, buf: int, src: torch.Tensor, plan, scale=None, other=None):
        """Write the token copies into the owners' buffer `buf`; returns the dot products when `other` is given."""
        self.epoch[buf] += 1
        e = self.epoch[buf]
        self.wait(buf, 1, e - 1)                                              # owners have consumed the previous content
        dot = self.ext.ep_push_rows(src, scale, plan["drank"], plan["drow"], self._ptrs(self.off_buf[buf]), self.cap, plan["k"], other)
        self.signal(buf, 0, e)
        return dot

    def receive(self, buf: int, plan) -> torch.Tensor:
        """Owner side of `push`: a private copy of the received rows (padding zeroed); frees the buffer."""
        e = self.epoch[buf]
        self.wait(buf, 0, e)
        rows = torch.empty(self.cap, self.D, dtype=torch.bfloat16, device=self.device)
        self.ext.ep_clone_rows(self.base + self.off_buf[buf], rows, plan["seg"], plan["totals"], True)
        self.signal(buf, 1, e)
        return rows

    def publish(self, buf: int, rows: torch.Tensor, plan) -> None:
        """Owner side of `pull`: expose `rows` (expert-major, this rank's experts) to the sources."""
        self.epoch[buf] += 1
        e = self.epoch[buf]
        self.wait(buf, 1, e - 1)                                              # sources have read the previous content
        dst = self.local_buf(buf)
        self.ext.ep_clone_rows(rows.data_ptr(), dst, plan["seg"], plan["totals"], False)
        self.signal(buf, 0, e)

    def pull(self, buf: int, plan, weights=None, keep: bool = False):
        e = self.epoch[buf]
        self.wait(buf, 0, e)
        res = self.ext.ep_pull_rows(self._ptrs(self.off_buf[buf]), plan["drank"], plan["drow"], weights, self.cap, plan["T"], plan["k"],
                                    self.D, keep)
        self.signal(buf, 1, e)
        return res


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ex: PeerExchange, plan):
        ex.push(BUF_X, x.contiguous(), plan)
        rows = ex.receive(BUF_X, plan)
        ctx.ex, ctx.plan = ex, plan
        return rows

    @staticmethod
    def backward(ctx, d_rows):
        ex, plan = ctx.ex, ctx.plan
        ex.publish(BUF_DX, d_rows.contiguous(), plan)
        (dx,) = ex.pull(BUF_DX, plan)
        return dx, None, None


class _PeerCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, weights, ex: PeerExchange, plan):
        ex.publish(BUF_Y, y.contiguous(), plan)
        w = weights.reshape(-1).float().contiguous()
        out, kept = ex.pull(BUF_Y, plan, w, keep=True)
        ctx.ex, ctx.plan = ex, plan
        ctx.save_for_backward(kept, w)
        ctx.wdtype, ctx.wshape = weights.dtype, weights.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        ex, plan = ctx.ex, ctx.plan
        kept, w = ctx.saved_tensors
        dw = ex.push(BUF_DY, dout.contiguous(), plan, scale=w, other=kept)      # dy rows to the owners, dw = <dout, y>
        dy = ex.receive(BUF_DY, plan)
        return dy, dw.view(ctx.wshape).to(ctx.wdtype), None, None


class PeerTokenDispatcher:
    """Drop-in for the all-to-all dispatcher (`dispatch` / `combine`) on CUDA bf16; falls back to `fallback` otherwise."""

    def __init__(self, num_experts: int, group, ep_size: int, ep_rank: int, fallback, capacity_factor: float | None = None,
                 max_copies_hint: int = 0):
        self.num_experts, self.group, self.ep_size, self.ep_rank = num_experts, group, ep_size, ep_rank
        self.local_experts = num_experts // ep_size
        self.fallback, self.capacity_factor = fallback, capacity_factor
        self.max_copies_hint = max_copies_hint       # tokens per rank x top-k of the largest micro-batch, when known
        self.exchange: PeerExchange | None = None

    def _exchange_for(self, x, indices):
        if not x.is_cuda or x.dtype != torch.bfloat16 or x.shape[1] % 8 or os.environ.get("LLMT_DISABLE_FUSED_EP") == "1":
            return None
        if self.ep_size > 8:
            return None
        copies = indices.numel()
        ex = _EXCHANGES.get(id(self.group))
        if ex is None:
            # collective: every rank of the group reaches its first MoE call in the same step
            ex = _EXCHANGES[id(self.group)] = PeerExchange(self.group, x.device, self.num_experts, max(copies, self.max_copies_hint),
                                                           x.shape[1], self.capacity_factor)
        if not ex.fits(copies, x.shape[1], self.num_experts):
            # Falling back on this rank alone would leave the others polling flags that never flip, and pushing with a
            # row count the arena was not sized for would write outside a peer's buffer.
            raise ConfigError(f"expert-parallel exchange was sized for {ex.max_copies} token copies per rank with hidden {ex.D}; "
                              f"this call has {copies} copies with hidden {x.shape[1]}. Set the largest micro-batch first "
                              "(max_seq_len x local batch) or use ep_token_dispatcher=domino / LLMT_DISABLE_FUSED_EP=1")
        return ex

    def dispatch(self, x, indices):
        ex = self._exchange_for(x, indices)
        if ex is None:
            rows, seg, st = self.fallback.dispatch(x, indices)
            st["_fallback"] = True
            return rows, seg, st
        plan = ex.plan(indices)
        rows = _PeerDispatch.apply(x, ex, plan)
        ex.stats["dispatches"] += 1
        return rows, plan["seg"], {"plan": plan, "ex": ex}

    def combine(self, y, weights, st):
        if st.get("_fallback"):
            return self.fallback.combine(y, weights, st)
        st["ex"].stats["combines"] += 1
        return _PeerCombine.apply(y, weights, st["ex"], st["plan"])


_EXCHANGES: dict = {}
