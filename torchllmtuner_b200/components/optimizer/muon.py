"""Distributed Muon over flat shards (reference: llmtuner/components/optimizer/flex_shard/dist_muon.py:181-2088,
_optimizer_reshard_runtime.py:108-879, optimizer_reshard.py).

Matrices (2-D parameters of the decoder blocks, and every expert's matrices inside the packed expert tensors) take the
Muon update: momentum 0.95 (Nesterov), five Newton-Schulz iterations in bf16 with coefficients (3.4445, -4.7750,
2.0315), decoupled weight decay. Every other parameter (embedding, head, norms, routers) takes AdamW. Storage stays the
flat fp32 shard layout of the FSDP units.

Newton-Schulz needs whole matrices while a rank stores an arbitrary flat range, so every step moves data twice:
  storage -> compute   each rank sends, to the owner of a matrix, exactly the part of that matrix it stores (bf16 on the
                       wire: the iteration starts with that cast anyway), one all-to-all per unit
  compute -> storage   the owner returns to each rank the part of the orthogonalised matrix that rank stores
so an element crosses the network once each way, instead of `world` times with a gather of whole units.
The plan (which rank orthogonalises what) is computed once, identically on every rank, and checked by a hash:
  * a job is one matrix, one row block of a fused projection (q, k and v rows of a fused QKV are orthogonalised
    separately), or a run of experts of one packed tensor (batched iteration);
  * jobs are placed longest first on the rank with the least Newton-Schulz work so far (work carried over from earlier
    units of the same group); ties go to the rank that already stores most of the job, then to the lower rank.
The products run on the tcgen05 GEMM on CUDA."""
from __future__ import annotations

import hashlib
import re
from dataclasses import dataclass

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


def newton_schulz_batched(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """[B, m, n]: every matrix of the batch orthogonalised on its own (packed experts)."""
    if g.shape[0] == 1 or g.is_cuda:
        return torch.stack([newton_schulz(x, steps, eps) for x in g])
    a, b, c = NS_COEFFS
    x = g.to(torch.bfloat16)
    transposed = x.shape[1] > x.shape[2]
    if transposed:
        x = x.transpose(1, 2).contiguous()
    x = x / (x.float().flatten(1).norm(dim=1) + eps).to(x.dtype)[:, None, None]
    for _ in range(steps):
        xf = x.float()
        A = xf @ xf.transpose(1, 2)
        x = (a * xf + (b * A + c * (A @ A)) @ xf).to(torch.bfloat16)
    return x.transpose(1, 2).contiguous() if transposed else x


def ns_cost(rows: int, cols: int, batch: int, steps: int) -> int:
    m, n = min(rows, cols), max(rows, cols)
    return batch * steps * (4 * m * m * n + 2 * m * m * m)


@dataclass(frozen=True)
class MuonJob:
    fqn: str
    offset: int          # first element inside the unit's flat buffer
    batch: int           # matrices orthogonalised together (1, or a run of experts)
    rows: int
    cols: int
    lr_shape: tuple      # shape that scales the learning rate (the whole parameter's matrix shape)

    @property
    def numel(self) -> int:
        return self.batch * self.rows * self.cols


def plan_owners(jobs, world: int, shard_numel: int, steps: int, carried=None):
    """Longest job first onto the least loaded rank; ties: the rank storing most of the job, then the lower rank.
    Returns (owner per job, loads after this unit)."""
    loads = list(carried) if carried is not None else [0] * world
    owners = [0] * len(jobs)
    order = sorted(range(len(jobs)), key=lambda i: (-ns_cost(jobs[i].rows, jobs[i].cols, jobs[i].batch, steps), jobs[i].fqn, jobs[i].offset))
    for i in order:
        j = jobs[i]
        stored = [max(0, min(j.offset + j.numel, (r + 1) * shard_numel) - max(j.offset, r * shard_numel)) for r in range(world)]
        r = min(range(world), key=lambda q: (loads[q], -stored[q], q))
        owners[i] = r
        loads[r] += ns_cost(j.rows, j.cols, j.batch, steps)
    return owners, loads


def exchange(send: list[torch.Tensor], recv_sizes: list[int], group) -> list[torch.Tensor]:
    """Variable-size all-to-all of 1-D tensors. NCCL: one `all_to_all_single`; backends without it (gloo): every rank
    publishes its padded send buffer and picks its parts."""
    world = len(send)
    dtype, dev = send[0].dtype, send[0].device
    if dist.get_backend(group) == "nccl":
        out = torch.empty(sum(recv_sizes), dtype=dtype, device=dev)
        dist.all_to_all_single(out, torch.cat(send), output_split_sizes=recv_sizes, input_split_sizes=[t.numel() for t in send], group=group)
        return list(out.split(recv_sizes))
    me = dist.get_rank(group)
    sizes = torch.tensor([t.numel() for t in send], dtype=torch.int64)
    all_sizes = [torch.empty_like(sizes) for _ in range(world)]
    dist.all_gather(all_sizes, sizes, group=group)
    width = int(max(int(x.sum()) for x in all_sizes))
    buf = torch.zeros(max(1, width), dtype=torch.float32, device=dev)
    flat = torch.cat(send).float()
    buf[:flat.numel()] = flat
    every = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(every, buf, group=group)
    out = []
    for src in range(world):
        start = int(all_sizes[src][:me].sum())
        out.append(every[src][start:start + int(all_sizes[src][me])].to(dtype))
    return out


class DistMuon:
    def __init__(self, rt, *, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5, eps: float = 1e-7, betas=(0.9, 0.999), adjust_lr: str = "original", adamw_lr: float | None = None,
                 muon_pattern: str = r"layers\.\d+\..*(proj|gate_proj|up_proj|down_proj)\.weight$", param_group_rules=None,
                 expert_pattern: str = r"experts\.(w1_EFD|w3_EFD|w2_EDF)$", row_blocks=None):
        """`row_blocks(fqn, shape) -> [rows, ...] | None` splits a fused projection into separately orthogonalised row
        blocks (fused QKV: query, key and value rows)."""
        self.rt, self.units = rt, list(rt.units)
        self.momentum, self.nesterov, self.ns_steps, self.eps, self.adjust = momentum, nesterov, ns_steps, eps, adjust_lr
        self.param_groups = [dict(lr=lr, weight_decay=weight_decay, name="muon", param_names=[])]
        self.pattern, self.expert_pattern = re.compile(muon_pattern), re.compile(expert_pattern)
        self.step_count = 0
        self.state: dict[str, dict[str, torch.Tensor]] = {}
        self.jobs: dict[str, list[MuonJob]] = {}
        self.owners: dict[str, list[int]] = {}
        self.matrices: dict[str, list[tuple[str, int, tuple]]] = {}      # (fqn, offset, shape) of every Muon-updated parameter
        carried: dict[int, list[int]] = {}
        plan = []
        for u in self.units:
            jobs, ms = [], []
            for s in u.slots:
                shape = tuple(int(x) for x in s.shape)
                if len(shape) == 2 and self.pattern.search(s.fqn) and not u.is_expert:
                    blocks = row_blocks(s.fqn, shape) if row_blocks is not None else None
                    if blocks:
                        if sum(blocks) != shape[0]:
                            raise ValueError(f"row blocks {blocks} of {s.fqn} do not sum to its {shape[0]} rows")
                        at = s.offset
                        for r in blocks:
                            jobs.append(MuonJob(s.fqn, at, 1, r, shape[1], (r, shape[1])))
                            at += r * shape[1]
                    else:
                        jobs.append(MuonJob(s.fqn, s.offset, 1, shape[0], shape[1], shape))
                    ms.append((s.fqn, s.offset, shape))
                elif len(shape) == 3 and u.is_expert and self.expert_pattern.search(s.fqn):
                    E, per = shape[0], shape[1] * shape[2]
                    run = -(-E // max(1, u.world))
                    for e0 in range(0, E, run):
                        jobs.append(MuonJob(s.fqn, s.offset + e0 * per, min(run, E - e0), shape[1], shape[2], shape[1:]))
                    ms.append((s.fqn, s.offset, shape))
            self.jobs[u.name], self.matrices[u.name] = jobs, ms
            owners, loads = plan_owners(jobs, u.world, u.shard_numel, ns_steps, carried.get(id(u.group)))
            carried[id(u.group)] = loads
            self.owners[u.name] = owners
            self.state[u.name] = {"momentum_buffer": torch.zeros(u.shard_numel, dtype=torch.float32, device=u.master.device)}
            self.param_groups[0]["param_names"] += [m[0] for m in ms]
            plan += [f"{u.name}:{j.fqn}:{j.offset}:{j.batch}x{j.rows}x{j.cols}->{o}" for j, o in zip(jobs, owners)]
        self.compute_loads = {k: v for k, v in carried.items()}
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

    # ------------------------------------------------------------------ redistribution
    def _pieces(self, u, rank: int):
        """For every job: (job index, lo, hi) of the part stored by `rank`, in unit-flat coordinates (hi > lo only)."""
        a, b = rank * u.shard_numel, (rank + 1) * u.shard_numel
        out = []
        for i, j in enumerate(self.jobs[u.name]):
            lo, hi = max(a, j.offset), min(b, j.offset + j.numel)
            if hi > lo:
                out.append((i, lo, hi))
        return out

    def _orthogonalise(self, u, upd: torch.Tensor) -> torch.Tensor:
        """upd: this rank's shard of the momentum-updated gradient (fp32). Returns this rank's shard of the direction,
        already scaled by the per-shape learning-rate factor (zero outside Muon ranges)."""
        jobs, owners = self.jobs[u.name], self.owners[u.name]
        W, me = u.world, u.rank
        a0 = me * u.shard_numel
        g0 = self.param_groups[0]
        out = torch.zeros_like(upd)

        def run(j, flat):
            o = newton_schulz_batched(flat.view(j.batch, j.rows, j.cols), self.ns_steps, self.eps)
            return o.reshape(-1)

        def scale(j):
            return adjusted_lr(g0["lr"], j.lr_shape, self.adjust) / max(g0["lr"], 1e-30)
        if W == 1:
            for j in jobs:
                out[j.offset:j.offset + j.numel] = run(j, upd[j.offset:j.offset + j.numel]).float() * scale(j)
            return out
        mine = self._pieces(u, me)
        send = [[] for _ in range(W)]
        for i, lo, hi in mine:
            send[owners[i]].append(upd[lo - a0:hi - a0].to(torch.bfloat16))
        send = [torch.cat(c) if c else upd.new_zeros(0, dtype=torch.bfloat16) for c in send]
        theirs = [self._pieces(u, r) for r in range(W)]
        recv_sizes = [sum(hi - lo for i, lo, hi in theirs[r] if owners[i] == me) for r in range(W)]
        got = exchange(send, recv_sizes, u.group)
        # assemble the jobs this rank owns, orthogonalise, cut the results back into the senders' pieces
        bufs = {i: torch.empty(j.numel, dtype=torch.bfloat16, device=upd.device) for i, j in enumerate(jobs) if owners[i] == me}
        for r in range(W):
            at = 0
            for i, lo, hi in theirs[r]:
                if owners[i] == me:
                    bufs[i][lo - jobs[i].offset:hi - jobs[i].offset] = got[r][at:at + hi - lo]
                    at += hi - lo
        done = {i: run(jobs[i], b) for i, b in bufs.items()}
        back = [[] for _ in range(W)]
        for r in range(W):
            for i, lo, hi in theirs[r]:
                if owners[i] == me:
                    back[r].append(done[i][lo - jobs[i].offset:hi - jobs[i].offset])
        back = [torch.cat(c) if c else upd.new_zeros(0, dtype=torch.bfloat16) for c in back]
        ret_sizes = [sum(hi - lo for i, lo, hi in mine if owners[i] == r) for r in range(W)]
        res = exchange(back, ret_sizes, u.group)
        cursor = [0] * W
        for i, lo, hi in mine:
            o = owners[i]
            out[lo - a0:hi - a0] = res[o][cursor[o]:cursor[o] + hi - lo].float() * scale(jobs[i])
            cursor[o] += hi - lo
        return out

    @torch.no_grad()
    def step(self, clip_coef=None) -> None:
        self.step_count += 1
        g0 = self.param_groups[0]
        coef = 1.0 if clip_coef is None else clip_coef
        # AdamW part first: it updates every element; Muon ranges are then overwritten from a snapshot of the
        # pre-update master values, so the two never mix on one element.
        snap = {u.name: u.master.clone() for u in self.units if self.jobs[u.name] and u.has_grad}
        self.adamw.step(clip_coef)
        for u in self.units:
            if not self.jobs[u.name] or not u.has_grad:
                continue
            buf = self.state[u.name]["momentum_buffer"]
            g = u.grad_shard.float() * coef
            buf.mul_(self.momentum).add_(g)
            upd = g.add(buf, alpha=self.momentum) if self.nesterov else buf.clone()
            mine = self._orthogonalise(u, upd)
            a, _ = u.my_range()
            pre = snap[u.name]
            for _, lo, hi in self._pieces(u, u.rank):
                sl = slice(lo - a, hi - a)
                u.master[sl] = pre[sl] * (1.0 - g0["lr"] * g0["weight_decay"]) - g0["lr"] * mine[sl]
            if u.separate_master:
                u.shard_lowp.copy_(u.master)
