"""Stock-PyTorch arms for the tensor-parallel and expert-parallel benchmark configurations.

They issue the library calls the reference issues on CUDA for these paths and nothing of this repository's kernels:
  tensor parallel + sequence parallel   `torch.ops.symm_mem.fused_all_gather_matmul` / `fused_matmul_reduce_scatter` inside
                                        hand-derived autograd functions, one unfused all-gather in front of q/k/v, gate and up
                                        each with their own fused gather, vocabulary-parallel embedding, replicated head with
                                        a gradient all-reduce (reference: llmtuner/accelerator/linear_collectives.py:197-453,
                                        llmtuner/parallel/tensor_parallel/linear.py:114-192, sequence_boundary.py:18-41)
  expert parallel                       count all-to-all, host read of the split sizes, token all-to-all, permute to
                                        expert-major, `torch._grouped_mm`, inverse path, score-weighted `index_add`; dense
                                        parameters under FSDP2 `fully_shard` (reference: llmtuner/parallel/expert_parallel/
                                        token_dispatch.py:327-636, llmtuner/models/common/moe/experts.py:206-268)
Attention is `F.scaled_dot_product_attention`, norms `F.rms_norm`, optimizer `torch.optim.AdamW(fused=True)`, activation
checkpointing `torch.utils.checkpoint`. These are stand-ins for the reference, which needs torch >= 2.12 to import.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1)


def _rope_tables(S, d, theta, dev):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=dev, dtype=torch.float32) / d))
    ang = torch.arange(S, device=dev, dtype=torch.float32)[:, None] * inv[None]
    return ang.cos().to(torch.bfloat16)[None, None], ang.sin().to(torch.bfloat16)[None, None]


def _init_dist():
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29534")
    os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    return world, rank, dev


def _time_steps(step, args, world, dev):
    warm = max(3, args.warmup)
    for _ in range(warm):
        step(True)

    def timed(k, read):
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = [step(read) for _ in range(k)]
        e1.record()
        dist.barrier(); torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms), out
    ms, _ = timed(args.steps, False)
    ms2, outs = timed(args.steps, True)
    return warm, ms, ms2, outs


# ================================================================================================ tensor parallel
class _AGLinear(torch.autograd.Function):
    """x_shard [T/R, K], w [N/R, K] -> gather(x) @ w^T with the fused symmetric-memory op; dual ops in backward."""

    @staticmethod
    def forward(ctx, x, w, gn):
        x_full, outs = torch.ops.symm_mem.fused_all_gather_matmul(x.contiguous(), [w.t()], 0, gn)
        ctx.save_for_backward(x_full, w)
        ctx.gn = gn
        return outs[0]

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        dx = torch.ops.symm_mem.fused_matmul_reduce_scatter(dy.contiguous(), w, "sum", 0, ctx.gn)
        return dx, dy.t() @ x_full, None


class _LinearRS(torch.autograd.Function):
    """x [T, K/R], w [N, K/R] -> reduce_scatter(x @ w^T) [T/R, N]."""

    @staticmethod
    def forward(ctx, x, w, gn):
        ctx.save_for_backward(x, w)
        ctx.gn = gn
        return torch.ops.symm_mem.fused_matmul_reduce_scatter(x.contiguous(), w.t(), "sum", 0, gn)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy_full, outs = torch.ops.symm_mem.fused_all_gather_matmul(dy.contiguous(), [w], 0, ctx.gn)
        return outs[0], dy_full.t() @ x, None


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty(x.shape[0] * dist.get_world_size(group), *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty(g.shape[0] // dist.get_world_size(ctx.group), *g.shape[1:], dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty(x.shape[0] // dist.get_world_size(group), *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty(g.shape[0] * dist.get_world_size(ctx.group), *g.shape[1:], dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class TPBlock(nn.Module):
    def __init__(self, c, R, group, gn):
        super().__init__()
        D, d = c["hidden_size"], c["head_dim"]
        self.hq, self.hk, self.d, self.R, self.group, self.gn = c["num_attention_heads"] // R, c["num_key_value_heads"] // R, d, R, group, gn
        mk = lambda n, k: nn.Parameter(torch.empty(n, k, dtype=torch.bfloat16))      # noqa: E731
        self.wq, self.wk, self.wv = mk(self.hq * d, D), mk(self.hk * d, D), mk(self.hk * d, D)
        self.wo = mk(D, self.hq * d)
        Fl = c["intermediate_size"] // R
        self.wg, self.wu, self.wd = mk(Fl, D), mk(Fl, D), mk(D, Fl)
        self.q_norm, self.k_norm = nn.RMSNorm(d, eps=1e-6, dtype=torch.bfloat16), nn.RMSNorm(d, eps=1e-6, dtype=torch.bfloat16)
        self.ln1, self.ln2 = nn.RMSNorm(D, eps=1e-6, dtype=torch.bfloat16), nn.RMSNorm(D, eps=1e-6, dtype=torch.bfloat16)

    def forward(self, x, cos, sin, B):
        """x: sequence shard [T/R, D] of B sequences laid end to end."""
        h = _Gather.apply(self.ln1(x), self.group)                      # [T, D]: one unfused gather in front of q/k/v
        T = h.shape[0]
        S = T // B
        q = self.q_norm(F.linear(h, self.wq).view(B, S, self.hq, self.d)).transpose(1, 2)
        k = self.k_norm(F.linear(h, self.wk).view(B, S, self.hk, self.d)).transpose(1, 2)
        v = F.linear(h, self.wv).view(B, S, self.hk, self.d).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True).transpose(1, 2).reshape(T, -1)
        x = x + _LinearRS.apply(o, self.wo, self.gn)
        h = self.ln2(x)
        a = F.silu(_AGLinear.apply(h, self.wg, self.gn)) * _AGLinear.apply(h, self.wu, self.gn)
        return x + _LinearRS.apply(a, self.wd, self.gn)


def run_stock_tp(args) -> int:
    from torch.utils.checkpoint import checkpoint
    import torch.distributed._symmetric_memory as symm_mem
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from torchllmtuner_b200.models.qwen3 import QWEN3_8B, Qwen3Config
    world, rank, dev = _init_dist()
    R = args.tp
    assert R == world, "the stock tensor-parallel arm runs TP over all ranks"
    group = dist.group.WORLD
    gn = group.group_name
    symm_mem.enable_symm_mem_for_group(gn)
    c = dict(QWEN3_8B)
    if args.layers:
        c["num_hidden_layers"] = args.layers
    V, D = c["vocab_size"], c["hidden_size"]
    chunk = -(-V // R)
    torch.manual_seed(1234 + rank)
    with torch.device(dev):
        blocks = nn.ModuleList(TPBlock(c, R, group, gn) for _ in range(c["num_hidden_layers"]))
        embed = nn.Parameter(torch.empty(chunk, D, dtype=torch.bfloat16))          # vocabulary rows [rank*chunk, ...)
        head = nn.Parameter(torch.empty(V, D, dtype=torch.bfloat16))               # replicated, gradient all-reduced
        final_norm = nn.RMSNorm(D, eps=1e-6, dtype=torch.bfloat16)
    params = list(blocks.parameters()) + [embed, head] + list(final_norm.parameters())
    replicated = [p for n, p in blocks.named_parameters() if "norm" in n or "ln" in n] + [head] + list(final_norm.parameters())
    with torch.no_grad():
        for p in params:
            p.normal_(0.0, 0.02) if p.dim() > 1 else p.fill_(1.0)
        for p in replicated:
            dist.broadcast(p, src=0)
    # bf16 compute parameters with fp32 masters and moments, as FSDP2's mixed-precision policy keeps them in the reference
    masters = [p.detach().float().requires_grad_() for p in params]
    opt = torch.optim.AdamW(masters, lr=3e-4, weight_decay=0.0, fused=True)
    B = args.global_batch or world * args.micro_batch            # sequences per step (dp = 1)
    S = args.seq
    T = B * S
    cr = T // R
    gen = torch.Generator().manual_seed(0)
    cos, sin = _rope_tables(S, c["head_dim"], c["rope_theta"], dev)
    pin = torch.empty(B, S, dtype=torch.int64).pin_memory()

    def step(read=True):
        pin.copy_(torch.randint(0, V, (B, S), generator=gen))
        ids = pin.to(dev, non_blocking=True).view(-1)
        labels = torch.cat([ids.view(B, S)[:, 1:], torch.full((B, 1), -100, device=dev)], 1).reshape(-1)
        gv = (labels != -100).sum().float()
        local = ids - rank * chunk
        mine = (local >= 0) & (local < chunk)
        rows = F.embedding(local.clamp(0, chunk - 1), embed) * mine[:, None].to(torch.bfloat16)
        x = _ReduceScatter.apply(rows, group)                           # [T/R, D]
        for blk in blocks:
            x = checkpoint(blk, x, cos, sin, B, use_reentrant=False)
        h = final_norm(x)
        hd = h.detach().requires_grad_()
        lab = labels[rank * cr:(rank + 1) * cr]
        total = torch.zeros((), device=dev)
        n = max(1, args.loss_chunks)
        stepn = -(-cr // n)
        for s in range(0, cr, stepn):
            l = F.cross_entropy(F.linear(hd[s:s + stepn], head).float(), lab[s:s + stepn], ignore_index=-100, reduction="sum") / gv
            l.backward()
            total += l.detach()
        h.backward(hd.grad)
        flat = torch.cat([p.grad.reshape(-1).float() for p in replicated])
        dist.all_reduce(flat, group=group)
        off = 0
        for p in replicated:
            p.grad.copy_(flat[off:off + p.numel()].view_as(p)); off += p.numel()
        rep_ids = {id(p) for p in replicated}
        sq = torch.stack([p.grad.float().pow(2).sum() for p in params if id(p) not in rep_ids]).sum()
        dist.all_reduce(sq, group=group)
        norm = (sq + flat.pow(2).sum()).sqrt()
        coef = torch.clamp(1.0 / (norm + 1e-6), max=1.0)
        for m, p in zip(masters, params):
            m.grad = p.grad.float() * coef
            p.grad = None
        opt.step(); opt.zero_grad(set_to_none=True)
        with torch.no_grad():
            torch._foreach_copy_(params, masters)
        if read:
            dist.all_reduce(total, group=group)
            return float(total), float(norm)
        return None

    warm, ms, ms2, outs = _time_steps(step, args, world, dev)
    tok = T
    cfgm = Qwen3Config(**c)
    res = {"impl": "stock", "metric": f"training tokens/sec/box (device-timed, max over ranks), qwen3_8b tp{R} bf16 seq {S}",
           "value": tok * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
           "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic uniform-random tokens, random-init weights",
           "config": {"model": args.model + (f"[layers={args.layers}]" if args.layers else ""), "global_batch": B, "seq_len": S,
                      "parallelism": f"tp{R}", "stack": "torch symm_mem fused_all_gather_matmul / fused_matmul_reduce_scatter + cuBLAS + SDPA + fused AdamW"},
           "e2e": {"value": tok * args.steps / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2 / args.steps},
           "tflops_per_gpu": tok * args.steps / (ms / 1e3) / world * cfgm.flops_per_token(S) / 1e12,
           "final_loss": outs[-1][0] if outs else None, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30, "gpu_launches": 0}
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()
    return 0


# ================================================================================================ expert parallel
class EPMoE(nn.Module):
    """Top-k softmax router + experts sharded over the EP group, all-to-all token dispatch with exact split sizes."""

    def __init__(self, c, R, group):
        super().__init__()
        D, E, Fe = c["hidden_size"], c["num_experts"], c["moe_intermediate_size"]
        self.E, self.El, self.k, self.R, self.group = E, E // R, c["num_experts_per_tok"], R, group
        self.gate = nn.Linear(D, E, bias=False)
        # fp32 masters outside FSDP (each expert lives on exactly one rank); cast to bf16 for the products
        self.w13 = nn.Parameter(torch.empty(self.El, D, 2 * Fe))     # [G, K, N] for torch._grouped_mm
        self.w2 = nn.Parameter(torch.empty(self.El, Fe, D))
        self.Fe = Fe

    def forward(self, x):
        from torch.distributed._functional_collectives import all_to_all_single_autograd
        T, D = x.shape
        logits = torch.mm(x.float(), self.gate.weight.float().t())
        scores = torch.softmax(logits, -1)
        w, idx = scores.topk(self.k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)                              # copies sorted by destination expert
        counts = torch.bincount(flat, minlength=self.E)
        recv = torch.empty_like(counts)
        dist.all_to_all_single(recv, counts, group=self.group)               # [R sources][El]
        send_splits = counts.view(self.R, self.El).sum(1).tolist()            # host reads of the split sizes
        recv_mat = recv.view(self.R, self.El)
        recv_splits = recv_mat.sum(1).tolist()
        xs = x[order // self.k]
        got = all_to_all_single_autograd(xs, recv_splits, send_splits, self.group)       # rank-major blocks
        # rank-major -> expert-major
        expert_of = torch.repeat_interleave(torch.arange(self.El, device=x.device).repeat(self.R), recv_mat.reshape(-1))
        perm = torch.argsort(expert_of, stable=True)
        rows = got[perm]
        offs = recv_mat.sum(0).cumsum(0).to(torch.int32)
        w13, w2 = self.w13.to(torch.bfloat16), self.w2.to(torch.bfloat16)
        if rows.shape[0] > 0:
            h = torch._grouped_mm(rows, w13, offs=offs)
            h = F.silu(h[:, : self.Fe]) * h[:, self.Fe:]
            y = torch._grouped_mm(h, w2, offs=offs)
        else:
            y = rows.new_zeros(0, D) + 0.0 * (w13.sum() + w2.sum())
        back = torch.empty_like(y)
        back[perm] = y
        ret = all_to_all_single_autograd(back, send_splits, recv_splits, self.group)
        out = torch.zeros(T, D, dtype=torch.float32, device=x.device)
        out.index_add_(0, order // self.k, ret.float() * w.reshape(-1)[order][:, None])
        return out.to(x.dtype)


class EPBlock(nn.Module):
    def __init__(self, c, R, group):
        super().__init__()
        D, d = c["hidden_size"], c["head_dim"]
        self.hq, self.hk, self.d = c["num_attention_heads"], c["num_key_value_heads"], d
        lin = lambda i, o: nn.Linear(i, o, bias=False)       # noqa: E731  (fp32 masters, bf16 compute through FSDP2's policy)
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = lin(D, self.hq * d), lin(D, self.hk * d), lin(D, self.hk * d), lin(self.hq * d, D)
        self.q_norm, self.k_norm = nn.RMSNorm(d, eps=1e-6), nn.RMSNorm(d, eps=1e-6)
        self.ln1, self.ln2 = nn.RMSNorm(D, eps=1e-6), nn.RMSNorm(D, eps=1e-6)
        self.moe = EPMoE(c, R, group)

    def forward(self, x, cos, sin):
        B, S, D = x.shape
        h = self.ln1(x)
        q = self.q_norm(self.q_proj(h).view(B, S, self.hq, self.d)).transpose(1, 2)
        k = self.k_norm(self.k_proj(h).view(B, S, self.hk, self.d)).transpose(1, 2)
        v = self.v_proj(h).view(B, S, self.hk, self.d).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.o_proj(o.transpose(1, 2).reshape(B, S, -1))
        return x + self.moe(self.ln2(x).view(B * S, D)).view(B, S, D)


class EPModel(nn.Module):
    def __init__(self, c, R, group):
        super().__init__()
        V, D = c["vocab_size"], c["hidden_size"]
        self.layers = nn.ModuleList(EPBlock(c, R, group) for _ in range(c["num_hidden_layers"]))
        self.embed = nn.Embedding(V, D)
        self.norm = nn.RMSNorm(D, eps=1e-6)
        self.head = nn.Linear(D, V, bias=False)

    def forward(self, ids, cos, sin):
        from torch.utils.checkpoint import checkpoint
        x = self.embed(ids)
        for l in self.layers:
            x = checkpoint(l, x, cos, sin, use_reentrant=False)
        return self.norm(x)


def run_stock_ep(args) -> int:
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from torch.utils.checkpoint import checkpoint
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from torchllmtuner_b200.models.qwen3 import QWEN3_30B_A3B, Qwen3Config
    world, rank, dev = _init_dist()
    R = args.ep
    assert R == world, "the stock expert-parallel arm runs EP (and FSDP of the dense parameters) over all ranks"
    group = dist.group.WORLD
    c = dict(QWEN3_30B_A3B)
    if args.layers:
        c["num_hidden_layers"] = args.layers
    V, D = c["vocab_size"], c["hidden_size"]
    torch.manual_seed(0)
    with torch.device(dev):
        model = EPModel(c, R, group)
    layers, head = model.layers, model.head
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.fill_(1.0) if p.dim() == 1 else p.normal_(0.0, 0.02)
    experts = {p for l in layers for p in (l.moe.w13, l.moe.w2)}
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for l in layers:
        fully_shard(l, mp_policy=mp, ignored_params={l.moe.w13, l.moe.w2})
    fully_shard(model, mp_policy=mp, ignored_params=experts)
    # sharded (DTensor) parameters and the plain expert tensors cannot share one fused update
    opt = torch.optim.AdamW([p for p in model.parameters() if p not in experts], lr=3e-4, weight_decay=0.0, fused=True)
    opt_e = torch.optim.AdamW(list(experts), lr=3e-4, weight_decay=0.0, fused=True)
    B, S = args.micro_batch, args.seq
    cos, sin = _rope_tables(S, c["head_dim"], c["rope_theta"], dev)
    gen = torch.Generator().manual_seed(rank)
    pin = torch.empty(B, S, dtype=torch.int64).pin_memory()

    def step(read=True):
        pin.copy_(torch.randint(0, V, (B, S), generator=gen))
        ids = pin.to(dev, non_blocking=True)
        labels = torch.cat([ids[:, 1:], torch.full((B, 1), -100, device=dev)], 1).reshape(-1)
        gv = (labels != -100).sum().float()
        dist.all_reduce(gv)
        h = model(ids, cos, sin).view(B * S, D)
        hd = h.detach().requires_grad_()
        total = torch.zeros((), device=dev)
        n = max(1, args.loss_chunks)
        stepn = -(-B * S // n)
        w = head.weight
        for s in range(0, B * S, stepn):
            l = F.cross_entropy(F.linear(hd[s:s + stepn], w.to(torch.bfloat16)).float(), labels[s:s + stepn], ignore_index=-100, reduction="sum") / gv
            l.backward()
            total += l.detach()
        h.backward(hd.grad)
        gn = torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p not in experts], 1.0)
        torch.nn.utils.clip_grad_norm_(list(experts), 1.0)
        opt.step(); opt.zero_grad(set_to_none=True)
        opt_e.step(); opt_e.zero_grad(set_to_none=True)
        if read:
            dist.all_reduce(total)
            gn = gn.full_tensor() if hasattr(gn, "full_tensor") else gn
            return float(total), float(gn)
        return None

    warm, ms, ms2, outs = _time_steps(step, args, world, dev)
    tok = world * B * S
    cfgm = Qwen3Config(**c)
    res = {"impl": "stock", "metric": f"training tokens/sec/box (device-timed, max over ranks), qwen3_30b_a3b fsdp{world}+ep{R} bf16 seq {S}",
           "value": tok * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
           "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic uniform-random tokens, random-init weights",
           "config": {"model": args.model + (f"[layers={args.layers}]" if args.layers else ""), "global_batch": world * B, "seq_len": S,
                      "parallelism": f"fsdp{world}+ep{R}", "stack": "funcol all_to_all_single + torch._grouped_mm + FSDP2 + SDPA + fused AdamW"},
           "e2e": {"value": tok * args.steps / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2 / args.steps},
           "tflops_per_gpu": tok * args.steps / (ms / 1e3) / world * cfgm.flops_per_token(S) / 1e12,
           "final_loss": outs[-1][0] if outs else None, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30, "gpu_launches": 0}
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()
    return 0
