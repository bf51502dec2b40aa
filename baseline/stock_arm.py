"""Stock-PyTorch arm: the same Qwen3 architecture, data, loss normalisation and schedule as `bench.py`'s own arm, driven
through the library calls the reference makes on CUDA: `nn.Linear` (cuBLAS), `F.scaled_dot_product_attention`,
`F.rms_norm`, torch FSDP2 `fully_shard` with bf16 parameters / fp32 reduction, `torch.utils.checkpoint` for full
activation checkpointing, chunked head + `F.cross_entropy`, `torch.optim.AdamW(fused=True)` and `clip_grad_norm_`
(reference: llmtuner/models/qwen/qwen3/model.py:125-285, llmtuner/parallel/fully_shard_parallel/fully_shard_parallel.py:198-604,
llmtuner/components/loss.py:246-316, llmtuner/components/optimizer/optimizer.py:62-106). It is a stand-in, not the
reference itself (which cannot be installed offline), and prints `"impl": "stock"`."""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), -1)


class Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        D, d = c["hidden_size"], c["head_dim"]
        self.hq, self.hk, self.d = c["num_attention_heads"], c["num_key_value_heads"], d
        self.q_proj = nn.Linear(D, self.hq * d, bias=False); self.k_proj = nn.Linear(D, self.hk * d, bias=False)
        self.v_proj = nn.Linear(D, self.hk * d, bias=False); self.o_proj = nn.Linear(self.hq * d, D, bias=False)
        self.q_norm = nn.RMSNorm(d, eps=1e-6); self.k_norm = nn.RMSNorm(d, eps=1e-6)
        self.input_layernorm = nn.RMSNorm(D, eps=1e-6); self.post_attention_layernorm = nn.RMSNorm(D, eps=1e-6)
        F_ = c["intermediate_size"]
        self.gate_proj = nn.Linear(D, F_, bias=False); self.up_proj = nn.Linear(D, F_, bias=False); self.down_proj = nn.Linear(F_, D, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        h = self.input_layernorm(x)
        q = self.q_norm(self.q_proj(h).view(B, S, self.hq, self.d)).transpose(1, 2)
        k = self.k_norm(self.k_proj(h).view(B, S, self.hk, self.d)).transpose(1, 2)
        v = self.v_proj(h).view(B, S, self.hk, self.d).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.o_proj(o.transpose(1, 2).reshape(B, S, -1))
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class Model(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c = c
        self.embed_tokens = nn.Embedding(c["vocab_size"], c["hidden_size"])
        self.layers = nn.ModuleList(Block(c) for _ in range(c["num_hidden_layers"]))
        self.norm = nn.RMSNorm(c["hidden_size"], eps=1e-6)
        self.lm_head = nn.Linear(c["hidden_size"], c["vocab_size"], bias=False)

    def forward(self, ids):
        from torch.utils.checkpoint import checkpoint
        B, S = ids.shape
        d = self.c["head_dim"]
        inv = 1.0 / (self.c["rope_theta"] ** (torch.arange(0, d, 2, device=ids.device, dtype=torch.float32) / d))
        ang = torch.arange(S, device=ids.device, dtype=torch.float32)[:, None] * inv[None]
        cos, sin = ang.cos().to(torch.bfloat16)[None, None], ang.sin().to(torch.bfloat16)[None, None]
        x = self.embed_tokens(ids)
        for l in self.layers:
            x = checkpoint(l, x, cos, sin, use_reentrant=False)
        return self.norm(x)


def run_stock(args) -> int:
    if getattr(args, "tp", 1) > 1 and args.model == "qwen3_8b" and getattr(args, "ep", 1) == 1:
        from baseline.stock_parallel import run_stock_tp
        return run_stock_tp(args)
    if getattr(args, "ep", 1) > 1 and args.model == "qwen3_30b_a3b" and getattr(args, "tp", 1) == 1:
        from baseline.stock_parallel import run_stock_ep
        return run_stock_ep(args)
    if getattr(args, "tp", 1) > 1 or getattr(args, "ep", 1) > 1 or getattr(args, "cp_ulysses", 1) > 1 or getattr(args, "cp_kv", 1) > 1 \
            or args.model != "qwen3_8b":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "stock", "unavailable": "the stock-PyTorch arms cover dense FSDP, TP + SP over all ranks and "
                              "EP over all ranks; the reference itself rejects context parallelism for Qwen models "
                              "(llmtuner/parallel/context_parallel/plan.py:27-34)"}))
        return 0
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from torchllmtuner_b200.datasets import RandomTokenDataLoader, RandomTokenSource
    from torchllmtuner_b200.models.qwen3 import QWEN3_8B, Qwen3Config
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    c = dict(QWEN3_8B)
    if args.layers:
        c["num_hidden_layers"] = args.layers
    torch.manual_seed(0)
    with torch.device("meta"):
        model = Model(c)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for l in model.layers:
        fully_shard(l, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    model.to_empty(device=dev)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n:
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.0, fused=True)
    src = RandomTokenSource(c["vocab_size"], world * args.micro_batch, args.seq, 0)
    loader = RandomTokenDataLoader(src, rank, world, args.micro_batch, pin_memory=True)
    chunks = max(1, args.loss_chunks)

    def step(read=True):
        b = next(loader)
        ids, labels = b["input"].to(dev, non_blocking=True), b["labels"].to(dev, non_blocking=True)
        gv = torch.tensor([float(b["num_valid_tokens"])], device=dev)
        if world > 1:
            dist.all_reduce(gv)
        h = model(ids)
        hd = h.detach().requires_grad_()
        T = hd.shape[0] * hd.shape[1]
        hf, lf = hd.view(T, -1), labels.view(T)
        total = torch.zeros((), device=dev)
        stepn = -(-T // chunks)
        w = model.lm_head.weight
        for s in range(0, T, stepn):
            logits = F.linear(hf[s:s + stepn], w.to(torch.bfloat16) if w.dtype != torch.bfloat16 else w)
            l = F.cross_entropy(logits.float(), lf[s:s + stepn], ignore_index=-100, reduction="sum") / gv[0]
            l.backward()
            total += l.detach()
        h.backward(hd.grad)
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step(); opt.zero_grad(set_to_none=True)
        return (float(total), float(norm)) if read else None

    warm = max(3, args.warmup)
    for _ in range(warm):
        step()

    def timed(k, read):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = [step(read) for _ in range(k)]
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms), out
    ms, _ = timed(args.steps, False)
    ms2, outs = timed(args.steps, True)
    tok = world * args.micro_batch * args.seq
    cfgm = Qwen3Config(**c)
    res = {"impl": "stock", "metric": "training tokens/sec/box (device-timed, max over ranks), Qwen3-8B FSDP bf16 seq 8192",
           "value": tok * args.steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
           "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic uniform-random tokens, random-init weights",
           "config": {"model": args.model, "global_batch": world * args.micro_batch, "seq_len": args.seq, "parallelism": f"fsdp{world}",
                      "stack": "torch FSDP2 + cuBLAS nn.Linear + SDPA + fused AdamW + torch.utils.checkpoint"},
           "e2e": {"value": tok * args.steps / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2 / args.steps},
           "tflops_per_gpu": tok * args.steps / (ms / 1e3) / world * cfgm.flops_per_token(args.seq) / 1e12,
           "final_loss": outs[-1][0] if outs else None, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30, "gpu_launches": 0}
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()
    return 0
