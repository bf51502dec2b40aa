"""Headline benchmark: training tokens/s of Qwen3-8B (FSDP over N GPUs of one node, bf16, sequence 8192, one sequence per
GPU and step, full activation checkpointing, synthetic uniform-random tokens, random-init weights).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Two timed regions, both CUDA-event timed on the launching stream between barrier + synchronize, max over ranks:
  value : K optimizer steps with the step's inputs already resident on the device and no host read of the result
  e2e   : K optimizer steps through `Trainer.train_step()`: every step copies its inputs from pinned host memory to the
          device and reads the step's loss / grad-norm back to the host
Rank 0 prints one JSON line. `--impl reference` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMI_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (read only)."""

    def __init__(self, gpu_index: int):
        self.path = f"/tmp/llmt_clocks_{os.getpid()}.csv"
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        os.unlink(self.path)
        if not sm:
            return {}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> int:
    """Runs the unmodified reference from `baseline/_ref` through its own CLI entry point. The attempt is real: the
    reference's trainer module is imported in a child interpreter with `baseline/_ref` first on the path, and the line
    printed when that fails carries the exception the import actually raised."""
    import subprocess
    root = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(root, "baseline", "_ref")
    rank0 = int(os.environ.get("RANK", "0")) == 0
    if not os.path.isdir(os.path.join(ref, "llmtuner")):
        why = "baseline/_ref/llmtuner is absent: the offline install of the reference was not done on this machine"
    else:
        probe = ("import sys; sys.path.insert(0, sys.argv[1]); import llmtuner.trainer.cli as c; "
                 "import torch.distributed.fsdp as f; f.DataParallelMeshDims; print('ok')")
        r = subprocess.run([sys.executable, "-c", probe, ref], capture_output=True, text=True, timeout=600)
        if r.returncode == 0 and r.stdout.strip().endswith("ok"):
            # The reference imports: hand over to its own CLI with the benchmark's configuration.
            from baseline.reference_cli import run_reference
            return run_reference(args, ref)
        last = [ln for ln in (r.stderr or r.stdout).strip().splitlines() if ln.strip()]
        why = "import of the reference's trainer failed: " + (last[-1].strip() if last else f"exit code {r.returncode}")
        why = why[:300] + f" (torch {__import__('torch').__version__}; the reference needs torch>=2.12)"
    if rank0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def build_config(args, world: int):
    from torchllmtuner_b200 import LLMTunerConfig
    cfg = LLMTunerConfig()
    dp = world // (args.tp * args.cp_ulysses * args.cp_kv)
    gb = args.global_batch or dp * args.micro_batch * args.accum
    flat = dict(model_name_or_path=args.model, initialization_device="meta", global_batch_size=gb,
                max_seq_len=args.seq, steps=10 ** 6, activation_checkpoint_mode=args.ac, chunked_loss_num_chunks=args.loss_chunks,
                seed=0, dump_folder="/tmp/llmt_bench", data_parallel_shard_size=dp, log_freq=10 ** 6, gc_freq=10 ** 6,
                fsdp_implementation=args.fsdp_impl, deterministic=False, gradient_accumulation_steps=args.accum)
    if args.qkv == "fused":
        flat["qkv_projection"] = "fused"
    if args.dataset != "random":
        flat["dataset"] = args.dataset
    if args.tp > 1:
        flat["tensor_parallel_size"] = args.tp
    if args.ep > 1:
        flat["expert_parallel_size"] = args.ep
    if args.cp_ulysses > 1:
        flat["context_parallel_ulysses_size"] = args.cp_ulysses
    if args.cp_kv > 1:
        flat.update(context_parallel_kv_allgather_size=args.cp_kv, context_parallel_load_balancer="headtail")
    cfg.apply_flat(flat)
    if args.layers:
        cfg.model.arch_overrides = dict(cfg.model.arch_overrides, num_hidden_layers=args.layers)
    return cfg


def _tp_stats():
    try:
        from torchllmtuner_b200.parallel import symm_tp
        for c in symm_tp._COMMS.values():
            return dict(c.stats)
    except Exception:
        pass
    return None


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "stock"])
    ap.add_argument("--model", default="qwen3_8b")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--ac", default="full")
    ap.add_argument("--loss-chunks", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (the result is then not the headline metric)")
    ap.add_argument("--fsdp-impl", default="native", choices=["native", "custom"])
    ap.add_argument("--qkv", default="separate", choices=["separate", "fused"], help="q/k/v as three GEMMs or one")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (sequence parallel); the rest of the GPUs shard with FSDP")
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel degree (MoE models)")
    ap.add_argument("--cp-ulysses", type=int, default=1)
    ap.add_argument("--cp-kv", type=int, default=1)
    ap.add_argument("--global-batch", type=int, default=0, help="sequences per step over the whole job (default: one per data-parallel rank)")
    ap.add_argument("--accum", type=int, default=1, help="gradient accumulation steps")
    ap.add_argument("--dataset", default="random", choices=["random", "random_packed"],
                    help="random: one document per row; random_packed: rows packed from documents of log-uniform length 512..32768")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "stock":
        from baseline.stock_arm import run_stock
        return run_stock(args)

    import torch
    import torch.distributed as dist
    from torchllmtuner_b200 import Trainer
    from torchllmtuner_b200.ops.cuda_ext import check_status, load
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1"
    warm = max(3, args.warmup)
    cfg = build_config(args, world)
    tr = Trainer(cfg)
    dev = tr.env.device
    ext = load()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, k: int) -> float:
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident inputs for the kernel-only region
    def device_batch():
        b = next(tr.data_iterator)
        return [{k: (v.to(dev) if isinstance(v, torch.Tensor) and k != "cu_seqlens" else v) for k, v in b.items()}]

    # the same call the training loop makes (`Trainer._run_training`): with `overlap_optimizer_step` (default on) the update
    # of a single-shard-rank run goes to its own stream and the next forward waits unit by unit
    ov = bool(cfg.training.overlap_optimizer_step)
    for _ in range(warm):
        tr.train_step(overlap_optimizer=ov)
    check_status("bench warm-up")
    pre = [device_batch() for _ in range(args.steps)]
    it = iter(pre)
    sampler = ClockSampler(tr.env.local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    n0 = ext.launch_count()
    ms_dev = timed(lambda: tr.train_step(batches=next(it), read_stats=False, overlap_optimizer=ov), args.steps)
    launches = ext.launch_count() - n0
    fused = getattr(getattr(tr.asm, "fsdp", None), "fused", None)
    qs = dict(fused.queue.stats) if fused is not None and fused.queue is not None else None
    clocks = sampler.stop() if sampler else {}
    # ---- end to end: pinned host -> device copy of every step's inputs, loss read back every step
    h2d = d2h = 0
    probe = next(tr.data_iterator)
    h2d = sum(v.numel() * v.element_size() for k, v in probe.items() if isinstance(v, torch.Tensor) and k != "cu_seqlens")
    d2h = 4 * 4                       # one read per step: loss sum, gradient norm, valid tokens, kernel status code
    results = []
    ms_e2e = timed(lambda: results.append(tr.train_step(overlap_optimizer=ov)), args.steps)
    check_status("bench")
    tokens_per_step = cfg.training.global_batch_size * args.seq
    par = "+".join(p for p in (f"fsdp{tr.env.topo.dp_shard}" if tr.env.topo.dp_shard > 1 or world == 1 else "", f"tp{args.tp}" if args.tp > 1 else "",
                               f"ep{args.ep}" if args.ep > 1 else "", f"cp_ulysses{args.cp_ulysses}" if args.cp_ulysses > 1 else "",
                               f"cp_kv{args.cp_kv}" if args.cp_kv > 1 else "") if p)
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e = tokens_per_step * args.steps / (ms_e2e / 1e3)
    fpt = tr.model.flops_per_token(args.seq)
    mem = torch.cuda.max_memory_allocated() / 2 ** 30
    out = {"metric": f"training tokens/sec/box (device-timed, max over ranks), {args.model} {par} bf16 seq {args.seq}", "value": value,
           "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_dev / args.steps,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens" + (" packed from documents of log-uniform length 512..32768" if args.dataset == "random_packed" else "") + ", random-init weights",
           "config": {"model": args.model + (f"[layers={args.layers}]" if args.layers else ""), "global_batch": cfg.training.global_batch_size,
                      "seq_len": args.seq, "parallelism": par, "activation_checkpointing": args.ac, "optimizer_overlap": ov,
                      "loss": f"chunked x{args.loss_chunks}", "l2": "inputs (16 GB of weights per step) larger than the 126 MB L2",
                      "fsdp_implementation": args.fsdp_impl},
           "clocks": clocks, "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d,
                                      "d2h_bytes_per_step": d2h},
           "gpu_launches": int(launches), "mfu_nominal_pct": 100 * value / world * fpt / 2.25e15,
           "tflops_per_gpu": value / world * fpt / 1e12, "final_loss": results[-1].loss if results else None,
           "peak_mem_gib": mem, "impl": "ours",
           "tp_fused": _tp_stats(),
           "comm_fused_fraction": (qs["bytes_fused"] / max(1, qs["bytes_fused"] + qs["bytes_standalone"])) if qs else None}
    tr.close()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
