"""Reference arm of the benchmark: drives the unmodified reference (installed under `baseline/_ref`) through its own
public entry points, `llmtuner.trainer.cli.parse_config` and `llmtuner.Trainer(config).train_step()`, with the flat flags
of the benchmark configuration. Nothing of this repository's models, kernels or engine is on that path.

It is reached only when `import llmtuner.trainer.cli` succeeds (see `bench.py::reference_arm`); with the torch 2.11 of
this image the import fails and the arm prints its `unavailable` line instead. Dense Qwen3 is expressed the reference's
way: `qwen3_moe` with every layer listed in `mlp_only_layers` (its examples/qwen3-dense recipe does the same).
"""
from __future__ import annotations

import json
import os
import sys


def _flags(args, world: int) -> list[str]:
    dense = args.model == "qwen3_8b"
    dp = world // max(1, args.tp)
    sizes = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                 num_key_value_heads=8) if dense else dict(vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
                                                           num_attention_heads=32, num_key_value_heads=4)
    flat = dict(model_name_or_path="qwen3_moe", initialization_device="meta", global_batch_size=dp * args.micro_batch,
                max_seq_len=args.seq, steps=10 ** 6, activation_checkpoint_mode=args.ac, seed=0, dump_folder="/tmp/llmt_ref_bench",
                data_parallel_shard_size=dp, tensor_parallel_size=args.tp, expert_parallel_size=args.ep, log_freq=10 ** 6,
                compute_dtype="bfloat16", **sizes)
    out = []
    for k, v in flat.items():
        out += [f"--{k}", str(v)]
    if dense:
        out += ["--arch_overrides", json.dumps({"mlp_only_layers": list(range(36)), "head_dim": 128})]
    else:
        out += ["--arch_overrides", json.dumps({"num_experts": 128, "num_experts_per_tok": 8, "moe_intermediate_size": 768, "head_dim": 128})]
    return out


def run_reference(args, ref_root: str) -> int:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sys.path.insert(0, ref_root)
    try:
        import torch
        import torch.distributed as dist
        import llmtuner
        from llmtuner.trainer.cli import parse_config
        cfg = parse_config(_flags(args, world))
        trainer = llmtuner.Trainer(cfg)
        warm = max(3, args.warmup)
        for _ in range(warm):
            trainer.train_step()

        def sync():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            trainer.train_step()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        tokens = int(cfg.training.global_batch_size) * args.seq * args.steps
        line = {"impl": "reference", "metric": f"training tokens/sec/box (device-timed, max over ranks), {args.model} bf16 seq {args.seq}",
                "value": tokens / (float(ms.item()) / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": float(ms.item()) / args.steps, "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
                "data": "synthetic uniform-random tokens, random-init weights",
                "e2e": {"value": tokens / (float(ms.item()) / 1e3), "unit": "tokens/s",
                        "note": "the reference's train_step reads its batch from the host loader and its loss back every step"}}
        trainer.close()
    except BaseException as e:      # the arm must print one line and exit 0 whatever the reference does
        line = {"impl": "reference", "unavailable": f"the reference raised {type(e).__name__}: {str(e)[:240]}"}
    if rank == 0:
        print(json.dumps(line))
    return 0
