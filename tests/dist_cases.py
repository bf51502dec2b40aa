"""Rank bodies of the multi-process tests. Each case trains a tiny model through the public Trainer API and returns
per-step losses from rank 0; the parent compares arms (the two-arm equivalence pattern of the reference's integration
scripts, e.g. tests/integration_tests/fsdp_mesh_equivalence.py, tp_equivalence.py, ep_equivalence.py)."""
import json
import os
import sys

import torch


def base_flat(**over):
    d = dict(model_name_or_path="qwen3", vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
             num_attention_heads=4, num_key_value_heads=2, global_batch_size=4, max_seq_len=32, steps=3, learning_rate=3e-3,
             seed=0, dump_folder="/tmp/llmt_dist_out", deterministic=True)
    d.update(over)
    return d


def train_case(flat: dict, arch: dict | None, out_path: str, steps: int = 3, repeat_batch: bool = True):
    """Special keys in `flat` (removed before the config is built): `_load` resumes from the run folder first,
    `_save_at` saves a full checkpoint after that many steps."""
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    flat = dict(flat)
    do_load, save_at = flat.pop("_load", False), flat.pop("_save_at", None)
    cfg = LLMTunerConfig()
    cfg.apply_flat(flat)
    if arch:
        cfg.model.arch_overrides = arch
    tr = Trainer(cfg)
    if do_load:
        assert tr.checkpointer.load()
    losses, norms = [], []
    for i in range(steps):
        if save_at is not None and i == save_at:
            tr.checkpointer.save(tr.progress.step, force=True)
        if repeat_batch:
            tr.dataloader.cursor = 0
        r = tr.train_step()
        losses.append(r.loss)
        norms.append(r.grad_norm)
    if save_at is not None and save_at >= steps:
        tr.checkpointer.save(tr.progress.step, force=True)
    if int(os.environ.get("RANK", "0")) == 0:
        with open(out_path, "w") as f:
            extra = {}
            try:
                from torchllmtuner_b200.parallel import symm_tp
                for c in symm_tp._COMMS.values():
                    extra["tp_fused"] = dict(c.stats)
            except Exception:
                pass
            fused = getattr(tr.asm.fsdp, "fused", None)
            if fused is not None and fused.queue is not None:
                extra["fsdp_fused_units"] = len(fused.units)
                extra["fsdp_block_units"] = sum(len(us) for us in tr.asm.fsdp.block_units.values())
            json.dump({"loss": losses, "grad_norm": norms, **extra}, f)
    tr.close()
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def _worker(rank: int, world: int, port: int, flat: dict, arch, out_path: str, steps: int, device: str):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if device == "cpu":
        os.environ["LLMTUNER_DEVICE"] = "cpu"
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    torch.set_num_threads(1)
    train_case(flat, arch, out_path, steps)


def run_ranks(world: int, flat: dict, arch=None, steps: int = 3, device: str = "cpu", port: int | None = None) -> dict:
    import tempfile

    import torch.multiprocessing as mp
    out = tempfile.mktemp(suffix=".json")
    port = port or (20000 + (os.getpid() * 7 + world * 131 + len(json.dumps(flat))) % 20000)
    if world == 1:
        env_backup = {k: os.environ.pop(k, None) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
        try:
            if device == "cpu":
                os.environ["LLMTUNER_DEVICE"] = "cpu"
            train_case(flat, arch, out, steps)
        finally:
            for k, v in env_backup.items():
                if v is not None:
                    os.environ[k] = v
    else:
        mp.spawn(_worker, args=(world, port, flat, arch, out, steps, device), nprocs=world, join=True)
    with open(out) as f:
        res = json.load(f)
    os.unlink(out)
    return res


def _pp_worker(rank, world, port, flat, schedule, out_path, steps):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      LLMTUNER_DEVICE="cpu")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    torch.set_num_threads(1)
    import torch.distributed as dist
    from torchllmtuner_b200 import LLMTunerConfig
    from torchllmtuner_b200.experiments.pipeline_parallel import PipelineTrainer
    cfg = LLMTunerConfig()
    cfg.apply_flat(flat)
    tr = PipelineTrainer(cfg, schedule, None)
    losses = []
    for _ in range(steps):
        tr.loader.cursor = 0
        losses.append(tr.train_step())
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"loss": losses}, f)
    dist.barrier()
    dist.destroy_process_group()


def run_pp(world, flat, schedule="1F1B", steps=3):
    import tempfile

    import torch.multiprocessing as mp
    out = tempfile.mktemp(suffix=".json")
    port = 20000 + (os.getpid() * 11 + world * 17 + len(schedule)) % 20000
    mp.spawn(_pp_worker, args=(world, port, flat, schedule, out, steps), nprocs=world, join=True)
    with open(out) as f:
        res = json.load(f)
    os.unlink(out)
    return res
