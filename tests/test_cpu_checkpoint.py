"""Checkpoint save / resume through the Trainer, resharding across DP and EP degrees, HF round trip."""
import os
import shutil

import pytest
import torch

from dist_cases import base_flat, run_ranks
from torchllmtuner_b200 import LLMTunerConfig, Trainer


def _cfg(folder, **flat):
    cfg = LLMTunerConfig()
    d = base_flat(dump_folder=folder, enable=True, interval=2, steps=4, last_save_model_only=False)
    d.update(flat)
    cfg.apply_flat(d)
    return cfg


def test_save_resume_is_bit_exact(tmp_path):
    folder = str(tmp_path / "run")
    tr = Trainer(_cfg(folder))
    ref = []
    for _ in range(4):
        r = tr.train_step()
        ref.append(r.loss)
        tr.checkpointer.save(r.step)
    tr.close()
    assert os.path.exists(os.path.join(folder, "checkpoint", "step-2", ".metadata"))
    # resume from step 2 in a fresh trainer and replay steps 3, 4
    shutil.rmtree(os.path.join(folder, "checkpoint", "step-4"))
    tr2 = Trainer(_cfg(folder))
    assert tr2.checkpointer.load()
    assert tr2.progress.step == 2
    got = [tr2.train_step().loss for _ in range(2)]
    tr2.close()
    assert got == ref[2:], (got, ref)


def test_keep_latest_k_and_atomic_publication(tmp_path):
    folder = str(tmp_path / "run")
    tr = Trainer(_cfg(folder, interval=1, keep_latest_k=2, steps=5))
    for _ in range(5):
        r = tr.train_step()
        tr.checkpointer.save(r.step)
    tr.close()
    names = sorted(os.listdir(os.path.join(folder, "checkpoint")))
    assert names == ["step-4", "step-5"], names
    # a folder without .metadata is never chosen
    os.makedirs(os.path.join(folder, "checkpoint", "step-9"))
    tr2 = Trainer(_cfg(folder, interval=1, keep_latest_k=2, steps=5))
    assert tr2.checkpointer.load() and tr2.progress.step == 5
    tr2.close()


def test_hf_export_import_round_trip(tmp_path):
    from torchllmtuner_b200.components.checkpointer.hf import load_hf_checkpoint, save_hf_checkpoint
    folder = str(tmp_path / "run")
    cfg = _cfg(folder, model_name_or_path="qwen3_moe")
    cfg.model.arch_overrides = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)
    tr = Trainer(cfg)
    tr.train_step()
    out = str(tmp_path / "hf")
    save_hf_checkpoint(tr, out, "float32")
    from safetensors import safe_open
    import json
    wm = json.load(open(os.path.join(out, "model.safetensors.index.json")))["weight_map"]
    assert "model.layers.0.mlp.experts.3.down_proj.weight" in wm and "model.layers.0.mlp.gate.weight" in wm
    before = [u.master.clone() for u in tr.asm.fsdp.units]
    for u in tr.asm.fsdp.units:
        u.master.zero_()
    load_hf_checkpoint(tr, out)
    for a, u in zip(before, tr.asm.fsdp.units):
        assert torch.equal(a[:u.numel], u.master[:u.numel])
    tr.close()


MOE = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)


def test_resume_at_other_dp_and_ep_degree(tmp_path):
    """Saved by 2 ranks with experts split over EP=2; resumed by one rank that owns every expert."""
    folder = str(tmp_path / "run")
    ck = dict(model_name_or_path="qwen3_moe", dump_folder=folder, enable=True, exclude_from_loading=["dataloader", "rng"])
    ref = run_ranks(1, base_flat(model_name_or_path="qwen3_moe"), arch=MOE, steps=4)
    run_ranks(2, base_flat(expert_parallel_size=2, data_parallel_shard_size=2, _save_at=2, **ck), arch=MOE, steps=2 + 0)
    # the 2-rank run trained 2 steps and saved before a third; resume on one rank and continue
    got = run_ranks(1, base_flat(_load=True, **ck), arch=MOE, steps=2)
    assert max(abs(a - b) for a, b in zip(ref["loss"][2:], got["loss"])) < 5e-5, (ref, got)


def test_checkpoint_key_names(tmp_path):
    """Keys follow the reference's flattened names: `model.<fqn>`, `optimizer.state.<fqn>.<moment>`, `ema.ema_params.<fqn>`,
    plus lr scheduler, train state, data loader and RNG entries."""
    import torch.distributed.checkpoint as dcp
    folder = str(tmp_path / "run")
    cfg = _cfg(folder)
    tr = Trainer(cfg)
    tr.train_step()
    tr.checkpointer.save(1, force=True)
    tr.checkpointer.wait()
    tr.close()
    keys = set(dcp.FileSystemReader(os.path.join(folder, "checkpoint", "step-1")).read_metadata().state_dict_metadata.keys())
    assert any(k.startswith("model.model.layers.0.self_attn.q_proj.weight@") for k in keys), sorted(keys)[:20]
    assert any(k.startswith("optimizer.state.model.layers.0.self_attn.q_proj.weight.exp_avg@") for k in keys)
    assert any(k.startswith("optimizer.state.model.layers.0.self_attn.q_proj.weight.exp_avg_sq@") for k in keys)
    for k in ("obj.lr_scheduler", "obj.train_state", "obj.format", "obj.optimizer.param_groups", "obj.dataloader.dp0", "obj.rng.rank0"):
        assert k in keys, k


def test_resume_at_other_tp_degree(tmp_path):
    """Saved by two tensor-parallel ranks (column / row shards of every projection, vocab-sharded embedding); resumed by
    one rank that holds full tensors, and the other way round."""
    folder = str(tmp_path / "run")
    ck = dict(dump_folder=folder, enable=True, exclude_from_loading=["dataloader", "rng"])
    ref = run_ranks(1, base_flat(), steps=4)
    run_ranks(2, base_flat(tensor_parallel_size=2, data_parallel_shard_size=1, _save_at=2, **ck), steps=2)
    got = run_ranks(1, base_flat(_load=True, **ck), steps=2)
    assert max(abs(a - b) for a, b in zip(ref["loss"][2:], got["loss"])) < 5e-5, (ref, got)
    folder2 = str(tmp_path / "run2")
    ck2 = dict(dump_folder=folder2, enable=True, exclude_from_loading=["dataloader", "rng"])
    run_ranks(1, base_flat(_save_at=2, **ck2), steps=2)
    got2 = run_ranks(2, base_flat(tensor_parallel_size=2, data_parallel_shard_size=1, _load=True, **ck2), steps=2)
    assert max(abs(a - b) for a, b in zip(ref["loss"][2:], got2["loss"])) < 5e-5, (ref, got2)


def test_async_checkpoint_is_published_in_a_later_step_and_adopted_after_a_crash(tmp_path):
    """A background save is renamed to `step-N` by the per-step hook as soon as it has finished, and a write that finished
    but was never renamed (the process died first) is adopted by the next load instead of resuming one interval earlier."""
    import time
    folder = str(tmp_path / "run")
    tr = Trainer(_cfg(folder, async_mode="async", interval=2, steps=8))
    tr.train_step(); r = tr.train_step()
    tr.checkpointer.save(r.step)                          # step 2, background write
    final = os.path.join(folder, "checkpoint", "step-2")
    for _ in range(200):                                  # the hook publishes without another save() or close()
        tr.checkpointer.maybe_wait_for_staging()
        if os.path.isdir(final):
            break
        time.sleep(0.05)
    assert os.path.exists(os.path.join(final, ".metadata"))
    assert tr.checkpointer._async_future is None
    tr.train_step(); r = tr.train_step()
    tr.checkpointer.save(r.step)                          # step 4: let the write finish, then "crash" before publication
    fut, tmp, final4, _ = tr.checkpointer._async_future
    fut.result()
    tr.checkpointer._async_future = None                  # the dying process never runs wait()
    assert os.path.isdir(tmp) and not os.path.isdir(final4)
    tr2 = Trainer(_cfg(folder, async_mode="async", interval=2, steps=8))
    assert tr2.checkpointer.load() and tr2.progress.step == 4
    assert os.path.isdir(final4) and not os.path.isdir(tmp)
    tr2.close()
    tr.close()
