"""Single-GPU runs through the public Trainer API: memory options must not change the numbers."""
import pytest
import torch

from torchllmtuner_b200 import LLMTunerConfig, Trainer

pytestmark = pytest.mark.gpu


def _cfg(**flat):
    cfg = LLMTunerConfig()
    base = dict(model_name_or_path="qwen3", vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, global_batch_size=2, max_seq_len=1024, steps=3, seed=0,
                dump_folder="/tmp/llmt_gpu_train", deterministic=False)
    base.update(flat)
    cfg.apply_flat(base)
    return cfg


def _run(cfg):
    tr = Trainer(cfg)
    out = []
    try:
        for _ in range(cfg.training.steps):
            tr.dataloader.cursor = 0
            out.append(tr.train_step().loss)
        extra = getattr(tr.model, "activation_swap", None)
        stats = dict(extra.stats) if extra is not None else None
    finally:
        tr.close()
    return out, stats


def test_activation_swap_offloads_saved_tensors_and_keeps_the_losses():
    ref, _ = _run(_cfg())
    got, stats = _run(_cfg(activation_swap=True))
    assert stats is not None and stats["swapped"] > 0, stats
    assert max(abs(a - b) for a, b in zip(ref, got)) < 1e-3, (ref, got)


def test_full_and_region_checkpointing_keep_the_losses():
    ref, _ = _run(_cfg(num_hidden_layers=4))
    full, _ = _run(_cfg(num_hidden_layers=4, activation_checkpoint_mode="full"))
    cfg = _cfg(num_hidden_layers=4, activation_checkpoint_mode="region")
    cfg.training.region_ac.recompute_regions = [r"layers\.(0|2)$"]
    region, _ = _run(cfg)
    for got in (full, region):
        assert max(abs(a - b) for a, b in zip(ref, got)) < 1e-3, (ref, got)


def test_host_resident_optimizer_state_keeps_the_losses():
    ref, _ = _run(_cfg())
    got, _ = _run(_cfg(fsdp_cpu_offload=True))
    assert max(abs(a - b) for a, b in zip(ref, got)) < 1e-3, (ref, got)
