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


def test_host_resident_moments_stream_through_two_device_slots_in_many_slices():
    """A 1 MiB slice budget cuts every unit into many slices: uploads, kernels and downloads of neighbouring slices
    overlap on three streams, the device holds two slices of moments, and the numbers do not change."""
    ref, _ = _run(_cfg())
    cfg = _cfg(optimizer_type="AdamWSwap", swap_max_device_bytes=1 << 20)
    tr = Trainer(cfg)
    try:
        got = []
        for _ in range(cfg.training.steps):
            tr.dataloader.cursor = 0
            got.append(tr.train_step().loss)
        stager = tr.optimizers.optimizers[0].stager
        assert stager is not None and stager.stats["slices"] > 3 * 8, stager.stats
        assert stager.stats["device_bytes"] == 2 * 2 * (1 << 20)
        assert stager.stats["uploaded_bytes"] == stager.stats["downloaded_bytes"] > 0
    finally:
        tr.close()
    assert max(abs(a - b) for a, b in zip(ref, got)) < 1e-3, (ref, got)


def _repeat_two_batches(tr, steps):
    """Random tokens carry nothing to learn unless they repeat: alternate between the first two batches of the stream."""
    out = []
    for i in range(steps):
        if i % 2 == 0:
            tr.dataloader.cursor = 0
        out.append(tr.train_step().loss)
    return out


def test_twenty_step_loss_curve_follows_the_fp32_oracle(tmp_path, monkeypatch):
    """The same model, weights and token stream trained twice through the public Trainer: once on the host in fp32 with
    the plain PyTorch statements of every op (the oracle), once on the GPU with the bf16 kernels. The weights travel
    through a checkpoint, so both runs start from identical parameters. The curves must track each other step by step;
    a kernel whose gradient is subtly wrong shows up as a drift that grows over the twenty steps."""
    steps = 20
    folder = str(tmp_path / "oracle")
    kw = dict(dump_folder=folder, enable=True, interval=1000, steps=steps, learning_rate=3e-3, warmup_steps=2,
              hidden_size=256, intermediate_size=512, max_seq_len=512, global_batch_size=4)
    monkeypatch.setenv("LLMTUNER_DEVICE", "cpu")
    tr = Trainer(_cfg(**kw))
    assert next(tr.model.parameters()).device.type == "cpu"
    tr.checkpointer.save(0, force=True)
    tr.checkpointer.wait()
    oracle = _repeat_two_batches(tr, steps)
    tr.close()
    monkeypatch.delenv("LLMTUNER_DEVICE")
    tr = Trainer(_cfg(exclude_from_loading=["rng"], **kw))
    assert next(tr.model.parameters()).device.type == "cuda"
    assert tr.checkpointer.load(0)
    got = _repeat_two_batches(tr, steps)
    tr.close()
    assert abs(got[0] - oracle[0]) < 0.02, (got[0], oracle[0])                     # same weights, same batch: forward only
    worst = max(abs(a - b) for a, b in zip(got, oracle))
    assert worst < 0.15, list(zip(got, oracle))
    assert oracle[0] - oracle[-1] > 0.5 and got[0] - got[-1] > 0.5, (oracle, got)   # both actually learn
    assert abs((got[0] - got[-1]) - (oracle[0] - oracle[-1])) < 0.15


def test_optimizer_update_under_the_next_forward_changes_nothing():
    """With `overlap_optimizer=True` the AdamW kernels run on their own stream in the order the next forward needs the
    units and the forward waits unit by unit. Same arithmetic, same order per element: the losses are identical, and
    after `sync_optimizer()` so are the parameters. (The attention backward runs in its bitwise-reproducible two-kernel
    mode here: the one-kernel mode sums dQ with reduce-adds whose order differs from run to run in the last bit.)"""
    from torchllmtuner_b200.ops import functional as F
    F.set_attention_backward("split")
    try:
        _overlap_case()
    finally:
        F.set_attention_backward(None)


def _overlap_case():
    cfg = _cfg(steps=5, num_hidden_layers=4)
    tr = Trainer(cfg)
    ref = [tr.train_step().loss for _ in range(5)]
    ref_master = [u.master.clone() for u in tr.asm.fsdp.units]
    tr.close()
    tr = Trainer(_cfg(steps=5, num_hidden_layers=4))
    got = [tr.train_step(overlap_optimizer=True).loss for _ in range(5)]
    assert any(getattr(u, "updated_event", None) is not None for u in tr.asm.fsdp.units)     # the last update is still pending or just done
    tr.asm.fsdp.sync_optimizer()
    assert all(getattr(u, "updated_event", None) is None for u in tr.asm.fsdp.units)
    torch.cuda.synchronize()
    try:
        assert got == ref, (got, ref)
        for a, u in zip(ref_master, tr.asm.fsdp.units):
            assert torch.equal(a, u.master)
    finally:
        tr.close()


def test_checkpoint_resume_is_bit_exact_on_the_gpu(tmp_path):
    """Saved from device shards as boxes of whole tensors (through pinned staging, asynchronously), resumed into a fresh
    trainer: the next steps repeat bit for bit. The save follows an overlapped optimizer update, so it must wait for it.
    (Bit for bit needs the reproducible two-kernel attention backward, see the test above.)"""
    from torchllmtuner_b200.ops import functional as F
    F.set_attention_backward("split")
    try:
        _resume_case(tmp_path)
    finally:
        F.set_attention_backward(None)


def _resume_case(tmp_path):
    import os
    import shutil
    kw = dict(dump_folder=str(tmp_path), enable=True, interval=2, steps=4, last_save_model_only=False, async_mode="async_with_pinned_mem",
              exclude_from_loading=[])
    tr = Trainer(_cfg(**kw))
    ref = []
    for _ in range(4):
        r = tr.train_step(overlap_optimizer=True)
        ref.append(r.loss)
        tr.checkpointer.save(r.step)
    tr.close()
    assert os.path.exists(os.path.join(str(tmp_path), "checkpoint", "step-2", ".metadata"))
    shutil.rmtree(os.path.join(str(tmp_path), "checkpoint", "step-4"))
    tr2 = Trainer(_cfg(**kw))
    assert tr2.checkpointer.load() and tr2.progress.step == 2
    got = [tr2.train_step().loss for _ in range(2)]
    tr2.close()
    assert got == ref[2:], (got, ref)


def test_vision_language_model_trains_on_the_gpu(tmp_path):
    """Tower (tcgen05 GEMMs, the non-causal attention kernel) + Qwen3.5 decoder under the Trainer on synthetic image-text rows."""
    cfg = LLMTunerConfig()
    cfg.apply_flat(dict(model_name_or_path="qwen3_5_vl", dataset="random_multimodal", vocab_size=2048, hidden_size=256, intermediate_size=512,
                        num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, global_batch_size=2, max_seq_len=512, steps=4, seed=0,
                        dump_folder=str(tmp_path), deterministic=False, learning_rate=2e-3, mm_max_pixels=14 * 14 * 4 * 16))
    cfg.model.arch_overrides = dict(head_dim=64, linear_key_head_dim=64, linear_value_head_dim=64,
                                    vision=dict(hidden_size=128, intermediate_size=256, depth=2, num_heads=2))
    tr = Trainer(cfg)
    try:
        losses = []
        for _ in range(4):
            tr.dataloader.cursor = 0
            losses.append(tr.train_step().loss)
    finally:
        tr.close()
    assert losses[-1] < losses[0] - 0.3, losses
