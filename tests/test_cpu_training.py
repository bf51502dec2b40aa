"""End-to-end CPU slice: tiny Qwen3 dense trains through the public Trainer API and the loss falls."""
import pytest
import torch

from torchllmtuner_b200 import LLMTunerConfig, Trainer


def tiny_config(**flat):
    cfg = LLMTunerConfig()
    base = dict(model_name_or_path="qwen3", vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, global_batch_size=4, max_seq_len=32, steps=8,
                learning_rate=3e-3, seed=0, dump_folder="/tmp/llmt_test_out")
    base.update(flat)
    cfg.apply_flat(base)
    return cfg


def run(cfg, repeat_batch=True):
    """Uniform random tokens carry no signal, so the tests replay the first global batch every step."""
    tr = Trainer(cfg)
    losses = []
    try:
        for _ in range(cfg.training.steps):
            if repeat_batch:
                tr.dataloader.cursor = 0
            losses.append(tr.train_step().loss)
    finally:
        tr.close()
    return losses


def test_dense_loss_decreases():
    losses = run(tiny_config())
    assert losses[-1] < losses[0] - 0.05, losses
    assert all(torch.isfinite(torch.tensor(losses)))


def test_full_ac_matches_no_ac():
    a = run(tiny_config(steps=3))
    b = run(tiny_config(steps=3, activation_checkpoint_mode="full"))
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5, (a, b)


def test_chunked_loss_matches_logits_loss():
    a = run(tiny_config(steps=3))
    b = run(tiny_config(steps=3, chunked_loss_num_chunks=3))
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-4, (a, b)


def test_grad_accumulation_matches_one_batch():
    a = run(tiny_config(steps=3))
    b = run(tiny_config(steps=3, gradient_accumulation_steps=2))
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-4, (a, b)


def test_moe_trains():
    cfg = tiny_config(model_name_or_path="qwen3_moe", steps=6)
    cfg.model.arch_overrides = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, router_bias_update_coeff=1e-3)
    losses = run(cfg)
    assert losses[-1] < losses[0], losses


def test_muon_trains():
    losses = run(tiny_config(steps=6, optimizer_type="DistMuon", learning_rate=2e-2))
    assert losses[-1] < losses[0], losses


def test_ema_and_wsd_schedule():
    from torchllmtuner_b200.components.optimizer import wsd_factor
    assert wsd_factor(0, warmup=4, total=20, decay_ratio=0.25) == 0.25
    assert wsd_factor(10, warmup=4, total=20, decay_ratio=0.25) == 1.0
    assert abs(wsd_factor(19, warmup=4, total=20, decay_ratio=0.25, decay_type="linear", min_lr_factor=0.1) - 0.1) < 0.2
    cfg = tiny_config(steps=3, warmup_steps=2)
    from torchllmtuner_b200.config import EMAConfig
    cfg.training.ema_config = EMAConfig(decay=0.5)
    tr = Trainer(cfg)
    before = [tr.ema.ema_params[u.name].clone() for u in tr.asm.fsdp.units]
    tr.train_step()
    assert any(not torch.equal(b, tr.ema.ema_params[u.name]) for b, u in zip(before, tr.asm.fsdp.units))
    assert tr.lr_schedulers.get_last_lr()[0] == cfg.optimizer.learning_rate      # warm-up finished after 2 steps
    tr.close()


@pytest.mark.parametrize("family", ["qwen3_5", "qwen3_5_moe", "kimi_linear", "kimi_k3", "deepseek_v4"])
def test_other_families_train(family):
    cfg = tiny_config(model_name_or_path=family, steps=4, max_seq_len=16, num_hidden_layers=4, hidden_size=64, num_attention_heads=2,
                      num_key_value_heads=2, learning_rate=5e-3)
    cfg.model.arch_overrides = dict(head_dim=64, qk_rope_dim=32, delta_heads=2, delta_head_dim=16)
    losses = run(cfg)
    assert losses[-1] < losses[0], (family, losses)


def test_registry_lists_every_family():
    from torchllmtuner_b200.models import registered_models
    have = set(registered_models())
    assert {"qwen3", "qwen3_moe", "qwen3_8b", "qwen3_30b_a3b", "qwen3_5", "qwen3_5_moe", "qwen3_5_moe_text", "deepseek_v4",
            "kimi_linear", "kimi_k3", "hybrid_kda_mla", "hybrid_gdn", "hybrid_gdn_moe"} <= have


def test_fsdp_cpu_offload_keeps_moments_on_the_host_and_trains():
    a = run(tiny_config(fsdp_cpu_offload=True, steps=3))
    b = run(tiny_config(steps=3))
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5


def test_moe_dispatch_timers_report_percentiles():
    cfg = tiny_config(model_name_or_path="qwen3_moe", measure_moe_dispatch=True, steps=2, log_freq=1)
    cfg.model.arch_overrides = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)
    tr = Trainer(cfg)
    try:
        tr.config.training.steps = 2
        tr.train()
        assert "moe/dispatch_p50(ms)" in tr.last_metrics and "moe/combine_p90(ms)" in tr.last_metrics, tr.last_metrics
    finally:
        tr.close()


def test_metric_names_and_profiler_trace_layout(tmp_path):
    """The logged step carries the reference's metric names; the profiler writes
    `<traces>/iteration_{step}/rank{rank}_trace.json.gz` on its schedule."""
    import glob
    import os
    cfg = tiny_config(steps=4, log_freq=1, dump_folder=str(tmp_path), enable_profiling=True, profile_freq=2, profiler_active=1,
                      profiler_warmup=1)
    tr = Trainer(cfg)
    try:
        tr.train()
        for k in ("loss_metrics/global_avg_loss", "loss_metrics/global_max_loss", "grad_norm", "lr", "throughput(tps)",
                  "tps_per_device", "tflops", "mfu(%)", "time_metrics/end_to_end(s)"):
            assert k in tr.last_metrics, (k, sorted(tr.last_metrics))
    finally:
        tr.close()
    traces = glob.glob(os.path.join(str(tmp_path), "**", "iteration_*", "rank0_trace.json*"), recursive=True)
    assert traces, list(os.walk(str(tmp_path)))[:5]


def test_cli_main_runs_a_tiny_job_and_seed_checkpoint(tmp_path, monkeypatch):
    """`python -m torchllmtuner_b200 <flat flags>` end to end, then the seed-checkpoint mode of the same CLI."""
    import os
    from torchllmtuner_b200.trainer.cli import main
    monkeypatch.setenv("LLMTUNER_DEVICE", "cpu")
    flags = ["--model_name_or_path", "qwen3", "--vocab_size", "256", "--hidden_size", "64", "--intermediate_size", "128",
             "--num_hidden_layers", "2", "--num_attention_heads", "4", "--num_key_value_heads", "2", "--global_batch_size", "2",
             "--max_seq_len", "32", "--steps", "3", "--enable", "true", "--interval", "2", "--last_save_model_only", "false"]
    assert main(flags + ["--dump_folder", str(tmp_path / "a")]) == 0
    assert os.path.exists(tmp_path / "a" / "checkpoint" / "step-2" / ".metadata")
    assert os.path.exists(tmp_path / "a" / "checkpoint" / "step-3" / ".metadata")          # the last step is always saved
    assert main(flags + ["--dump_folder", str(tmp_path / "b"), "--create_seed_checkpoint", "true"]) == 0
    assert os.path.exists(tmp_path / "b" / "checkpoint" / "step-0" / ".metadata")


def test_aux_loss_gradient_survives_full_activation_checkpointing():
    """The load-balance loss of MoE blocks must pull on the router under recomputation exactly as it does without it."""
    def cfg(ac):
        c = tiny_config(model_name_or_path="qwen3_moe", steps=4, activation_checkpoint_mode=ac, router_aux_loss_coef=0.5)
        c.model.arch_overrides = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, router_aux_loss_coef=0.5)
        return c
    a, b = run(cfg("none")), run(cfg("full"))
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5, (a, b)
    # and the aux term really matters for the trajectory (a coefficient of zero gives different losses after the first update)
    c0 = tiny_config(model_name_or_path="qwen3_moe", steps=4, activation_checkpoint_mode="full")
    c0.model.arch_overrides = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)
    z = run(c0)
    assert max(abs(x - y) for x, y in zip(b[1:], z[1:])) > 1e-6, (b, z)


def test_region_checkpointing_recomputes_exactly_the_named_blocks():
    """`region` mode: blocks whose name matches `recompute_regions` run their forward twice per step (once more in
    backward), the others once; the losses are those of the run without checkpointing."""
    cfg = tiny_config(steps=2, num_hidden_layers=4, activation_checkpoint_mode="region")
    cfg.training.region_ac.recompute_regions = [r"layers\.(1|3)$"]
    tr = Trainer(cfg)
    calls = {i: 0 for i in range(4)}
    layers = tr.model.model.layers
    for i in range(4):
        layer = layers[i] if not isinstance(layers, torch.nn.ModuleDict) else layers[str(i)]
        layer.register_forward_hook(lambda m, a_, o, i=i: calls.__setitem__(i, calls[i] + 1))
    a = []
    try:
        for _ in range(2):
            tr.dataloader.cursor = 0
            a.append(tr.train_step().loss)
    finally:
        tr.close()
    assert calls == {0: 2, 1: 4, 2: 2, 3: 4}, calls
    b = run(tiny_config(steps=2, num_hidden_layers=4))
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5


def test_tensorboard_sink_receives_logged_steps(tmp_path):
    import glob
    import os
    cfg = tiny_config(steps=2, log_freq=1, dump_folder=str(tmp_path), enable_tensorboard=True)
    tr = Trainer(cfg)
    try:
        tr.train()
    finally:
        tr.close()
    folder = os.path.join(str(tmp_path), cfg.training.metrics_config.save_tb_folder)
    files = glob.glob(os.path.join(folder, "events.out.tfevents.*")) + glob.glob(os.path.join(folder, "metrics.jsonl"))
    assert files and os.path.getsize(files[0]) > 0, os.listdir(str(tmp_path))


def test_validation_preserves_rng_and_training_mode_and_runs_on_schedule():
    from torchllmtuner_b200.config.training_config import ValidationConfig
    cfg = tiny_config(steps=4, log_freq=100)
    cfg.training.validation_config = ValidationConfig(freq=2, steps=2)
    tr = Trainer(cfg)
    try:
        state = torch.get_rng_state()
        v = tr.validate()
        assert torch.equal(state, torch.get_rng_state()) and tr.model.training
        assert 0.0 < v < 20.0
        tr.validator.history.clear()
        tr.train()
        assert [s for s, _ in tr.validator.history] == [1, 2, 4], tr.validator.history
    finally:
        tr.close()


def test_newton_schulz_pushes_singular_values_towards_one_and_lr_modes():
    from torchllmtuner_b200.components.optimizer.muon import adjusted_lr, newton_schulz
    torch.manual_seed(0)
    for shape in [(32, 64), (96, 48)]:
        g = torch.randn(*shape)
        x = newton_schulz(g, steps=5).float()
        sv = torch.linalg.svdvals(x)
        assert 0.5 < float(sv.min()) and float(sv.max()) < 1.3, (shape, sv.min(), sv.max())   # the quintic's band around 1
        # same singular vectors as the input: U^T X V is close to diagonal
        u, _, vt = torch.linalg.svd(g, full_matrices=False)
        d = u.t() @ x @ vt.t()
        assert float((d - torch.diag(torch.diagonal(d))).abs().max()) < 0.12
    assert adjusted_lr(1e-3, (128, 64), "original") == pytest.approx(1e-3 * 2 ** 0.5)
    assert adjusted_lr(1e-3, (64, 128), "original") == pytest.approx(1e-3)
    assert adjusted_lr(1e-3, (64, 256), "match_rms_adamw") == pytest.approx(1e-3 * 0.2 * 16)
    assert adjusted_lr(1e-3, (64, 256), "spectral_unclamped") == pytest.approx(1e-3 * 0.5)


def test_regex_param_groups_first_match_wins_and_overrides_apply():
    from torchllmtuner_b200.config.optimizer_config import ParamGroupConfig
    cfg = tiny_config(steps=1)
    cfg.optimizer.param_groups = [ParamGroupConfig(pattern=r"norm", optimizer_kwargs={"learning_rate": 0.0}),
                                  ParamGroupConfig(pattern=r"layers\.0\.", optimizer_kwargs={"weight_decay": 0.5}),
                                  ParamGroupConfig(pattern=r"q_proj", optimizer_kwargs={"learning_rate": 1.0})]
    tr = Trainer(cfg)
    try:
        opt = tr.optimizers.optimizers[0]
        groups = {g["name"]: g for g in opt.param_groups}
        assert set(groups) == {".*", "norm", r"layers\.0\.", "q_proj"}
        names = {g["name"]: set(g["param_names"]) for g in opt.param_groups}
        assert "model.layers.0.input_layernorm.weight" in names["norm"]                     # first match wins over layers.0.
        assert "model.layers.0.self_attn.q_proj.weight" in names[r"layers\.0\."]            # ... and over q_proj
        assert "model.layers.1.self_attn.q_proj.weight" in names["q_proj"]
        assert "model.embed_tokens.weight" in names[".*"]
        assert groups["norm"]["lr"] == 0.0 and groups[r"layers\.0\."]["weight_decay"] == 0.5
        before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
        tr.train_step()
        after = dict(tr.model.named_parameters())
        assert torch.equal(before["model.norm.weight"], after["model.norm.weight"])          # lr 0: frozen
        assert not torch.equal(before["model.layers.1.mlp.up_proj.weight"], after["model.layers.1.mlp.up_proj.weight"])
    finally:
        tr.close()


def test_accumulation_with_unequal_valid_tokens_equals_one_batch():
    """Micro-batches with different numbers of valid targets: the loss is the sum of token losses over the whole step
    divided by the step's valid-token count, so two micro-batches must give the gradients of the joint batch."""
    one = Trainer(tiny_config(steps=1, global_batch_size=4))
    two = Trainer(tiny_config(steps=1, global_batch_size=4, gradient_accumulation_steps=2))
    try:
        big = one.fetch_batch()
        big["labels"] = big["labels"].clone()
        big["labels"][0, 5:] = -100                      # row 0 keeps 5 targets, rows 1-3 keep all
        big["labels"][3, :20] = -100
        big["num_valid_tokens"] = int((big["labels"] != -100).sum())
        halves = []
        for a in (0, 2):
            h = {k: (v[a:a + 2].clone() if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == 4 else v) for k, v in big.items()}
            h["num_valid_tokens"] = int((h["labels"] != -100).sum())
            halves.append(h)
        assert halves[0]["num_valid_tokens"] != halves[1]["num_valid_tokens"]
        r1 = one.train_step(batches=[big])
        r2 = two.train_step(batches=halves)
        assert abs(r1.loss - r2.loss) < 1e-5 and abs(r1.grad_norm - r2.grad_norm) < 1e-4, (r1, r2)
        # Adam's first update is lr * sign-like in every element, so elements whose gradient is ~0 may flip on rounding:
        # compare in bulk
        for (n, p), (_, q) in zip(one.model.named_parameters(), two.model.named_parameters()):
            assert float(((p - q).abs() > 1e-5).float().mean()) < 1e-3, n
    finally:
        one.close()
        two.close()


def test_kernel_status_code_rides_in_the_step_read_and_stops_the_step(monkeypatch):
    """The status word of the device kernels is read with the step's loss; a non-zero code raises at that step."""
    from torchllmtuner_b200.errors import KernelStatusError
    from torchllmtuner_b200.trainer import trainer as trainer_mod
    from torchllmtuner_b200.trainer.runtime.metrics import build_step_metrics

    class Red:
        loss_group = None
    out = build_step_metrics(torch.tensor(6.0), torch.tensor(2.0), torch.tensor(3.0), Red(), torch.tensor([2, 7, 1, 0], dtype=torch.int32))
    assert out == (2.0, 2.0, 3.0, 2)
    assert build_step_metrics(torch.tensor(6.0), torch.tensor(2.0), torch.tensor(3.0), Red()) == (2.0, 2.0, 3.0)

    word = torch.zeros(8, dtype=torch.int32)
    monkeypatch.setattr(trainer_mod, "status_word", lambda device: word)

    def fake_check(where):
        raise KernelStatusError(where, int(word[0]), "bounded flag wait expired at site 7")
    monkeypatch.setattr(trainer_mod, "check_status", fake_check)
    tr = Trainer(tiny_config(steps=3))
    try:
        assert tr.train_step().step == 1                              # code 0: nothing happens
        word[0] = 2
        with pytest.raises(KernelStatusError, match="training step 2"):
            tr.train_step()
    finally:
        tr.close()


def test_per_op_selective_checkpointing_matches_no_checkpointing():
    """selective / policy "op": attention and every other linear keep their outputs, the rest is replayed. The curve is the
    one without checkpointing, the frame keeps strictly less than a whole block, and a forced-recompute weight shape changes
    what is kept without changing the result."""
    from torchllmtuner_b200.ops import functional as F
    kept = []
    orig = F.SelectiveReplay.put

    def spy(self, value):
        orig(self, value)
        kept.append(self.kept_bytes)
    F.SelectiveReplay.put = spy
    try:
        base = run(tiny_config(steps=3, activation_checkpoint_mode="none"))
        sel = run(tiny_config(steps=3, activation_checkpoint_mode="selective"))
        n_default = len(kept)
        forced = run(tiny_config(steps=3, activation_checkpoint_mode="selective", force_recompute_mm_shapes_by_fqns=["mlp.gate_proj"]))
        n_forced = len(kept) - n_default
        blk = run(tiny_config(steps=3, activation_checkpoint_mode="selective", selective_ac_policy="block"))
    finally:
        F.SelectiveReplay.put = orig
    for other in (sel, forced, blk):
        assert max(abs(a - b) for a, b in zip(base, other)) < 1e-5, (base, other)
    assert n_default > 0 and 0 < n_forced < n_default          # gate/up share a shape: both leave the kept set
    with pytest.raises(ValueError):
        run(tiny_config(steps=1, activation_checkpoint_mode="selective", force_recompute_mm_shapes_by_fqns=["no_such_module"]))


def test_ema_firing_count_decay_and_buffer_tracking(tmp_path):
    """Firing n = (step - start_step) / every + step_bias, derived from the step; decay 2^(-1 / (hl * n)); a MoE block's
    selection bias is averaged when `buffer_patterns` names it, travels in the checkpoint, and a replaced buffer is an
    error rather than a frozen average."""
    from torchllmtuner_b200.config.training_config import EMAConfig
    cfg = tiny_config(model_name_or_path="qwen3_moe", steps=8, dump_folder=str(tmp_path), enable=True, interval=100)
    cfg.model.arch_overrides = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, router_bias_update_coeff=1e-2)
    cfg.training.ema_config = EMAConfig(half_life_fraction=0.5, start_step=1, update_every_n_steps=2, step_bias=3, buffer_patterns=[r"expert_bias_E$"])
    tr = Trainer(cfg)
    ema = tr.ema
    assert [ema.firing(s) for s in range(7)] == [0, 0, 0, 4, 0, 5, 0]
    assert abs(ema.decay_at(4) - 2.0 ** (-1.0 / (0.5 * 4))) < 1e-12
    assert sorted(ema.ema_buffers) == ["model.layers.0.mlp.expert_bias_E", "model.layers.1.mlp.expert_bias_E"]
    for _ in range(3):
        tr.train_step()
    name = "model.layers.0.mlp.expert_bias_E"
    live = dict(tr.model.named_buffers())[name]
    assert live.abs().sum() > 0 and ema.ema_buffers[name].abs().sum() > 0 and not torch.equal(ema.ema_buffers[name], live)
    tr.checkpointer.save(3, force=True)
    tr.checkpointer.wait()
    kept = ema.ema_buffers[name].clone()
    ema.ema_buffers[name].zero_()
    assert tr.checkpointer.load(3)
    assert torch.equal(ema.ema_buffers[name], kept)
    blk = tr.model.model.layers[0].mlp
    blk.register_buffer("expert_bias_E", blk.expert_bias_E.clone())
    with pytest.raises(RuntimeError, match="identity"):
        ema.step(5)
    tr.close()
