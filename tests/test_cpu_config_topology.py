"""Config surface, topology arithmetic for every rank of 8 (no process group needed), closed-form helpers."""
import json
import math

import pytest
import torch

from torchllmtuner_b200 import LLMTunerConfig
from torchllmtuner_b200.config import build_parser
from torchllmtuner_b200.errors import ConfigError, LLMTunerError, UnsupportedCombinationError
from torchllmtuner_b200.parallel.topology import ParallelTopology, resolve_parallel_topology
from torchllmtuner_b200.trainer.cli import parse_config


# ------------------------------------------------------------------------------------------------ CLI / config
def test_flat_flags_cover_the_thirteen_groups_without_collisions():
    p = build_parser()
    flags = {a.dest for a in p._actions}
    for name in ("model_name_or_path", "data_parallel_shard_size", "tensor_parallel_size", "expert_parallel_size",
                 "context_parallel_ulysses_size", "context_parallel_kv_allgather_size", "fsdp_reshard_after_forward",
                 "enable_sequence_parallel", "context_parallel_load_balancer", "ep_token_dispatcher", "optimizer_type",
                 "learning_rate", "warmup_steps", "global_batch_size", "max_seq_len", "activation_checkpoint_mode", "interval",
                 "dataset", "log_freq", "enable_profiling"):
        assert name in flags, name


def test_cli_overrides_file_and_round_trips(tmp_path):
    f = tmp_path / "run.yaml"
    f.write_text("model_name_or_path: qwen3\nmax_seq_len: 128\nglobal_batch_size: 4\nlearning_rate: 1.0e-3\n")
    cfg = parse_config(["--config", str(f), "--max_seq_len", "256"])
    assert cfg.training.max_seq_len == 256 and cfg.training.global_batch_size == 4
    assert cfg.optimizer.learning_rate == pytest.approx(1e-3)
    j = tmp_path / "run.json"
    j.write_text(json.dumps({"model_name_or_path": "qwen3", "steps": 7}))
    assert parse_config(["--config", str(j)]).training.steps == 7


@pytest.mark.parametrize("flat,err", [
    (dict(ep_token_dispatcher="deepep"), ConfigError),
    (dict(ep_token_dispatcher="nonsense"), ConfigError),
    (dict(context_parallel_load_balancer="ptrr"), (ConfigError, UnsupportedCombinationError)),
    (dict(global_batch_size=0), ConfigError),
    (dict(interval=0), ConfigError),
    (dict(qkv_projection="fused", tensor_parallel_size=2), (ConfigError, UnsupportedCombinationError)),
])
def test_invalid_values_and_combinations_raise_the_framework_classes(flat, err):
    with pytest.raises(err) as e:
        cfg = LLMTunerConfig()
        cfg.apply_flat(flat)
        cfg.__post_init__()
    assert isinstance(e.value, LLMTunerError)


# ------------------------------------------------------------------------------------------------ topology
def _cfg(**flat):
    cfg = LLMTunerConfig()
    cfg.apply_flat(flat)
    return cfg.parallel


def test_world_size_formula_and_derived_shard():
    t = resolve_parallel_topology(_cfg(tensor_parallel_size=2, data_parallel_shard_size=-1), 8, 0)
    assert (t.dp_shard, t.tp, t.world_size) == (4, 2, 8)
    with pytest.raises(ConfigError):
        resolve_parallel_topology(_cfg(tensor_parallel_size=3), 8, 0)
    with pytest.raises(ConfigError):
        resolve_parallel_topology(_cfg(data_parallel_shard_size=2, expert_parallel_size=4), 2, 0)   # (dp_shard*cp*tp) % ep


def test_mesh_order_tp_innermost_for_every_rank_of_eight():
    for rank in range(8):
        t = resolve_parallel_topology(_cfg(data_parallel_replicate_size=2, data_parallel_shard_size=2, tensor_parallel_size=2), 8, rank)
        c = t.coords(rank)
        assert rank == (c["dp_replicate"] * 2 + c["dp_shard"]) * 2 + c["tp"]
        assert t.group_ranks("tp", rank) == [rank - rank % 2, rank - rank % 2 + 1]          # TP ranks are adjacent
        assert t.group_ranks("dp_shard", rank) == sorted({rank, rank ^ 2})
        assert t.group_ranks("dp_replicate", rank) == sorted({rank, rank ^ 4})


def test_sparse_view_ep_is_innermost_and_efsdp_is_the_rest():
    for rank in range(8):
        t = resolve_parallel_topology(_cfg(data_parallel_shard_size=8, expert_parallel_size=4), 8, rank)
        assert t.efsdp == 2
        assert t.group_ranks("ep", rank) == list(range(rank // 4 * 4, rank // 4 * 4 + 4))
        assert t.group_ranks("efsdp", rank) == sorted({rank % 4, rank % 4 + 4})


def test_groups_partition_the_world():
    t = resolve_parallel_topology(_cfg(data_parallel_shard_size=2, context_parallel_ulysses_size=2, tensor_parallel_size=2), 8, 0)
    for name in ("tp", "cp", "dp_shard"):
        groups = t.all_groups(name)
        assert sorted(r for g in groups for r in g) == list(range(8)), name


# ------------------------------------------------------------------------------------------------ closed forms
def test_stage_order_and_vocab_shards():
    from torchllmtuner_b200.parallel.stages import STAGE_ORDER
    from torchllmtuner_b200.utils.vocabulary import vocab_shard_bounds
    assert list(STAGE_ORDER) == ["tp", "ep", "cp", "ac", "activation_swap", "compile", "fsdp"]
    V, R = 151936, 8
    cuts = [vocab_shard_bounds(V, R, r) for r in range(R)]
    assert cuts[0][0] == 0 and cuts[-1][1] == V and all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
    assert cuts[0][1] - cuts[0][0] == math.ceil(V / R) == 18992
    assert vocab_shard_bounds(10, 4, 3) == (9, 10) and vocab_shard_bounds(5, 8, 7) == (5, 5)


def test_flops_per_token_match_the_published_evaluations():
    from torchllmtuner_b200.models.qwen3 import QWEN3_8B, QWEN3_30B_A3B, Qwen3Config
    assert Qwen3Config(**QWEN3_8B).flops_per_token(8192) / 1e9 == pytest.approx(59.9, abs=0.1)
    assert Qwen3Config(**QWEN3_8B).flops_per_token(131072) / 1e9 == pytest.approx(277.3, abs=0.2)
    assert Qwen3Config(**QWEN3_30B_A3B).flops_per_token(4096) / 1e9 == pytest.approx(27.9, abs=0.1)


def test_wsd_schedule_formula():
    from torchllmtuner_b200.components.optimizer.lr_scheduler import wsd_factor
    total, warm, ratio = 100, 10, 0.2
    decay = int(total * ratio)
    stable = total + 1 - warm - decay
    kw = dict(warmup=warm, total=total, decay_ratio=ratio)
    assert wsd_factor(0, decay_type="linear", **kw) == pytest.approx(1 / warm)
    assert wsd_factor(warm - 1, decay_type="linear", **kw) == pytest.approx(1.0)
    assert wsd_factor(50, decay_type="cosine", min_lr_factor=0.1, **kw) == pytest.approx(1.0)
    step = warm + stable + 4
    p = (step + 1 - warm - stable) / decay
    assert wsd_factor(step, decay_type="linear", **kw) == pytest.approx(1 - p)
    assert wsd_factor(step, decay_type="sqrt", **kw) == pytest.approx(1 - math.sqrt(p))
    assert wsd_factor(step, decay_type="cosine", min_lr_factor=0.2, **kw) == pytest.approx(0.2 + 0.8 * 0.5 * (1 + math.cos(math.pi * p)))


def test_seed_derivation_is_distinct_and_stable():
    from torchllmtuner_b200.utils.seeding import derive_distinct_seed
    seeds = {derive_distinct_seed(42, r) for r in range(64)}
    assert len(seeds) == 64 and derive_distinct_seed(42, 3) == derive_distinct_seed(42, 3)


def test_aux_loss_free_bias_update_rule():
    from torchllmtuner_b200.models.moe.layer import MoE
    moe = MoE(32, 4, 2, 16, bias_update_coeff=1e-3, dtype=torch.float32)
    moe.tokens_per_expert_E.copy_(torch.tensor([10.0, 0.0, 5.0, 5.0]))
    moe.update_expert_bias()
    delta = 1e-3 * torch.sign(torch.tensor([5.0 - 10, 5.0 - 0, 0.0, 0.0]))
    assert torch.allclose(moe.expert_bias_E, delta - delta.mean(), atol=1e-7)
    assert float(moe.tokens_per_expert_E.sum()) == 0.0


def test_spmd_context_nesting_and_replay_snapshot():
    from torchllmtuner_b200.accelerator import spmd
    dense = resolve_parallel_topology(_cfg(tensor_parallel_size=2, data_parallel_shard_size=4), 8, 3)
    sparse = resolve_parallel_topology(_cfg(data_parallel_shard_size=8, expert_parallel_size=4), 8, 3)
    spmd.set_spmd_meshes(dense, sparse)
    assert spmd.current_spmd_mesh() is dense and spmd.spmd_mesh_size("tp") == 2
    with spmd.spmd_context(sparse):
        assert spmd.current_spmd_mesh() is sparse and spmd.spmd_mesh_size("ep") == 4
        snap = spmd.capture_spmd_context()
    assert spmd.current_spmd_mesh() is dense
    with spmd.restore_spmd_context(snap):
        assert spmd.current_spmd_mesh() is sparse
    assert spmd.current_spmd_mesh() is dense


def test_kernel_argument_contracts_raise_config_errors():
    from torchllmtuner_b200.ops import validation as v
    q, k = torch.zeros(8, 4, 64), torch.zeros(8, 3, 64)
    with pytest.raises(ConfigError):
        v.validate_attention_inputs(q, k, k)
    v.validate_attention_inputs(q, torch.zeros(8, 2, 64), torch.zeros(8, 2, 64))
    with pytest.raises(ConfigError):
        v.validate_rms_norm_inputs(torch.zeros(4, 16), torch.zeros(8))
    with pytest.raises(ConfigError):
        v.require_last_dim_contiguous(torch.zeros(8, 16).t(), "x")
    with pytest.raises(ConfigError):
        v.validate_router_inputs(torch.zeros(4, 8), 9)


def test_runtime_validator_reports_a_working_cpu_path(monkeypatch):
    monkeypatch.setenv("LLMTUNER_DEVICE", "cpu")
    from torchllmtuner_b200.utils.validate_runtime import collect
    rep = collect()
    assert "train_step_loss" in rep and rep["distributed"]["gloo"] and "extension" in rep


def test_compatibility_matrix_entries_reject_before_any_mutation():
    from types import SimpleNamespace as NS

    from torchllmtuner_b200.parallel.compatibility import ENTRIES, check_compatibility
    cfg = LLMTunerConfig()

    def topo(**kw):
        d = dict(tp=1, ep=1, cp_ulysses=1, cp_kv=1, kcp=1, pp=1)
        d.update(kw)
        return NS(**d)
    dense = NS(num_experts=0, num_attention_heads=8, num_key_value_heads=2, model_type="qwen3", tie_word_embeddings=False)
    moe = NS(num_experts=6, num_attention_heads=8, num_key_value_heads=4, model_type="qwen3_moe", tie_word_embeddings=False,
             shared_expert_intermediate_size=0)
    check_compatibility(cfg, topo(), dense)                                   # the plain case passes
    cases = {"ep_without_experts": (topo(ep=2), dense), "ep_divides_experts": (topo(ep=4), moe),
             "tp_divides_heads": (topo(tp=4), dense), "ulysses_divides_heads": (topo(cp_ulysses=4), dense),
             "kcp_needs_delta_attention": (topo(kcp=2), dense)}
    for name, (t, m) in cases.items():
        with pytest.raises(UnsupportedCombinationError) as e:
            check_compatibility(cfg, t, m)
        assert f"[{name}]" in str(e.value), (name, str(e.value))
    assert {n for n, _, _ in ENTRIES} >= set(cases)


def test_inert_flags_are_reported_and_every_other_flag_is_read_somewhere():
    """A flag is either read by the package or listed as inert with a reason; nothing is silently ignored."""
    import dataclasses
    import os
    import re

    import torchllmtuner_b200.config.training_config as tc
    from torchllmtuner_b200.config.cli_config import PARSER_GROUPS
    from torchllmtuner_b200.config.inert_fields import INERT_FIELDS, UNSUPPORTED_FIELDS, check_unsupported_fields, inert_fields_set
    from torchllmtuner_b200.errors import UnsupportedCombinationError
    cfg = LLMTunerConfig()
    assert inert_fields_set(cfg) == []
    check_unsupported_fields(cfg)
    for flat in (dict(grad_norm_precision="parameter"), dict(fsdp_expert_reduce_layout="split")):
        bad = LLMTunerConfig()
        bad.apply_flat(flat)
        with pytest.raises(UnsupportedCombinationError):          # semantics-changing flags raise instead of being ignored
            check_unsupported_fields(bad)
    cfg.apply_flat(dict(norm_backend="other", sharded_expert_parallel=True))
    assert {n for n, _ in inert_fields_set(cfg)} == {"norm_backend", "sharded_expert_parallel"}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = ""
    for d, _, files in os.walk(os.path.join(root, "torchllmtuner_b200")):
        if "__pycache__" in d:
            continue
        for f in files:
            if f.endswith(".py") and f != "inert_fields.py" and not (d.endswith("config") and f.endswith("_config.py") and f != "llmtuner_config.py"):
                src += open(os.path.join(d, f)).read()
    groups = list(PARSER_GROUPS) + [o for o in vars(tc).values() if dataclasses.is_dataclass(o) and isinstance(o, type)]
    silent = [f"{g.__name__}.{f.name}" for g in dict.fromkeys(groups) for f in dataclasses.fields(g)
              if f.name not in INERT_FIELDS and f.name not in UNSUPPORTED_FIELDS and not re.search(r"\b" + re.escape(f.name) + r"\b", src)]
    assert silent == [], silent


def _wsd_statement(step, warmup, total, ratio, kind, floor):
    """The schedule written out independently: phase lengths, then the factor of a 0-indexed step."""
    warmup = min(warmup, total)
    decay = min(round(total * ratio), total - warmup)
    stable = total + 1 - warmup - decay
    if step < warmup:
        return (step + 1) / warmup
    if step < warmup + stable:
        return 1.0
    p = (step + 1 - warmup - stable) / decay
    shape = {"linear": 1 - p, "sqrt": 1 - math.sqrt(p), "cosine": 0.5 * (1 + math.cos(math.pi * p))}[kind]
    return floor + (1 - floor) * shape


@pytest.mark.parametrize("kind", ["linear", "sqrt", "cosine"])
@pytest.mark.parametrize("floor", [0.0, 0.1])
@pytest.mark.parametrize("total,warmup,ratio", [(100, 10, 0.29), (100, 0, 0.0), (20, 4, 0.25), (10, 30, 0.5), (50, 30, 0.8), (7, 3, 0.5)])
def test_wsd_schedule_every_step(kind, floor, total, warmup, ratio):
    from torchllmtuner_b200.components.optimizer.lr_scheduler import resolve_phases, wsd_factor
    w, s, d = resolve_phases(total, warmup, ratio)
    assert w + s + d == total + 1 and w >= 0 and s >= 1 and d >= 0       # phases never overlap, stable never negative
    for step in range(total):
        got = wsd_factor(step, warmup=warmup, total=total, decay_ratio=ratio, decay_type=kind, min_lr_factor=floor)
        assert got == pytest.approx(_wsd_statement(step, warmup, total, ratio, kind, floor), abs=1e-12), step
        assert got >= min(floor, 1.0 / max(1, w)) - 1e-12
    if warmup > 0:   # warm-up is not blended with the floor
        assert wsd_factor(0, warmup=warmup, total=total, decay_ratio=ratio, decay_type=kind, min_lr_factor=floor) == pytest.approx(1 / min(warmup, total))
    assert round(100 * 0.29) == 29 and resolve_phases(100, 10, 0.29)[2] == 29   # rounded, not truncated


def test_module_pattern_grammar():
    from torchllmtuner_b200.parallel.module_patterns import compile_module_pattern, module_name_matches, resolve_module_patterns
    names = [f"model.layers.{i}.{m}" for i in range(12) for m in ("mlp", "mlp.gate_proj", "self_attn")] + ["model.norm", "lm_head"]
    assert resolve_module_patterns(names, ["model.layers.{0-3}.mlp"]) == {f"model.layers.{i}.mlp" for i in range(4)}
    assert resolve_module_patterns(names, ["model.layers.{*}.self_attn"]) == {f"model.layers.{i}.self_attn" for i in range(12)}
    assert module_name_matches("model.layers.10.mlp.gate_proj", "model.layers.1?.mlp.*")
    assert not module_name_matches("model.layers.1.mlp", "model.layers.{10-11}.mlp")       # a range is a number, not a prefix
    assert not module_name_matches("model.layers.x.mlp", "model.layers.{*}.mlp")
    assert module_name_matches("lm_head", "lm_head") and not module_name_matches("lm_head2", "lm_head")    # whole-name match
    with pytest.raises(ValueError):
        resolve_module_patterns(names, ["model.layer.{0-3}.mlp"], "test")                  # a typo selects nothing: refused
    for bad in ("a.{3-1}", "a.{x}", "a.{1-", "a.}"):
        with pytest.raises(ValueError):
            compile_module_pattern(bad)
