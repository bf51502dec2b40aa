"""Resolve-then-execute plans, the execution layout and the model execution contracts."""
import pytest
import torch
import torch.nn as nn

from torchllmtuner_b200 import LLMTunerConfig
from torchllmtuner_b200.errors import ConfigError, UnsupportedCombinationError
from torchllmtuner_b200.parallel.plan import ParallelPlan, PlanTarget, StalePlanError


class _Topo:
    def __init__(self, **kw):
        self.tp = self.ep = self.cp = self.cp_kv = self.cp_ulysses = self.kcp = 1
        self.__dict__.update(kw)


def _model(**arch):
    from torchllmtuner_b200.models.registry import build_registered_model
    cfg = LLMTunerConfig()
    cfg.apply_flat(dict(model_name_or_path="qwen3_moe" if arch else "qwen3", vocab_size=128, hidden_size=64, intermediate_size=128,
                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2))
    if arch:
        cfg.model.arch_overrides = arch
    return build_registered_model(cfg.model, dtype=torch.float32, device=None), cfg


def test_tp_plan_names_every_projection_and_rejects_bad_degrees():
    from torchllmtuner_b200.parallel.tensor_parallel import build_tp_plan
    model, cfg = _model()
    plan = build_tp_plan(model, _Topo(tp=2), cfg.parallel.tp_config)
    assert plan.stage == "tp" and plan.degree == 2
    assert plan.count("dense") == 2 * 7 and plan.count("attention") == 2 and plan.count("vocab") == 1 and plan.count("head") == 1
    assert {t.layout for t in plan.targets if t.path.endswith("o_proj") or t.path.endswith("down_proj")} == {"rowwise"}
    assert [t.layout for t in plan.targets if t.kind == "head"] == ["vocab"]
    plan.validate_binding(model)                                        # nothing changed: passes
    with pytest.raises(UnsupportedCombinationError):                    # 4 query heads / 2 kv heads: tp=4 does not divide the kv heads
        build_tp_plan(model, _Topo(tp=4), cfg.parallel.tp_config)


def test_a_plan_goes_stale_when_the_model_changes_under_it():
    from torchllmtuner_b200.parallel.tensor_parallel import build_tp_plan
    model, cfg = _model()
    fresh = lambda: build_tp_plan(model, _Topo(tp=2), cfg.parallel.tp_config)      # noqa: E731
    plan = fresh()
    blk = model.model.layers[0]
    old = blk.self_attn.q_proj.weight
    blk.self_attn.q_proj.weight = nn.Parameter(old.detach().clone())    # same geometry, different object
    with pytest.raises(StalePlanError, match="replaced"):
        plan.validate_binding(model)
    blk.self_attn.q_proj.weight = old
    plan.validate_binding(model)
    plan = fresh()
    blk.mlp.down_proj.forward = lambda x: x                            # somebody patched a forward
    with pytest.raises(StalePlanError, match="re-bound"):
        plan.validate_binding(model)
    del blk.mlp.down_proj.forward
    plan = fresh()
    keep = blk.mlp.gate_proj
    blk.mlp.gate_proj = type(keep)(64, 128, torch.float32, None)       # a module swapped out
    with pytest.raises(StalePlanError, match="no longer part"):
        plan.validate_binding(model)
    blk.mlp.gate_proj = keep
    plan = fresh()
    model.model.embed_tokens.register_buffer("scratch", torch.zeros(1), persistent=False)
    with pytest.raises(StalePlanError, match="buffers"):
        plan.validate_binding(model)


def test_ep_plan_binds_blocks_only_and_is_resolved_before_any_mutation():
    from torchllmtuner_b200.parallel.expert_parallel import build_ep_plan
    model, cfg = _model(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)
    plan = build_ep_plan(model, _Topo(ep=2), cfg.parallel.ep_config)
    assert plan.count("moe") == 2 and plan.binds == ("modules",)
    ex = model.model.layers[0].mlp.routed.experts
    ex.w1_EFD = nn.Parameter(ex.w1_EFD.detach()[:, :16].clone())        # what tensor parallelism does to the experts first
    plan.validate_binding(model)                                        # still valid: the block objects are the same
    with pytest.raises(ConfigError):
        build_ep_plan(model, _Topo(ep=3), cfg.parallel.ep_config)       # 3 does not divide 4 experts
    dense, dcfg = _model()
    with pytest.raises(ConfigError):
        build_ep_plan(dense, _Topo(ep=2), dcfg.parallel.ep_config)


def test_plan_and_target_reject_malformed_input():
    with pytest.raises(ValueError):
        PlanTarget("model..layers", "dense")
    with pytest.raises(ValueError):
        PlanTarget("model.layers.0", "pattern")
    with pytest.raises(ValueError):
        ParallelPlan("tp", 0, "x", ())
    with pytest.raises(ValueError):
        ParallelPlan("", 1, "x", ())
    with pytest.raises(ValueError):
        ParallelPlan("tp", 1, "x", (PlanTarget("a", "dense"), PlanTarget("a", "dense")))
    p = ParallelPlan("tp", 2, "peer-memory", (PlanTarget("a", "dense", "colwise"), PlanTarget("b", "moe")))
    assert p.describe()["targets"] == {"dense": 1, "moe": 1} and p.paths("moe") == ["b"]


def test_execution_layout_follows_topology_and_plans():
    from torchllmtuner_b200.parallel.execution import ExecutionLayout, resolve_execution_layout
    from torchllmtuner_b200.parallel.tensor_parallel import build_tp_plan
    model, cfg = _model()
    cfg.apply_flat(dict(max_seq_len=64))
    lay = resolve_execution_layout(cfg, _Topo(), model, {})
    assert lay.output_kind == "logits" and lay.sequence_shards == 1 and not lay.vocabulary_sharded
    cfg.apply_flat(dict(chunked_loss_num_chunks=4))
    assert resolve_execution_layout(cfg, _Topo(), model, {}).loss_chunks == 4
    cfg.apply_flat(dict(chunked_loss_num_chunks=0))
    plans = {"tp": build_tp_plan(model, _Topo(tp=2), cfg.parallel.tp_config)}
    lay = resolve_execution_layout(cfg, _Topo(tp=2, cp=2, cp_kv=2), model, plans)
    assert lay.vocabulary_sharded and lay.output_kind == "hidden" and lay.sequence_shard_axes == ("cp", "tp")
    assert lay.tokens_per_rank(64) == 16
    with pytest.raises(ConfigError):
        lay.tokens_per_rank(66)
    cfg.apply_flat(dict(max_seq_len=68, context_parallel_load_balancer="headtail"))
    with pytest.raises(ConfigError):                                    # head-tail needs a multiple of 2 * cp * tp
        resolve_execution_layout(cfg, _Topo(tp=2, cp=2, cp_kv=2), model, plans)
    with pytest.raises(UnsupportedCombinationError):
        ExecutionLayout("logits", ("tp",), 2, True, 0)


def test_model_execution_contracts():
    from torchllmtuner_b200.models.execution import (ModelExecutionCapabilities, capabilities_of, validate_prepared_model_inputs,
                                                     validate_training_output)
    model, _ = _model()
    caps = capabilities_of(model)
    assert caps.hidden_states and caps.logits and caps.width("hidden") == 64 and caps.width("logits") == 128
    ok = dict(tokens=torch.zeros(8, dtype=torch.long), targets=torch.zeros(8, dtype=torch.long), positions=torch.arange(8), attn_meta=None)
    assert validate_prepared_model_inputs(ok) is ok
    for bad in (dict(ok, targets=torch.zeros(7, dtype=torch.long)), dict(ok, tokens=torch.zeros(8)), {k: v for k, v in ok.items() if k != "positions"}):
        with pytest.raises((ValueError, TypeError, KeyError)):
            validate_prepared_model_inputs(bad)
    with pytest.raises(TypeError):
        validate_prepared_model_inputs((1, 2, 3))
    validate_training_output(torch.zeros(8, 64), ok["targets"], output_width=64)
    validate_training_output(torch.zeros(2, 4, 64), torch.zeros(2, 4, dtype=torch.long))
    for out, tgt, kw in ((torch.zeros(7, 64), ok["targets"], {}), (torch.zeros(8, 64), ok["targets"], dict(output_width=32)),
                         (torch.zeros(8, 64, dtype=torch.long), ok["targets"], {}), (torch.zeros(4, 2, 64), torch.zeros(2, 4, dtype=torch.long), {})):
        with pytest.raises((ValueError, TypeError)):
            validate_training_output(out, tgt, **kw)
    with pytest.raises(ValueError):
        ModelExecutionCapabilities(True, False, 64)
    with pytest.raises(ValueError):
        ModelExecutionCapabilities(True, False).require("hidden")


# ------------------------------------------------------------------------------------------ model part layout
def _tied():
    import torch.nn as nn

    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(8, 4)
            self.body = nn.Sequential(nn.Linear(4, 4, bias=False))
            self.head = nn.Linear(4, 8, bias=False)
            self.head.weight = self.embed.weight
    return Tied()


def test_layout_names_aliases_and_owner():
    from torchllmtuner_b200.parallel.assembly import ModelPartLayout
    m = _tied()
    lay = ModelPartLayout()
    lay.refresh(m)
    assert list(lay.bindings) == ["embed.weight", "body.0.weight", "head.weight"]
    assert lay.aliases[m.embed.weight] == ("embed.weight", "head.weight")
    assert lay.owner_names[m.embed.weight] == "embed.weight"          # first registration names the state
    assert lay.validate(m)["head.weight"] == "head.weight"


def test_layout_refresh_accepts_materialisation_and_rejects_split_alias():
    import torch
    import torch.nn as nn
    from torchllmtuner_b200.parallel.assembly import LayoutError, ModelPartLayout
    m = _tied()
    lay = ModelPartLayout()
    lay.refresh(m)
    snap = lay.snapshot()
    # a whole-model materialisation swaps every object and keeps the sharing
    new = nn.Parameter(torch.zeros(8, 4))
    old = m.embed.weight
    m.embed.weight = new
    m.head.weight = new
    lay.refresh(m)
    assert lay.replaced[id(old)] is new and lay.validate(m)
    with pytest.raises(LayoutError, match="ownership changed"):
        snap.validate(lay, consumer="optimizer")
    # replacing one path of a shared parameter splits the alias
    m.head.weight = nn.Parameter(torch.zeros(8, 4))
    with pytest.raises(LayoutError, match="split"):
        lay.refresh(m)


def test_layout_rejects_wrapper_name_collision_and_stale_model():
    import torch.nn as nn
    from torchllmtuner_b200.parallel.assembly import LayoutError, ModelPartLayout, validate_layouts, capture_layouts

    class Wrap(nn.Module):
        def __init__(self):
            super().__init__()
            self.inner = nn.Linear(2, 2, bias=False)
            self.weight = nn.Parameter(self.inner.weight.detach().clone())      # collapses onto inner.weight -> "weight"
    lay = ModelPartLayout()
    lay.refresh(Wrap())
    with pytest.raises(LayoutError, match="collapse"):
        lay.state_names
    m = _tied()
    lay = ModelPartLayout()
    lay.refresh(m)
    m.extra = nn.Linear(2, 2)
    with pytest.raises(LayoutError, match="stale"):
        lay.validate(m)
    a, b = _tied(), _tied()
    with pytest.raises(LayoutError, match="claimed by model parts"):
        validate_layouts([a, b], capture_layouts([a, b]))


def test_trainer_layout_binds_optimizer_and_checkpointer(tmp_path):
    import torch
    from dist_cases import base_flat
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.parallel.assembly import LayoutError
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(dump_folder=str(tmp_path), enable=True, interval=1, steps=2))
    tr = Trainer(cfg)
    lay = tr.asm.layout
    assert lay is not None and tr.optimizers.layout_snapshot is not None
    names = set(lay.state_names.values())
    assert "model.layers.0.self_attn.q_proj.weight" in names and not any(".inner." in n for n in names)
    tr.train_step()
    tr.checkpointer.save(1, force=True)
    tr.checkpointer.wait()
    # a parameter swapped behind the optimizer's back: the next save refuses instead of writing state under a stale name
    blk = next(m for n, m in tr.model.named_modules() if n.endswith("self_attn.q_proj"))
    blk.weight = torch.nn.Parameter(blk.weight.detach().clone())
    with pytest.raises(LayoutError):
        tr.checkpointer.save(2, force=True)
    tr.close()


def test_replacement_map_composes_events_by_identity():
    import gc
    import torch
    import torch.nn as nn
    from torchllmtuner_b200.parallel.replacements import ReplacementMap
    rm = ReplacementMap()
    a, b, c, d = (nn.Parameter(torch.zeros(2)) for _ in range(4))          # equal values: only identity may tell them apart
    rm.record(parameters={a: (b,)})
    rm.record(parameters={b: (c, d)})
    assert rm.parameters(a) == (c, d) and rm.parameters(b) == (c, d) and rm.parameters(c) == (c,)
    rm.record(parameters={c: ()})                                           # removal
    assert rm.parameters(a) == (d,)
    m0, m1, m2 = nn.Linear(2, 2), nn.Linear(2, 2), nn.Linear(2, 2)
    rm.record(modules={m0: m1})
    rm.record(modules={m1: m2})
    assert rm.module(m0) is m2 and rm.module(m2) is m2
    with pytest.raises(TypeError):
        rm.record(parameters={a: b})
    n = len(rm._params)
    del a
    gc.collect()
    assert len(rm._params) == n - 1                                         # sources are held weakly


def test_heads_must_divide_by_the_axes_that_cut_them():
    from torchllmtuner_b200.errors import UnsupportedCombinationError
    from torchllmtuner_b200.models.qwen3 import Qwen3Config, Qwen3ForCausalLM
    from torchllmtuner_b200.parallel.attention_heads import head_counts, require_heads_divisible_by
    m = Qwen3ForCausalLM(Qwen3Config(num_attention_heads=8, num_key_value_heads=2, hidden_size=64), device="meta")
    assert head_counts(m) == [("num_attention_heads", 8), ("num_key_value_heads", 2)]
    require_heads_divisible_by(m, size=2, axis="tp", why="whole heads per rank")
    with pytest.raises(UnsupportedCombinationError, match=r"num_key_value_heads \(2\) must be divisible by tp \(4\): whole heads"):
        require_heads_divisible_by(m, size=4, axis="tp", why="whole heads per rank")
    with pytest.raises(UnsupportedCombinationError, match="Ulysses"):
        m.validate_parallel(tp=2, cp_ulysses=2)
