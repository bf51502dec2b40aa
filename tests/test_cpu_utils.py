"""Small services on their own: FLOP accounting, aligned garbage collection, tensor trees, corpus identity, collation,
input sharding for context and tensor parallelism, the non-finite guard, capability probes, meta materialisation,
metric loggers, dispatch timing, progress state."""
import gc
import json
import os

import pytest
import torch
import torch.nn as nn

from torchllmtuner_b200.errors import ConfigError, EnvironmentUnsupportedError, LLMTunerError


def test_flops_per_token_formula():
    from torchllmtuner_b200.utils.flops import generic_flops_per_token
    D, L, H, Hkv, d, F, V, S = 64, 3, 4, 2, 16, 128, 1000, 256
    attn = 2 * (D * H * d + 2 * D * Hkv * d + H * d * D)
    want = 3 * (L * (attn + 6 * D * F) + 2 * V * D) + L * 6 * H * 2 * d * S
    got = generic_flops_per_token(hidden_size=D, num_layers=L, num_heads=H, num_kv_heads=Hkv, head_dim=d, intermediate_size=F,
                                  vocab_size=V, seq_len=S)
    assert got == want
    # experts replace the dense MLP only on the layers the mask names
    moe = 2 * (D * 8 + 2 * 3 * D * 32 + 3 * D * 16)
    got = generic_flops_per_token(hidden_size=D, num_layers=L, num_heads=H, num_kv_heads=Hkv, head_dim=d, intermediate_size=F,
                                  vocab_size=V, seq_len=S, num_experts=8, top_k=2, moe_intermediate_size=32,
                                  shared_intermediate_size=16, moe_layer_mask=[False, True, True])
    assert got == 3 * (L * attn + 6 * D * F + 2 * moe + 2 * V * D) + L * 6 * H * 2 * d * S


def test_peak_flops_table_and_measured_override(monkeypatch):
    from torchllmtuner_b200.utils import monitoring
    assert monitoring.get_peak_flops("NVIDIA B200") == 2.25e15 and monitoring.get_peak_flops("NVIDIA H100 PCIe") == 756e12
    assert monitoring.get_peak_flops("some other device") == 0.0
    monkeypatch.setenv("LLMT_MEASURED_PEAK_TFLOPS", "1400")
    assert monitoring.get_measured_peak_flops() == 1.4e15


def test_garbage_collection_runs_on_its_own_schedule_and_restores_the_setting():
    from torchllmtuner_b200.utils.garbage_collection import GarbageCollection
    assert gc.isenabled()
    with GarbageCollection(gc_freq=3) as g:
        assert not gc.isenabled()
        seen = []
        for step in range(1, 10):
            g.last_pause_s = -1.0
            g.run(step)
            if g.last_pause_s >= 0:
                seen.append(step)
        assert seen == [3, 6, 9]
    assert gc.isenabled()
    with pytest.raises(ValueError):
        GarbageCollection(gc_freq=0)


def test_tensor_trees():
    from torchllmtuner_b200.accelerator.tensor_tree import clone_local_tensor, get_tensor_tree_device, move_tensor_tree
    tree = {"a": [torch.ones(2), ("x", torch.zeros(1))], "b": 3}
    assert get_tensor_tree_device(tree) == torch.device("cpu") and get_tensor_tree_device({"n": [1, "s"]}) is None
    moved = move_tensor_tree(tree, "cpu")
    assert moved["b"] == 3 and isinstance(moved["a"][1], tuple) and torch.equal(moved["a"][0], tree["a"][0])
    p = nn.Parameter(torch.ones(3))
    c = clone_local_tensor(p)
    assert not c.requires_grad and c.data_ptr() != p.data_ptr()


def test_corpus_identity_follows_data_and_settings(tmp_path):
    from types import SimpleNamespace as NS
    from torchllmtuner_b200.datasets.corpus_identity import corpus_data_identity
    f = tmp_path / "a.jsonl"
    f.write_text('{"text": "one"}\n')
    cfg = NS(data_identity="", dataset="local_text", packing="greedy", num_packing_bins=4, max_num_documents=0, prompt_field="p",
             response_field="r", text_field="text", messages_field="m", chat_template=None)
    a = corpus_data_identity(cfg, "tok-1", [str(f)])
    assert a == corpus_data_identity(cfg, "tok-1", [str(f)]) and len(a) == 24
    assert a != corpus_data_identity(cfg, "tok-2", [str(f)])
    cfg2 = NS(**{**vars(cfg), "packing": "none"})
    assert a != corpus_data_identity(cfg2, "tok-1", [str(f)])
    f.write_text('{"text": "two!"}\n')
    assert a != corpus_data_identity(cfg, "tok-1", [str(f)])
    assert corpus_data_identity(NS(**{**vars(cfg), "data_identity": "pinned"}), "tok-9") == "pinned"


def test_text_collator_builds_global_document_cuts():
    from types import SimpleNamespace as NS
    from torchllmtuner_b200.datasets.collators import TextCollator
    from torchllmtuner_b200.datasets.contracts import IGNORE_INDEX
    rows = [NS(tokens=[1, 2, 3, 4], labels=[2, 3, IGNORE_INDEX, 9], positions=[0, 1, 0, 1], cuts=[0, 2, 4]),
            NS(tokens=[5, 6, 7, 8], labels=[6, 7, 8, IGNORE_INDEX], positions=[0, 1, 2, 3], cuts=[0, 4])]
    b = TextCollator(4)(rows)
    assert b["input"].shape == (2, 4) and b["cu_seqlens"].tolist() == [0, 2, 4, 8] and b["num_valid_tokens"] == 6
    assert b["positions"][0].tolist() == [0, 1, 0, 1]


def test_input_sharding_covers_every_row_exactly_once():
    from torchllmtuner_b200.parallel.input_sharding import (contiguous_chunk, cp_row_index, headtail_chunks,
                                                            shard_model_inputs)
    assert headtail_chunks(16, 2, 0) == [(0, 4), (12, 16)] and headtail_chunks(16, 2, 1) == [(4, 8), (8, 12)]
    with pytest.raises(ConfigError):
        headtail_chunks(10, 2, 0)
    with pytest.raises(ConfigError):
        contiguous_chunk(10, 3, 0)
    for lb in (None, "headtail"):
        rows = torch.cat([cp_row_index(2, 16, 4, r, lb) for r in range(4)])
        assert sorted(rows.tolist()) == list(range(32))
    B, S = 2, 16
    inputs = {"batch": B, "seq": S, "tokens": torch.arange(B * S), "targets": torch.arange(B * S) + 1,
              "positions": torch.arange(S).repeat(B), "cu_seqlens": torch.tensor([0, 16, 32], dtype=torch.int32)}
    assert shard_model_inputs(inputs, None) is inputs and shard_model_inputs(inputs, {"cp": 1, "tp": 1}) is inputs
    # CP 2 (head-tail) x TP 2: four ranks tile the tokens; positions stay whole per CP rank
    seen = []
    for c in range(2):
        for t in range(2):
            out = shard_model_inputs(inputs, {"cp": 2, "cp_rank": c, "tp": 2, "tp_rank": t, "load_balancer": "headtail"})
            assert out["positions"].numel() == 16 and out["tokens"].numel() == 8 and out["global_rows"] == 32
            assert torch.equal(out["targets"], out["tokens"] + 1)
            assert torch.equal(out["cp_rows"][out["tp_span"][0]:out["tp_span"][1]], out["tokens"])
            seen += out["tokens"].tolist()
    assert sorted(seen) == list(range(32))
    # two-level CP: key/value axis 2 x ulysses 2
    seen = []
    for kv in range(2):
        for u in range(2):
            out = shard_model_inputs(inputs, {"cp": 4, "cp_kv": 2, "cp_ulysses": 2, "cp_kv_rank": kv, "cp_ulysses_rank": u,
                                              "cp_rank": kv * 2 + u, "tp": 1, "load_balancer": "headtail"})
            seen += out["tokens"].tolist()
    assert sorted(seen) == list(range(32))


def test_non_finite_guard_names_the_first_bad_block_without_reading_back_in_forward():
    from torchllmtuner_b200.parallel.graph_capture import SDCGuard, check_sdc

    class Scale(nn.Module):
        def __init__(self, s):
            super().__init__()
            self.s, self.width = s, 7

        def forward(self, x):
            return x * self.s
    model = nn.Sequential()
    model._sdc_flag = torch.zeros((), dtype=torch.int32)
    for i, s in enumerate([1.0, float("inf"), float("nan")]):
        model.append(SDCGuard(Scale(s), i, model._sdc_flag))
    assert model[0].width == 7                                # attributes of the wrapped block stay reachable
    model[0](torch.ones(3))
    check_sdc(model)                                           # healthy: nothing raised
    model(torch.ones(3))
    with pytest.raises(LLMTunerError, match="block 1"):
        check_sdc(model)
    check_sdc(model)                                           # the flag was cleared by the report
    check_sdc(nn.Linear(2, 2))                                 # a model without the guard


def test_capability_gates_for_tests():
    import caps
    assert caps.available("yaml") and caps.available("dcp") and not caps.missing("yaml")
    assert caps.available("cuda") == torch.cuda.is_available()
    mark = caps.skip_without("yaml", "dcp")
    assert mark.args == (False,) and "missing" in mark.kwargs["reason"]
    with pytest.raises(KeyError):
        caps.available("warp_drive")


def test_capability_probes():
    from torchllmtuner_b200.accelerator import capabilities as cap
    rep = cap.report()
    assert set(rep) == set(cap.CAPABILITIES) and rep["dcp"] and rep["yaml"]
    assert rep["cuda"] == torch.cuda.is_available()
    with pytest.raises(KeyError):
        cap.has("warp_drive")
    if not rep["cuda"]:
        with pytest.raises(EnvironmentUnsupportedError, match="needs a device"):
            cap.require("cuda", "needs a device")


def test_meta_materialisation_keeps_ties_marks_and_buffer_persistence():
    from torchllmtuner_b200.memory.materialization import materialize_meta_model

    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(10, 4)
            self.head = nn.Linear(4, 10, bias=False)
            self.head.weight = self.embed.weight
            self.frozen = nn.Parameter(torch.empty(3), requires_grad=False)
            self.register_buffer("table", torch.empty(5), persistent=False)
            self.other = nn.Module()
            self.other.register_buffer("table", self.table)
    with torch.device("meta"):
        m = Tied()
    m.embed.weight.tp_shard_dim = 0
    assert materialize_meta_model(m, "cpu") == 3
    assert m.head.weight is m.embed.weight and not m.embed.weight.is_meta and m.embed.weight.tp_shard_dim == 0
    assert not m.frozen.requires_grad and m.table is m.other.table and float(m.table.abs().sum()) == 0.0
    assert "table" not in m.state_dict() and len(list(m.parameters())) == 2
    assert materialize_meta_model(m, "cpu") == 0


def test_metric_loggers(tmp_path):
    from types import SimpleNamespace as NS
    from torchllmtuner_b200.utils.metric_loggers import JsonlLogger, LoggerContainer, build_metric_logger
    path = tmp_path / "m" / "metrics.jsonl"
    lg = LoggerContainer([JsonlLogger(str(path))])
    lg.log({"loss": 1.5, "tps": 10}, 3)
    lg.log({"loss": torch.tensor(1.25), "note": "warm-up", "skipped": None, "ok": True}, 4)       # only numbers are written
    lg.close()
    lines = [json.loads(x) for x in path.read_text().splitlines()]
    assert [x["step"] for x in lines] == [3, 4] and lines[0]["loss"] == 1.5 and lines[1] == {"step": 4, "loss": 1.25}
    cfg = NS(log_ranks=[0], save_for_all_ranks=False, enable_tensorboard=False, enable_wandb=False, save_tb_folder="tb", tag=None)
    assert build_metric_logger(cfg, str(tmp_path), rank=1).loggers == []
    assert build_metric_logger(cfg, str(tmp_path), rank=0).loggers == []
    cfg.enable_tensorboard, cfg.save_for_all_ranks = True, True
    c = build_metric_logger(cfg, str(tmp_path), rank=1)
    assert len(c.loggers) == 1
    c.log({"loss": 2.0}, 1)
    c.close()
    assert os.path.isdir(tmp_path / "tb" / "rank_1")


def test_dispatch_timer_percentiles_on_the_host():
    from torchllmtuner_b200.trainer.runtime.observer import DispatchTimer
    t = DispatchTimer("cpu")
    for _ in range(5):
        with t.span("dispatch"):
            pass
    with t.span("combine"):
        pass
    out = t.collect()
    assert {"moe/dispatch_p50(ms)", "moe/dispatch_p90(ms)", "moe/dispatch_total(ms)", "moe/combine_p50(ms)"} <= set(out)
    assert out["moe/dispatch_p50(ms)"] <= out["moe/dispatch_p90(ms)"] <= out["moe/dispatch_total(ms)"]
    assert t.collect() == {}


def test_progress_state_round_trip():
    from torchllmtuner_b200.trainer.runtime.results import StepResult, TrainingProgress
    p = TrainingProgress(step=7, ntokens_seen=1234)
    q = TrainingProgress()
    q.load_state_dict(json.loads(json.dumps(p.state_dict())))
    assert q == p
    r = StepResult(step=1, loss=2.0, grad_norm=0.5, lr=1e-3, global_tokens=64, step_seconds=0.1)
    assert r.extra == {} and r.max_loss is None


def test_nvtx_ranges_are_free_when_disabled():
    from torchllmtuner_b200.utils import nvtx
    nvtx.enable(True)                      # without a device this stays off
    assert nvtx._ENABLED == torch.cuda.is_available()
    nvtx.enable(False)
    with nvtx.nvtx_range("step"):
        pass


# ---------------------------------------------------------------------------------------------- config groups on their own
def test_parallel_config_rules():
    from torchllmtuner_b200.config.parallel_config import (ContextParallelConfig, ExpertParallelConfig, FSDPConfig, ParallelConfig,
                                                           TensorParallelConfig)
    p = ParallelConfig(tensor_parallel_size=2, context_parallel_ulysses_size=2)
    assert p.cp_size == 2 and p.derive_dp(8) == (1, 2)
    assert ParallelConfig(data_parallel_replicate_size=2, data_parallel_shard_size=2).derive_dp(4) == (2, 2)
    with pytest.raises(ConfigError, match="not divisible"):
        ParallelConfig(tensor_parallel_size=3).derive_dp(8)
    with pytest.raises(ConfigError, match="!= world size"):
        ParallelConfig(data_parallel_shard_size=3).derive_dp(8)
    with pytest.raises(ConfigError):
        ParallelConfig(tensor_parallel_size=0)
    with pytest.raises(ConfigError, match="sequence-parallel"):
        ParallelConfig(tensor_parallel_size=2, tp_config=TensorParallelConfig(enable_sequence_parallel=False))
    with pytest.raises(ConfigError):
        FSDPConfig(fsdp_reduce_dtype="float16")
    with pytest.raises(ConfigError, match="cpu_offload"):
        FSDPConfig(fsdp_cpu_offload=True, enable_fsdp_symm_mem=True)
    with pytest.raises(ConfigError):
        FSDPConfig(fsdp_ignored_modules=[""])
    with pytest.raises(ConfigError, match="ptrr"):
        ContextParallelConfig(context_parallel_load_balancer="ptrr")
    with pytest.raises(ConfigError):
        ContextParallelConfig(context_parallel_strategy="ring")
    with pytest.raises(ConfigError, match=">= 1"):
        ExpertParallelConfig(ep_capacity_factor=0.5)
    with pytest.raises(ConfigError, match=">= 0"):
        ExpertParallelConfig(router_aux_loss_coef=-1.0)
    with pytest.raises(ConfigError, match="registered gap"):
        ExpertParallelConfig(ep_token_dispatcher="mc2")


def test_model_and_observability_config_rules():
    from torchllmtuner_b200.config.model_config import ModelConfig
    from torchllmtuner_b200.config.observability_config import MetricsConfig, ProfilerConfig
    assert ModelConfig(compute_dtype="bfloat16").compute_dtype == "bfloat16"
    for bad in (dict(initialization_device="tpu"), dict(hidden_size=0), dict(qkv_projection="packed"),
                dict(experts_implementation="triton"), dict(compute_dtype="int8")):
        with pytest.raises(ConfigError):
            ModelConfig(**bad)
    assert MetricsConfig(log_ranks=("0", 3)).log_ranks == [0, 3]
    with pytest.raises(ConfigError):
        MetricsConfig(log_freq=0)
    ProfilerConfig(enable_profiling=True, profile_freq=4, profiler_active=1, profiler_warmup=3)
    with pytest.raises(ConfigError, match="profile_freq"):
        ProfilerConfig(enable_profiling=True, profile_freq=3, profiler_active=1, profiler_warmup=3)
    with pytest.raises(ConfigError, match="Ascend"):
        ProfilerConfig(npu_profiler_level="level1")


def test_rank_aware_logging(monkeypatch, tmp_path):
    import logging
    from torchllmtuner_b200.utils import logging as L
    flt = L._RankFilter()
    rec = lambda lvl: logging.LogRecord("x", lvl, __file__, 1, "m", None, None)  # noqa: E731
    monkeypatch.setenv("RANK", "3")
    L.set_log_ranks([0])
    assert not flt.filter(rec(logging.INFO)) and flt.filter(rec(logging.ERROR))      # every rank prints errors
    L.set_log_ranks([0, 3])
    assert flt.filter(rec(logging.INFO))
    L.set_log_ranks([0])
    monkeypatch.setenv("RANK", "0")
    root = logging.getLogger("torchllmtuner_b200")
    earlier = [h for h in root.handlers if isinstance(h, logging.FileHandler)]      # one file per process: set any aside
    for h in earlier:
        root.removeHandler(h)
    log = L.get_logger("torchllmtuner_b200.trainer", log_file=str(tmp_path / "logs" / "run.log"))
    assert log.name == "torchllmtuner_b200.trainer"
    log.info("hello from the test")
    for h in logging.getLogger("torchllmtuner_b200").handlers:
        h.flush()
    assert "hello from the test" in (tmp_path / "logs" / "run.log").read_text()
    for h in [h for h in root.handlers if isinstance(h, logging.FileHandler)]:
        root.removeHandler(h)
        h.close()
    for h in earlier:
        root.addHandler(h)


def test_graph_replay_follows_the_forward_context():
    """A replayed block must read the CURRENT call's context. The capture backend is replaced by one that re-runs the
    captured closure (which only sees the static buffers), so stale buffers would show."""
    from dataclasses import dataclass
    from torchllmtuner_b200.ops.attn_meta import AttnMeta
    from torchllmtuner_b200.parallel.graph_capture import GraphedInference, context_leaves
    from torchllmtuner_b200.models.qwen3 import ForwardContext

    class Block(nn.Module):
        def forward(self, x, ctx):
            return x * ctx.cos.sum() + len(ctx.attn_meta.pieces)

    def fake_capture(fn):
        out = fn()
        def replay():
            out.copy_(fn())
        return out, replay
    g = GraphedInference(Block(), capture=fake_capture).eval()
    ctx = lambda c, cu: ForwardContext(torch.full((4,), float(c)), torch.zeros(4), AttnMeta.build(torch.tensor(cu)))  # noqa: E731
    x = torch.ones(3)
    with torch.no_grad():
        assert g(x, ctx(1, [0, 8])).tolist() == [5.0] * 3 and g.captures == 1
        assert g(x * 2, ctx(2, [0, 8])).tolist() == [17.0] * 3 and g.captures == 1       # same layout: tensors copied, replayed
        assert g(x, ctx(1, [0, 3, 8])).tolist() == [6.0] * 3 and g.captures == 2         # other documents: captured anew
        assert g(torch.ones(5), ctx(1, [0, 3, 8])).shape == (5,) and g.captures == 3     # other input shape
    y = g(x.requires_grad_(), ctx(3, [0, 8]))                                           # with gradients: the plain block
    assert y.requires_grad and g.captures == 3
    t, c = context_leaves(ctx(1, [0, 4, 8]))
    assert len(t) >= 2 and (0, 4, 0, 4, 0) in [tuple(p) for p in AttnMeta.build(torch.tensor([0, 4, 8])).pieces] and "pieces" in c


def test_loss_helpers_on_one_rank():
    from torchllmtuner_b200.components.loss import (chunked_lm_head_cross_entropy, compute_logprobs, cross_entropy_loss, mse_loss,
                                                    vocab_parallel_entropy)
    from torchllmtuner_b200.ops import IGNORE_INDEX
    torch.manual_seed(0)
    logits = torch.randn(6, 11)
    tgt = torch.tensor([1, 4, IGNORE_INDEX, 10, 0, IGNORE_INDEX])
    keep = tgt != IGNORE_INDEX
    want = torch.nn.functional.cross_entropy(logits[keep], tgt[keep], reduction="sum")
    assert torch.allclose(cross_entropy_loss(logits, tgt), want, atol=1e-5)                       # a SUM over valid tokens
    lp = compute_logprobs(logits, tgt)
    assert torch.allclose(-lp.sum(), want, atol=1e-5) and float(lp[2]) == 0.0
    p = logits.softmax(-1)
    assert torch.allclose(vocab_parallel_entropy(logits), -(p * p.log()).sum(-1), atol=1e-5)
    assert float(mse_loss(torch.ones(2, 3), torch.zeros(2, 3))) == 6.0
    h, w = torch.randn(6, 5, requires_grad=True), torch.randn(11, 5, requires_grad=True)
    full = cross_entropy_loss(h @ w.t(), tgt)
    gh, gw = torch.autograd.grad(full, [h, w])
    for chunks in (1, 3, 8):
        loss = chunked_lm_head_cross_entropy(h, w, tgt, chunks)
        a, b = torch.autograd.grad(loss, [h, w])
        assert torch.allclose(loss, full, atol=1e-5) and torch.allclose(a, gh, atol=1e-5) and torch.allclose(b, gw, atol=1e-5)
