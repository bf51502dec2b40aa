"""Checkpoint save / resume through the Trainer, resharding across DP and EP degrees, HF round trip."""
import os
import shutil

import pytest
import torch

from caps import skip_without
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


@skip_without("safetensors")
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
    """Keys follow the reference's flattened names: bare `<fqn>` for model tensors (whole N-D tensors),
    `optimizer.state.<fqn>.<moment>`, `ema.ema_params.<fqn>`, plus lr scheduler, train state, data loader and RNG entries."""
    import torch.distributed.checkpoint as dcp
    folder = str(tmp_path / "run")
    cfg = _cfg(folder)
    tr = Trainer(cfg)
    tr.train_step()
    tr.checkpointer.save(1, force=True)
    tr.checkpointer.wait()
    tr.close()
    md = dcp.FileSystemReader(os.path.join(folder, "checkpoint", "step-1")).read_metadata().state_dict_metadata
    keys = set(md.keys())
    assert "model.layers.0.self_attn.q_proj.weight" in keys, sorted(keys)[:20]
    assert "optimizer.state.model.layers.0.self_attn.q_proj.weight.exp_avg" in keys
    assert "optimizer.state.model.layers.0.self_attn.q_proj.weight.exp_avg_sq" in keys
    assert len(md["model.layers.0.self_attn.q_proj.weight"].size) == 2          # a whole matrix, not a flat piece
    # any DCP reader gets the whole tensor without this framework's code
    want = {"model.layers.0.self_attn.q_proj.weight": torch.zeros(tuple(md["model.layers.0.self_attn.q_proj.weight"].size))}
    dcp.load(want, checkpoint_id=os.path.join(folder, "checkpoint", "step-1"), no_dist=True)
    assert want["model.layers.0.self_attn.q_proj.weight"].abs().sum() > 0
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


def test_reference_key_layout_round_trip(tmp_path):
    """A checkpoint of this framework is exported to the reference's key layout (whole tensors under the names of the
    reference's modules, packed experts as gate_up_proj / down_proj, optimizer flattened per parameter name), read back
    into a native folder, and a fresh trainer that resumes from that folder continues bit for bit."""
    import torch.distributed.checkpoint as dcp
    from torchllmtuner_b200.components.checkpointer.reference_layout import (export_reference_layout, import_reference_layout,
                                                                             native_shapes)
    folder = str(tmp_path / "run")

    def cfg_of(f):
        cfg = _cfg(f, model_name_or_path="qwen3_moe", exclude_from_loading=["dataloader", "rng"])
        cfg.model.arch_overrides = dict(MOE)
        return cfg
    tr = Trainer(cfg_of(folder))
    for _ in range(2):
        tr.train_step()
    tr.checkpointer.save(2, force=True)
    tr.checkpointer.wait()
    shapes = native_shapes(tr.model)
    E, F, D = shapes["model.layers.0.mlp.routed.experts.w1_EFD"]
    w1 = dict(tr.model.named_parameters())["model.layers.0.mlp.routed.experts.w1_EFD"]
    masters = [u.master.clone() for u in tr.asm.fsdp.units]
    moments = {n: {k: v.clone() for k, v in st.items() if torch.is_tensor(v)} for n, st in tr.optimizers.optimizers[0].state.items()}
    batches = [tr.train_step().loss for _ in range(2)]
    tr.close()

    ref_dir = str(tmp_path / "reference_layout")
    info = export_reference_layout(os.path.join(folder, "checkpoint", "step-2"), ref_dir)
    keys = set(info["keys"])
    for k in ("model.layers.0.self_attn.q_proj.weight", "model.layers.0.mlp.experts.gate_up_proj", "model.layers.0.mlp.experts.down_proj",
              "model.layers.0.mlp.gate.weight", "optimizer.state.model.layers.0.self_attn.q_proj.weight.exp_avg",
              "optimizer.state.model.layers.0.mlp.experts.gate_up_proj.exp_avg_sq", "optimizer.state.model.embed_tokens.weight.step",
              "optimizer.param_groups.model.layers.0.self_attn.q_proj.weight.lr",
              "optimizer.param_groups.model.norm.weight.weight_decay", "lr_scheduler.last_epoch", "train_state.step"):
        assert k in keys, (k, sorted(keys)[:40])
    md = dcp.FileSystemReader(ref_dir).read_metadata().state_dict_metadata
    assert tuple(md["model.layers.0.mlp.experts.gate_up_proj"].size) == (E, 2 * F, D)
    assert tuple(md["optimizer.state.model.layers.0.mlp.experts.down_proj.exp_avg"].size) == (E, D, F)
    # gate rows then up rows of each expert
    want = {"model.layers.0.mlp.experts.gate_up_proj": torch.empty(E, 2 * F, D)}
    dcp.load(want, checkpoint_id=ref_dir, no_dist=True)
    del w1

    folder2 = str(tmp_path / "run2")
    back = import_reference_layout(ref_dir, os.path.join(folder2, "checkpoint", "step-2"), shapes, state_format="qwen3")
    assert back["step"] == 2
    tr2 = Trainer(cfg_of(folder2))
    assert tr2.checkpointer.load()
    assert tr2.progress.step == 2
    for a, u in zip(masters, tr2.asm.fsdp.units):
        assert torch.equal(a[:u.numel], u.master[:u.numel])
    for n, st in tr2.optimizers.optimizers[0].state.items():
        for k, v in st.items():
            if torch.is_tensor(v) and k in moments[n]:
                assert torch.equal(v, moments[n][k]), (n, k)
    tr2.close()


def test_flat_range_boxes_tile_the_range_exactly():
    """A flat range of a row-major tensor is at most 2N-1 boxes whose concatenation, in order, is the range."""
    import random
    from torchllmtuner_b200.components.checkpointer.boxes import boxes_of_slice, flat_range_boxes
    rnd = random.Random(0)
    for shape in [(7,), (5, 4), (3, 4, 5), (2, 3, 2, 4), (6, 1, 3)]:
        n = 1
        for s in shape:
            n *= s
        ref = torch.arange(n).view(shape)
        for _ in range(100):
            lo = rnd.randint(0, n)
            hi = rnd.randint(lo, n)
            bx = flat_range_boxes(lo, hi, shape)
            assert len(bx) <= max(1, 2 * len(shape) - 1)
            pos = lo
            for off, size, start in bx:
                v = ref[tuple(slice(o, o + s) for o, s in zip(off, size))].reshape(-1)
                assert start == pos - lo and torch.equal(v, torch.arange(pos, pos + v.numel()))
                pos += v.numel()
            assert pos == hi
    # a column cut places the boxes at the rank's columns; padding rows of a vocabulary cut are clipped
    b = boxes_of_slice("w", 0, 6, (3, 2), (3, 8), (0, 4))
    assert [(x.offsets, x.sizes) for x in b] == [((0, 4), (3, 2))]
    b = boxes_of_slice("emb", 0, 12, (4, 3), (6, 3), (4, 0))          # rank 1 of a vocabulary of 6 padded to 8
    assert [(x.offsets, x.sizes, x.numel) for x in b] == [((4, 0), (2, 3), 6)]


def test_format_2_pieces_are_still_read(tmp_path):
    """A folder in the previous format (flat pieces keyed `model.<fqn>@lo:hi`) resumes: the loader migrates on read."""
    import torch.distributed.checkpoint as dcp
    from torchllmtuner_b200.components.checkpointer.dcp_manager import _pack, iter_pieces
    folder = str(tmp_path / "run")
    tr = Trainer(_cfg(folder))
    tr.train_step()
    state = {}
    for fqn, tag, glo, ghi, u, slo in iter_pieces(tr.asm.fsdp):
        mid = glo + (ghi - glo) // 2                       # two pieces per tensor, as two ranks would have written
        for a, b in ((glo, mid), (mid, ghi)):
            if b > a:
                state[f"model.{fqn}{tag}@{a}:{b}"] = u.master[slo + a - glo: slo + b - glo].clone()
    state["obj.format"] = _pack({"version": 2})
    state["obj.train_state"] = _pack(tr.progress.state_dict())
    os.makedirs(os.path.join(folder, "checkpoint"), exist_ok=True)
    dcp.save(state, checkpoint_id=os.path.join(folder, "checkpoint", "step-1"), no_dist=True)
    masters = [u.master.clone() for u in tr.asm.fsdp.units]
    tr.close()
    tr2 = Trainer(_cfg(folder, exclude_from_loading=["optimizer", "lr_scheduler", "dataloader", "rng"]))
    for u in tr2.asm.fsdp.units:
        u.master.zero_()
    assert tr2.checkpointer.load()
    for a, u in zip(masters, tr2.asm.fsdp.units):
        assert torch.equal(a[:u.numel], u.master[:u.numel])
    tr2.close()


@skip_without("fsspec")
def test_checkpoints_on_an_fsspec_store(tmp_path):
    """The same save / publish / purge / resume cycle against a URI: the in-memory fsspec filesystem stands in for an
    object store. A second run then starts from that store through `initial_load_path` while writing locally."""
    import fsspec
    uri = f"memory://ckpt-{os.getpid()}/run"

    def cfg_of(**flat):
        c = _cfg(str(tmp_path / "unused"), interval=1, keep_latest_k=2, **flat)
        c.training.checkpoint_config.folder = uri
        return c
    tr = Trainer(cfg_of())
    ref = []
    for _ in range(4):
        r = tr.train_step()
        ref.append(r.loss)
        tr.checkpointer.save(r.step)
    tr.close()
    fs = fsspec.filesystem("memory")
    names = sorted(os.path.basename(p) for p in fs.ls(uri[len("memory://"):], detail=False))
    assert names == ["step-3", "step-4"], names                      # purged to the latest two, no temporary folder left
    assert not os.path.exists(str(tmp_path / "unused" / "checkpoint"))
    fs.rm(uri[len("memory://"):] + "/step-4", recursive=True)
    tr2 = Trainer(cfg_of())
    assert tr2.checkpointer.load() and tr2.progress.step == 3
    got = tr2.train_step().loss
    tr2.close()
    assert got == ref[3]
    # a local run seeded from the store
    c3 = _cfg(str(tmp_path / "local"), initial_load_path=uri + "/step-3", initial_load_model_only=False)
    tr3 = Trainer(c3)
    assert tr3.checkpointer.load() and tr3.progress.step == 3
    assert tr3.train_step().loss == ref[3]
    tr3.close()
    fs.rm(uri[len("memory://"):], recursive=True)


@skip_without("fsspec")
def test_storage_path_rules():
    from torchllmtuner_b200.components.checkpointer.storage import FsspecStorage, LocalStorage, is_remote, storage_for
    assert is_remote("gs://bucket/run") and is_remote("memory://x") and not is_remote("/abs/run") and not is_remote("C:\\run")
    assert isinstance(storage_for("./out"), LocalStorage) and isinstance(storage_for("s3://b/k"), FsspecStorage)
    st = FsspecStorage()
    assert st.join("./outputs", "gs://bucket/ck") == "gs://bucket/ck"          # a URI restarts the path
    assert st.join("gs://bucket/run", "checkpoint", "step-3") == "gs://bucket/run/checkpoint/step-3"
    assert LocalStorage().join("/a", "b", "c") == os.path.join("/a", "b", "c")
    st.makedirs("memory://rules/a/a")
    with __import__("fsspec").open("memory://rules/a/a/f", "wb") as f:
        f.write(b"x")
    assert st.listdir("memory://rules/a") == ["a"] and st.listdir("memory://rules/a/a") == ["f"]
    st.rmtree("memory://rules/a")
    st.rmtree("memory://rules/a")                                              # missing is fine
    assert not st.exists("memory://rules/a/a/f")


@pytest.mark.parametrize("name", ["qwen3", "qwen3_moe", "qwen3_5", "qwen3_5_moe", "kimi_linear", "kimi_k3", "deepseek_v4"])
def test_a_config_json_written_by_the_export_builds_the_same_architecture(name, tmp_path):
    """`model_name_or_path=<folder>`: every family's exported config.json maps back to its registered builder and to the
    same architecture (parameter names and shapes), through the state format's `arch_from_hf`."""
    import json
    from torchllmtuner_b200.config.model_config import ModelConfig
    from torchllmtuner_b200.models.registry import build_registered_model
    from torchllmtuner_b200.models.state import get_state_format
    mc = ModelConfig(model_name_or_path=name, vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                     num_attention_heads=4, num_key_value_heads=2)
    with torch.device("meta"):
        m0 = build_registered_model(mc)
    (tmp_path / "config.json").write_text(json.dumps(get_state_format(m0.state_format).hf_config(m0.config)))
    with torch.device("meta"):
        m1 = build_registered_model(ModelConfig(model_name_or_path=str(tmp_path)))
    assert m1.state_format == m0.state_format and type(m1) is type(m0)
    assert {n: tuple(p.shape) for n, p in m1.named_parameters()} == {n: tuple(p.shape) for n, p in m0.named_parameters()}
    import dataclasses
    a, b = dataclasses.asdict(m0.config), dataclasses.asdict(m1.config)
    assert {k for k in a if a[k] != b[k]} <= {"model_type", "intermediate_size"}      # labels; V4 has no dense MLP width


@skip_without("safetensors")
def test_an_exported_folder_is_a_model_name_and_an_initial_checkpoint(tmp_path):
    """Export a Kimi-K3 run as Hugging Face files; a new run names that folder as its model and its initial checkpoint and
    starts from the same weights."""
    from torchllmtuner_b200.components.checkpointer.hf import save_hf_checkpoint
    cfg = _cfg(str(tmp_path / "run"), model_name_or_path="kimi_k3", num_hidden_layers=4)
    cfg.model.arch_overrides = dict(head_dim=16, linear_heads=2, linear_head_dim=8)
    tr = Trainer(cfg)
    tr.train_step()
    out = str(tmp_path / "hf")
    save_hf_checkpoint(tr, out, "float32")
    cfg2 = _cfg(str(tmp_path / "run2"), model_name_or_path=out, initial_load_path=out, initial_load_in_hf=True)
    tr2 = Trainer(cfg2)
    assert tr2.checkpointer.load()
    a = {u.name: u.master[:u.numel].clone() for u in tr.asm.fsdp.units}
    b = {u.name: u.master[:u.numel].clone() for u in tr2.asm.fsdp.units}
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    tr.close()
    tr2.close()
    # the preflight agrees, and notices a tensor that went missing or changed shape
    import json
    from safetensors.torch import load_file, save_file
    from torchllmtuner_b200.components.checkpointer import hf_preflight
    rep = hf_preflight.preflight(out)
    assert rep["ok"] and rep["registered_model"] == "kimi_linear" and rep["missing_count"] == rep["unused_count"] == 0
    assert hf_preflight.main([out]) == 0
    wm = json.load(open(os.path.join(out, "model.safetensors.index.json")))["weight_map"]
    victim = "model.layers.0.self_attn.A_log"
    path = os.path.join(out, wm[victim])
    tensors = load_file(path)
    tensors[victim] = tensors[victim][:-1].clone()
    dropped = next(k for k in tensors if k.endswith("q_conv1d.weight"))
    del tensors[dropped]
    save_file(tensors, path)
    rep = hf_preflight.preflight(out)
    assert not rep["ok"] and victim in rep["shape_mismatches"] and dropped in rep["missing"] and hf_preflight.main([out, "--json"]) == 1
