"""Qwen3.5 / Qwen3.5-MoE against the Hugging Face implementation that ships with `transformers` (an oracle, used only
here): same weights through this framework's state format, same tokens, logits compared in fp32. Plus three-axis rotary
positions, document isolation of the convolution and recurrence, and sequence parallelism."""
import json
import os

import pytest
import torch

from dist_cases import base_flat, run_ranks
from torchllmtuner_b200.models import qwen3_5 as q35
from torchllmtuner_b200.models.state import get_state_format
from torchllmtuner_b200.ops import AttnMeta

hf = pytest.importorskip("transformers.models.qwen3_5_moe.modeling_qwen3_5_moe")
from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig  # noqa: E402

ARCH = dict(vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
            head_dim=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, shared_expert_intermediate_size=40,
            linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=24, linear_conv_kernel_dim=4,
            rope_theta=10000.0, partial_rotary_factor=0.5, mrope_section=[4, 2, 2], rms_norm_eps=1e-6, linear_chunk_size=8)


def _ours():
    torch.manual_seed(0)
    m = q35.Qwen35ForCausalLM(q35.Qwen35Config(**ARCH), dtype=torch.float32)
    m.initialize_parameters(seed=5)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2 and "conv1d" not in n:
                p.mul_(4.0)
            if n.endswith("layernorm.weight") or n.endswith("_norm.weight") or n == "model.norm.weight":
                p.normal_(0, 0.2)                                  # zero-centred weights away from zero
    return m.eval()


def _theirs(ours):
    cfg = Qwen3_5MoeTextConfig(vocab_size=96, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                               num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, shared_expert_intermediate_size=40,
                               linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=24,
                               linear_conv_kernel_dim=4, rms_norm_eps=1e-6, tie_word_embeddings=False,
                               rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                                "mrope_section": [4, 2, 2], "mrope_interleaved": True})
    cfg._attn_implementation = "eager"
    model = hf.Qwen3_5MoeForCausalLM(cfg).eval()
    fmt = get_state_format("qwen3_5")
    sd = model.state_dict()
    filled = {k: torch.zeros(v.numel()) for k, v in sd.items()}
    seen = set()
    for name, p in ours.named_parameters():
        for pc in fmt.hf_pieces(name, tuple(p.shape)):
            assert pc.name in sd, (name, pc.name, [k for k in sd if "layers.0" in k])
            assert tuple(sd[pc.name].shape) == tuple(pc.shape), (pc.name, sd[pc.name].shape, pc.shape)
            filled[pc.name][pc.ref_lo:pc.ref_lo + pc.n] = p.detach().reshape(-1)[pc.native_lo:pc.native_lo + pc.n]
            seen.add(pc.name)
    assert seen == set(sd), (set(sd) - seen, seen - set(sd))       # every HF tensor has a native source and vice versa
    model.load_state_dict({k: filled[k].view(sd[k].shape) for k in sd})
    return model


def test_logits_match_the_hugging_face_model():
    ours = _ours()
    theirs = _theirs(ours)
    S = 37
    tok = torch.randint(0, 96, (S,))
    with torch.no_grad():
        ctx = ours.build_context(torch.arange(S), AttnMeta.build(torch.tensor([0, S], dtype=torch.int32), causal=True))
        got = ours(tok, ctx)
        want = theirs(input_ids=tok[None]).logits[0]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (got - want).abs().max()


def test_three_axis_positions_match_the_hugging_face_rotary():
    ours = _ours()
    theirs = _theirs(ours)
    S = 24
    tok = torch.randint(0, 96, (S,))
    pos = torch.stack((torch.arange(S), torch.arange(S) // 3, torch.arange(S) % 5))        # time, height, width
    with torch.no_grad():
        ctx = ours.build_context(pos, AttnMeta.build(torch.tensor([0, S], dtype=torch.int32), causal=True))
        got = ours(tok, ctx)
        want = theirs(input_ids=tok[None], position_ids=pos[:, None, :]).logits[0]
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (got - want).abs().max()
    with torch.no_grad():
        flat = ours(tok, ours.build_context(torch.arange(S), ctx.attn_meta))
    assert not torch.allclose(flat, got, atol=1e-3)                # the extra axes matter


def test_documents_are_isolated_in_the_convolution_and_the_recurrence():
    ours = _ours()
    lens = [15, 9]
    tok = torch.randint(0, 96, (24,))
    cu = torch.tensor([0, 15, 24], dtype=torch.int32)
    with torch.no_grad():
        both = ours(tok, ours.build_context(torch.cat([torch.arange(n) for n in lens]), AttnMeta.build(cu, causal=True)))
        alone = ours(tok[15:], ours.build_context(torch.arange(9), AttnMeta.build(torch.tensor([0, 9], dtype=torch.int32), causal=True)))
    assert torch.allclose(both[15:], alone, atol=1e-5)


def test_hf_export_writes_packed_experts_and_imports_back(tmp_path):
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.components.checkpointer.hf import load_hf_checkpoint, save_hf_checkpoint
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path="qwen3_5_moe", num_hidden_layers=4, dump_folder=str(tmp_path / "run")))
    cfg.model.arch_overrides = dict(head_dim=16)
    tr = Trainer(cfg)
    tr.train_step()
    out = str(tmp_path / "hf")
    save_hf_checkpoint(tr, out, "float32")
    wm = json.load(open(os.path.join(out, "model.safetensors.index.json")))["weight_map"]
    for k in ("model.layers.0.linear_attn.in_proj_qkv.weight", "model.layers.0.linear_attn.A_log", "model.layers.0.linear_attn.conv1d.weight",
              "model.layers.3.self_attn.q_proj.weight", "model.layers.1.mlp.experts.gate_up_proj", "model.layers.1.mlp.experts.down_proj",
              "model.layers.1.mlp.gate.weight", "model.layers.1.mlp.shared_expert.up_proj.weight", "model.layers.1.mlp.shared_expert_gate.weight"):
        assert k in wm, (k, sorted(wm)[:40])
    from safetensors import safe_open
    with safe_open(os.path.join(out, wm["model.layers.1.mlp.experts.gate_up_proj"]), "pt") as f:
        gu = f.get_tensor("model.layers.1.mlp.experts.gate_up_proj")
    ex = tr.model.model.layers[1].mlp.routed.experts
    E, Fi, D = ex.w1_EFD.shape
    assert gu.shape == (E, 2 * Fi, D)
    before = [u.master.clone() for u in tr.asm.fsdp.units]
    for u in tr.asm.fsdp.units:
        u.master.zero_()
    load_hf_checkpoint(tr, out)
    for a, u in zip(before, tr.asm.fsdp.units):
        assert torch.equal(a[:u.numel], u.master[:u.numel])
    tr.close()


def test_sequence_parallel_matches_one_rank():
    arch = dict(head_dim=16, linear_chunk_size=8)
    base = dict(model_name_or_path="qwen3_5_moe", num_hidden_layers=4)
    ref = run_ranks(1, base_flat(**base), arch=arch)
    got = run_ranks(2, base_flat(data_parallel_shard_size=1, context_parallel_kv_allgather_size=2, **base), arch=arch)
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 5e-5, (ref, got)
    assert max(abs(a - b) for a, b in zip(ref["grad_norm"], got["grad_norm"])) < 5e-4, (ref, got)


def test_a_folder_written_by_save_pretrained_loads_and_gives_the_same_logits(tmp_path):
    """Files as transformers writes them (text decoder under `model.language_model.`, one tensor per expert and
    projection): the preflight accepts the folder, a run names it as model and initial checkpoint, and the loaded model
    reproduces the Hugging Face model's logits."""
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.components.checkpointer import hf_preflight
    theirs = _theirs(_ours())
    folder = str(tmp_path / "hf")
    theirs.save_pretrained(folder, safe_serialization=True)
    rep = hf_preflight.preflight(folder)
    assert rep["ok"] and rep["registered_model"] == "qwen3_5_moe" and rep["expected_tensors"] == rep["stored_tensors"], rep
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path=folder, dump_folder=str(tmp_path / "run"), enable=True, initial_load_path=folder,
                             initial_load_in_hf=True))
    cfg.model.arch_overrides = dict(linear_chunk_size=8)
    tr = Trainer(cfg)
    assert tr.checkpointer.load()
    S = 29
    tok = torch.randint(0, 96, (S,))
    with torch.no_grad():
        ctx = tr.model.build_context(torch.arange(S), AttnMeta.build(torch.tensor([0, S], dtype=torch.int32), causal=True))
        got = tr.model(tok, ctx)
        want = theirs(input_ids=tok[None]).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=2e-4, rtol=1e-4), (got - want).abs().max()
