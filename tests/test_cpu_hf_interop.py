"""Folders as Hugging Face `transformers` writes them (`save_pretrained`): the preflight accepts them, a run names the
folder as its model and initial checkpoint, and the loaded model reproduces the library model's logits. This pins what a
config.json of today's library looks like: `rope_theta` nested in `rope_parameters`, `num_local_experts` for the expert
count, a `dtype` key."""
import pytest
import torch

from caps import require_env

require_env("transformers", "safetensors")

from dist_cases import base_flat  # noqa: E402
from torchllmtuner_b200 import LLMTunerConfig, Trainer  # noqa: E402
from torchllmtuner_b200.components.checkpointer import hf_preflight  # noqa: E402
from torchllmtuner_b200.ops import AttnMeta  # noqa: E402

DENSE = dict(vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
             head_dim=16, tie_word_embeddings=False)


def _case(kind):
    import transformers as T
    if kind == "dense":
        return T.Qwen3ForCausalLM, T.Qwen3Config(**DENSE)
    return T.Qwen3MoeForCausalLM, T.Qwen3MoeConfig(**DENSE, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24,
                                                   norm_topk_prob=(kind == "moe_renormalised"))


@pytest.mark.parametrize("kind", ["dense", "moe", "moe_renormalised"])
def test_qwen3_folder_from_save_pretrained(kind, tmp_path):
    torch.manual_seed(0)
    cls, hf_cfg = _case(kind)
    hf_cfg._attn_implementation = "eager"
    theirs = cls(hf_cfg).eval()
    folder = str(tmp_path / "hf")
    theirs.save_pretrained(folder, safe_serialization=True)
    rep = hf_preflight.preflight(folder)
    assert rep["ok"] and rep["registered_model"] == "qwen3_moe" and rep["expected_tensors"] == rep["stored_tensors"], rep
    assert rep["parameters"] == sum(p.numel() for p in theirs.parameters())
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path=folder, dump_folder=str(tmp_path / "run"), enable=True, initial_load_path=folder,
                             initial_load_in_hf=True))
    tr = Trainer(cfg)
    assert tr.checkpointer.load()
    assert tr.model.config.rope_theta == 10000.0                      # the library's default, not this framework's
    S = 23
    tok = torch.randint(0, 96, (S,))
    with torch.no_grad():
        ctx = tr.model.build_context(torch.arange(S), AttnMeta.build(torch.tensor([0, S], dtype=torch.int32), causal=True))
        got = tr.model(tok, ctx)
        want = theirs(input_ids=tok[None]).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=1e-5), (got - want).abs().max()


def test_preflight_names_an_unknown_model_type(tmp_path):
    (tmp_path / "config.json").write_text('{"model_type": "gpt_oss"}')
    rep = hf_preflight.preflight(str(tmp_path))
    assert not rep["ok"] and "no registered model" in rep["error"] and hf_preflight.main([str(tmp_path)]) == 1


def test_preflight_without_weights_reports_what_it_would_need(tmp_path):
    import json
    _, hf_cfg = _case("moe")
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg.to_dict()))
    rep = hf_preflight.preflight(str(tmp_path))
    assert not rep["ok"] and "no readable weights" in rep["error"] and rep["expected_tensors"] > 0 and rep["registered_model"] == "qwen3_moe"


@pytest.mark.parametrize("name,arch", [("qwen3", dict(head_dim=16)),
                                       ("qwen3_moe", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, head_dim=16)),
                                       ("qwen3_5", dict(head_dim=16, linear_chunk_size=8)),
                                       ("qwen3_5_moe", dict(head_dim=16, linear_chunk_size=8))])
def test_the_library_loads_this_frameworks_export(name, arch, tmp_path):
    """The other direction: `save_hf_checkpoint` output goes through `from_pretrained` and gives this model's logits."""
    import transformers as T
    from torchllmtuner_b200.components.checkpointer.hf import save_hf_checkpoint
    if name == "qwen3_5_moe":
        cls = pytest.importorskip("transformers.models.qwen3_5_moe.modeling_qwen3_5_moe").Qwen3_5MoeForCausalLM
    elif name == "qwen3_5":
        cls = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5").Qwen3_5ForCausalLM
    else:
        cls = T.Qwen3ForCausalLM if name == "qwen3" else T.Qwen3MoeForCausalLM
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path=name, num_hidden_layers=4, dump_folder=str(tmp_path / "run")))
    cfg.model.arch_overrides = arch
    tr = Trainer(cfg)
    tr.train_step()
    out = str(tmp_path / "hf")
    save_hf_checkpoint(tr, out, "float32")
    theirs = cls.from_pretrained(out, attn_implementation="eager", dtype=torch.float32).eval()
    S = 19
    tok = torch.randint(0, 100, (S,))
    with torch.no_grad():
        ctx = tr.model.build_context(torch.arange(S), AttnMeta.build(torch.tensor([0, S], dtype=torch.int32), causal=True))
        got = tr.model(tok, ctx)
        want = theirs(input_ids=tok[None], use_cache=False).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=1e-5), (got - want).abs().max()
    # and back: what the library writes from that model passes the preflight
    back = str(tmp_path / "back")
    theirs.save_pretrained(back, safe_serialization=True)
    rep = hf_preflight.preflight(back)
    assert rep["ok"] and rep["expected_tensors"] == rep["stored_tensors"], rep


@pytest.mark.parametrize("change,word", [(dict(attention_bias=True), "attention_bias"), (dict(hidden_act="gelu"), "hidden_act"),
                                         (dict(rope_parameters={"rope_type": "yarn", "rope_theta": 1e4, "factor": 4.0}), "yarn")])
def test_a_config_that_asks_for_something_unbuilt_is_refused(change, word, tmp_path):
    import json
    from torchllmtuner_b200.config.model_config import ModelConfig
    from torchllmtuner_b200.errors import UnsupportedCombinationError
    from torchllmtuner_b200.models.registry import build_registered_model
    hf = dict(model_type="qwen3", **DENSE)
    hf.update(change)
    (tmp_path / "config.json").write_text(json.dumps(hf))
    with pytest.raises(UnsupportedCombinationError, match=word):
        with torch.device("meta"):
            build_registered_model(ModelConfig(model_name_or_path=str(tmp_path)))


def test_published_style_config_files_build_the_registered_architectures(tmp_path):
    """config.json as the Qwen3-8B and Qwen3-30B-A3B repositories carry it (top-level `rope_theta`, `num_experts`, null
    `rope_scaling`): the same parameter names and shapes as the registry's own entries."""
    import json
    from torchllmtuner_b200.config.model_config import ModelConfig
    from torchllmtuner_b200.models.registry import build_registered_model
    common = {"attention_bias": False, "attention_dropout": 0.0, "head_dim": 128, "hidden_act": "silu", "max_position_embeddings": 40960,
              "rms_norm_eps": 1e-06, "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None, "tie_word_embeddings": False,
              "torch_dtype": "bfloat16", "use_cache": True, "use_sliding_window": False, "vocab_size": 151936}
    dense = dict(common, architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, intermediate_size=12288,
                 num_attention_heads=32, num_hidden_layers=36, num_key_value_heads=8, max_window_layers=36)
    moe = dict(common, architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=2048, intermediate_size=6144,
               moe_intermediate_size=768, norm_topk_prob=True, num_attention_heads=32, num_experts=128, num_experts_per_tok=8,
               num_hidden_layers=48, num_key_value_heads=4, decoder_sparse_step=1, mlp_only_layers=[], output_router_logits=False,
               router_aux_loss_coef=0.001)
    for hf, preset, params in ((dense, "qwen3_8b", 8190735360), (moe, "qwen3_30b_a3b", 30532122624)):
        d = tmp_path / preset
        d.mkdir()
        (d / "config.json").write_text(json.dumps(hf))
        with torch.device("meta"):
            a = build_registered_model(ModelConfig(model_name_or_path=str(d)))
            b = build_registered_model(ModelConfig(model_name_or_path=preset))
        assert sum(p.numel() for p in a.parameters()) == params and a.config.rope_theta == 1000000
        assert {n: tuple(p.shape) for n, p in a.named_parameters()} == {n: tuple(p.shape) for n, p in b.named_parameters()}


def test_grouped_biased_sigmoid_routing_matches_the_librarys_deepseek_v3_router():
    """Group-limited top-k with the aux-loss-free bias (sigmoid scores, groups ranked by their two best biased scores,
    weights from the unbiased scores, renormalised and scaled): same experts and weights as `DeepseekV3MoE`."""
    import transformers as T
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as m
    from torchllmtuner_b200.models.moe.routing import TokenChoiceTopKRouter
    torch.manual_seed(0)
    cfg = T.DeepseekV3Config(hidden_size=32, n_routed_experts=16, num_experts_per_tok=4, n_group=4, topk_group=2, norm_topk_prob=True,
                             routed_scaling_factor=2.5, moe_intermediate_size=8, n_shared_experts=1, num_hidden_layers=1,
                             intermediate_size=16, vocab_size=32, num_attention_heads=2)
    moe = m.DeepseekV3MoE(cfg)
    with torch.no_grad():
        torch.nn.init.normal_(moe.gate.weight, std=1.0)
        moe.gate.e_score_correction_bias.copy_(torch.randn(16) * 0.2)
        x = torch.randn(40, 32)
        idx_hf, w_hf = moe.route_tokens_to_experts(moe.gate(x))
        ours = TokenChoiceTopKRouter(32, 16, 4, score_fn="sigmoid", norm_topk_prob=True, route_scale=2.5, num_groups=4, topk_groups=2)
        ours.gate.weight.copy_(moe.gate.weight)
        w, idx, counts, _ = ours(x, expert_bias=moe.gate.e_score_correction_bias)
    a = {(t, int(e)): float(v) for t in range(40) for e, v in zip(idx_hf[t], w_hf[t])}
    b = {(t, int(e)): float(v) for t in range(40) for e, v in zip(idx[t], w[t])}
    assert a.keys() == b.keys() and max(abs(a[k] - b[k]) for k in a) < 1e-6
    assert float(counts.sum()) == 40 * 4


def test_latent_attention_matches_the_librarys_multi_head_latent_attention():
    """Low-rank queries, one compressed key/value row per token with a shared positional part, per-head expansion: Kimi's
    latent attention against `DeepseekV3Attention` with the rotation switched off (cos = 1, sin = 0; this family carries
    positions in its delta-rule layers)."""
    import transformers as T
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as m
    from torchllmtuner_b200.models import kimi_k3 as km
    torch.manual_seed(0)
    D, H, dn, dr, dv, ql, kvl, S = 64, 4, 16, 8, 12, 24, 20, 21
    cfg = T.DeepseekV3Config(hidden_size=D, num_attention_heads=H, num_key_value_heads=H, qk_nope_head_dim=dn, qk_rope_head_dim=dr,
                             v_head_dim=dv, q_lora_rank=ql, kv_lora_rank=kvl, num_hidden_layers=1, vocab_size=32, intermediate_size=32,
                             n_routed_experts=4, moe_intermediate_size=8, attention_bias=False, rms_norm_eps=1e-6)
    cfg._attn_implementation = "eager"
    theirs = m.DeepseekV3Attention(cfg, layer_idx=0).eval()
    kc = km.KimiConfig(vocab_size=32, hidden_size=D, intermediate_size=32, num_hidden_layers=4, num_attention_heads=H, num_key_value_heads=H,
                       head_dim=16, q_lora_rank=ql, kv_lora_rank=kvl, qk_nope_head_dim=dn, qk_rope_head_dim=dr, v_head_dim=dv,
                       mla_use_output_gate=False, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=8, linear_heads=2,
                       linear_head_dim=8)
    ours = km.KimiLatentAttention(kc).eval()
    with torch.no_grad():
        for p in theirs.parameters():
            torch.nn.init.normal_(p, std=0.3) if p.dim() > 1 else torch.nn.init.normal_(p, mean=1.0, std=0.2)
        for n in ("q_a_proj", "q_b_proj", "kv_a_proj_with_mqa", "kv_b_proj", "o_proj"):
            getattr(ours, n).weight.copy_(getattr(theirs, n).weight)
        ours.q_a_layernorm.weight.copy_(theirs.q_a_layernorm.weight)
        ours.kv_a_layernorm.weight.copy_(theirs.kv_a_layernorm.weight)
        x = torch.randn(S, D)
        mask = torch.full((S, S), float("-inf")).triu(1)[None, None]
        want = theirs(x[None], position_embeddings=(torch.ones(1, S, dr), torch.zeros(1, S, dr)), attention_mask=mask)[0][0]
        ctx = km.KimiContext(None, None, AttnMeta.build(torch.tensor([0, S], dtype=torch.int32)), None, torch.arange(S))
        got = ours(x, ctx)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-5), (got - want).abs().max()


VIT = dict(depth=2, hidden_size=32, intermediate_size=64, num_heads=2, num_position_embeddings=64, patch_size=4, temporal_patch_size=2,
           in_channels=3, spatial_merge_size=2)


def test_vision_tower_matches_the_librarys_qwen3_5_vision_model():
    """Same parameter names and shapes (a plain `load_state_dict`), same output rows for images and a two-frame video in
    the processors' merge-block order; patches given row-major (this framework's data pipeline) land on the same rows."""
    hf = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5VisionConfig
    from torchllmtuner_b200.models.qwen_vit import QwenViTConfig, QwenViTTower, merge_block_order
    torch.manual_seed(0)
    hcfg = Qwen3_5VisionConfig(**VIT, out_hidden_size=48)
    hcfg._attn_implementation = "eager"
    theirs = hf.Qwen3_5VisionModel(hcfg).eval()
    with torch.no_grad():
        for p in theirs.parameters():
            torch.nn.init.normal_(p, std=0.2)
    ours = QwenViTTower(QwenViTConfig(**VIT, out_hidden_size=48, patch_order="merge_blocks")).eval()
    ours.load_state_dict(theirs.state_dict())
    grids = [(1, 4, 6), (2, 2, 4), (1, 8, 8)]
    N = sum(t * h * w for t, h, w in grids)
    x = torch.randn(N, 3 * 2 * 4 * 4)
    with torch.no_grad():
        want = theirs(x, grid_thw=torch.tensor(grids)).pooler_output
        got = ours(x, grids)
        assert got.shape == want.shape == (N // 4, 48) and torch.allclose(got, want, atol=1e-5), (got - want).abs().max()
        ours.config.patch_order = "row_major"
        inv = torch.empty(N, dtype=torch.long)
        inv[merge_block_order(grids, 2)] = torch.arange(N)
        assert torch.equal(ours(x[inv], grids), got)
        # an image row without the temporal axis is the frame repeated over it
        one = torch.randn(16, 3 * 4 * 4)
        both = one.view(16, 3, 1, 16).expand(16, 3, 2, 16).reshape(16, -1)
        assert torch.allclose(ours(one, [(1, 4, 4)]), ours(both, [(1, 4, 4)]), atol=1e-6)


def test_vision_language_folder_in_the_published_layout_loads(tmp_path):
    """Tensors named as the library's vision-language model holds them (`model.language_model.*`, `model.visual.*`,
    `lm_head.weight`): the `_vl` model with the published tower imports them, and its tower and text decoder compute what
    the library's do."""
    hf = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    from safetensors.torch import save_file
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5Config
    torch.manual_seed(0)
    txt = dict(vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
               head_dim=32, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=24,
               linear_conv_kernel_dim=4, rms_norm_eps=1e-6,
               rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5, "mrope_section": [4, 2, 2],
                                "mrope_interleaved": True})
    cfg = Qwen3_5Config(text_config=txt, vision_config=dict(VIT, out_hidden_size=64), image_token_id=90, video_token_id=91,
                        vision_start_token_id=92, vision_end_token_id=93, tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    cfg.text_config._attn_implementation = "eager"
    cfg.vision_config._attn_implementation = "eager"
    theirs = hf.Qwen3_5ForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in theirs.named_parameters():
            if "visual" in n:
                torch.nn.init.normal_(p, std=0.2)
    folder = tmp_path / "hf"
    folder.mkdir()
    save_file({k: v.contiguous() for k, v in theirs.state_dict().items()}, str(folder / "model.safetensors"))
    import json
    (folder / "config.json").write_text(json.dumps(cfg.to_dict()))
    c = LLMTunerConfig()      # the folder names the model; asking for the tower turns it into the vision-language entry
    c.apply_flat(base_flat(model_name_or_path=str(folder), dump_folder=str(tmp_path / "run"), enable=True, initial_load_path=str(folder),
                           initial_load_in_hf=True))
    c.model.arch_overrides = dict(vision_tower="qwen3_5", vision=dict(patch_order="merge_blocks"), linear_chunk_size=8)
    tr = Trainer(c)
    assert tr.model.state_format == "qwen3_5_vl" and tr.model.image_token_id == 90 and tr.model.visual.config.hidden_size == 32
    assert tr.checkpointer.load()
    grids = [(1, 4, 4), (1, 2, 6)]
    patches = torch.randn(sum(t * h * w for t, h, w in grids), 3 * 2 * 4 * 4)
    S = 17
    tok = torch.randint(0, 80, (S,))
    with torch.no_grad():
        rows = tr.model.visual(patches, grids)
        want_rows = theirs.model.visual(patches, grid_thw=torch.tensor(grids)).pooler_output
        assert torch.allclose(rows.float(), want_rows, atol=1e-5), (rows - want_rows).abs().max()
        ctx = tr.model.build_context(torch.arange(S), AttnMeta.build(torch.tensor([0, S], dtype=torch.int32), causal=True))
        got = tr.model(tok, ctx)
        want = theirs(input_ids=tok[None], use_cache=False).logits[0]
        assert torch.allclose(got.float(), want, atol=2e-4, rtol=1e-4), (got - want).abs().max()
        # two images between words: placeholders, three-axis positions and the merged rows land where the library puts them
        from torchllmtuner_b200.datasets.multimodal import build_mrope_positions, insert_vision_placeholders
        words = torch.randint(0, 80, (20,)).tolist()
        ids = insert_vision_placeholders(words[:5] + [92, 90, 93] + words[5:12] + [92, 90, 93] + words[12:], 90, grids)
        pos = build_mrope_positions(ids, 90, grids)
        ids_t = torch.tensor(ids)
        kinds = (ids_t[None] == 90).int()
        their_pos = theirs.model.get_rope_index(ids_t[None], mm_token_type_ids=kinds, image_grid_thw=torch.tensor(grids))[0]
        assert torch.equal(their_pos[:, 0], pos)
        ctx = tr.model.build_context(pos, AttnMeta.build(torch.tensor([0, len(ids)], dtype=torch.int32), causal=True))
        got = tr.model(ids_t, ctx, patches=patches, grids=grids)
        want = theirs(input_ids=ids_t[None], pixel_values=patches, image_grid_thw=torch.tensor(grids), mm_token_type_ids=kinds,
                      use_cache=False).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=2e-4, rtol=1e-4), (got - want).abs().max()


def test_the_library_loads_a_vision_language_export(tmp_path):
    """`save_hf_checkpoint` of the `_vl` model with the published tower: `from_pretrained` builds the library's
    vision-language model from the written config.json and tensors, and a forward with an image gives this model's logits."""
    hf = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    from torchllmtuner_b200.components.checkpointer.hf import save_hf_checkpoint
    from torchllmtuner_b200.datasets.multimodal import build_mrope_positions, insert_vision_placeholders
    c = LLMTunerConfig()
    c.apply_flat(base_flat(model_name_or_path="qwen3_5_vl", vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                           num_attention_heads=4, num_key_value_heads=2, dump_folder=str(tmp_path / "run")))
    c.model.arch_overrides = dict(head_dim=32, linear_chunk_size=8, image_token_id=90, vision_tower="qwen3_5",
                                  vision=dict(VIT, patch_order="merge_blocks"))
    tr = Trainer(c)
    out = str(tmp_path / "hf")
    save_hf_checkpoint(tr, out, "float32")
    theirs = hf.Qwen3_5ForConditionalGeneration.from_pretrained(out, attn_implementation="eager", dtype=torch.float32).eval()
    rep = hf_preflight.preflight(out, vision=True)           # every tensor of the folder, the tower's included
    assert rep["ok"] and rep["registered_model"] == "qwen3_5_vl" and rep["unused_count"] == 0 and rep["expected_tensors"] == rep["stored_tensors"], rep
    text_only = hf_preflight.preflight(out)                  # as a text decoder: the tower's tensors are simply not read
    assert text_only["ok"] and text_only["registered_model"] == "qwen3_5" and text_only["unused_count"] > 0
    grids = [(1, 4, 4)]
    torch.manual_seed(1)
    patches = torch.randn(16, 3 * 2 * 4 * 4)
    words = torch.randint(0, 80, (12,)).tolist()
    ids = insert_vision_placeholders(words[:5] + [90] + words[5:], 90, grids)
    pos = build_mrope_positions(ids, 90, grids)
    ids_t = torch.tensor(ids)
    with torch.no_grad():
        ctx = tr.model.build_context(pos, AttnMeta.build(torch.tensor([0, len(ids)], dtype=torch.int32), causal=True))
        got = tr.model(ids_t, ctx, patches=patches, grids=grids)
        want = theirs(input_ids=ids_t[None], pixel_values=patches, image_grid_thw=torch.tensor(grids),
                      mm_token_type_ids=(ids_t[None] == 90).int(), use_cache=False).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=2e-4, rtol=1e-4), (got - want).abs().max()


def test_moe_vision_language_folder_builds_loads_and_matches(tmp_path):
    """Qwen3.5-MoE with its tower, tensors as the library's model holds them (packed experts under
    `model.language_model.`): preflight with the tower, build from the folder, load, and a forward with an image."""
    hf = pytest.importorskip("transformers.models.qwen3_5_moe.modeling_qwen3_5_moe")
    import json
    from safetensors.torch import save_file
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeConfig
    from torchllmtuner_b200.datasets.multimodal import build_mrope_positions, insert_vision_placeholders
    torch.manual_seed(0)
    txt = dict(vocab_size=96, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=4,
               num_experts_per_tok=2, moe_intermediate_size=24, shared_expert_intermediate_size=40, linear_num_value_heads=4,
               linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=24, linear_conv_kernel_dim=4, rms_norm_eps=1e-6,
               rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5, "mrope_section": [4, 2, 2],
                                "mrope_interleaved": True})
    cfg = Qwen3_5MoeConfig(text_config=txt, vision_config=dict(VIT, out_hidden_size=64), image_token_id=90, video_token_id=91,
                           vision_start_token_id=92, vision_end_token_id=93, tie_word_embeddings=False)
    for part in (cfg, cfg.text_config, cfg.vision_config):
        part._attn_implementation = "eager"
    theirs = hf.Qwen3_5MoeForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in theirs.named_parameters():
            if "visual" in n:
                torch.nn.init.normal_(p, std=0.2)
    folder = tmp_path / "hf"
    folder.mkdir()
    save_file({k: v.contiguous() for k, v in theirs.state_dict().items()}, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(cfg.to_dict()))
    rep = hf_preflight.preflight(str(folder), vision=True)
    assert rep["ok"] and rep["registered_model"] == "qwen3_5_moe_vl" and rep["unused_count"] == 0, rep
    c = LLMTunerConfig()
    c.apply_flat(base_flat(model_name_or_path=str(folder), dump_folder=str(tmp_path / "run"), enable=True, initial_load_path=str(folder),
                           initial_load_in_hf=True))
    c.model.arch_overrides = dict(vision_tower="qwen3_5", vision=dict(patch_order="merge_blocks"), linear_chunk_size=8)
    tr = Trainer(c)
    assert tr.checkpointer.load() and tr.model.config.num_experts == 4
    grids = [(1, 4, 4)]
    patches = torch.randn(16, 96)
    words = torch.randint(0, 80, (14,)).tolist()
    ids = insert_vision_placeholders(words[:6] + [90] + words[6:], 90, grids)
    pos = build_mrope_positions(ids, 90, grids)
    ids_t = torch.tensor(ids)
    with torch.no_grad():
        ctx = tr.model.build_context(pos, AttnMeta.build(torch.tensor([0, len(ids)], dtype=torch.int32), causal=True))
        got = tr.model(ids_t, ctx, patches=patches, grids=grids)
        want = theirs(input_ids=ids_t[None], pixel_values=patches, image_grid_thw=torch.tensor(grids),
                      mm_token_type_ids=(ids_t[None] == 90).int(), use_cache=False).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=2e-4, rtol=1e-4), (got - want).abs().max()


def test_packed_documents_match_the_library_run_with_a_block_diagonal_mask(tmp_path):
    """Three documents packed into one row: document cut points and per-document positions here, an explicit
    block-diagonal causal mask and the same position ids in the library."""
    import transformers as T
    torch.manual_seed(0)
    hf_cfg = T.Qwen3MoeConfig(**DENSE, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, norm_topk_prob=True)
    hf_cfg._attn_implementation = "eager"
    theirs = T.Qwen3MoeForCausalLM(hf_cfg).eval()
    folder = str(tmp_path / "hf")
    theirs.save_pretrained(folder, safe_serialization=True)
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path=folder, dump_folder=str(tmp_path / "run"), enable=True, initial_load_path=folder,
                             initial_load_in_hf=True))
    tr = Trainer(cfg)
    assert tr.checkpointer.load()
    lens = [7, 12, 5]
    S = sum(lens)
    tok = torch.randint(0, 96, (S,))
    pos = torch.cat([torch.arange(n) for n in lens])
    doc = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens))
    allowed = (doc[:, None] == doc[None, :]) & (torch.arange(S)[None, :] <= torch.arange(S)[:, None])
    mask = torch.zeros(S, S).masked_fill(~allowed, float("-inf"))[None, None]
    with torch.no_grad():
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
        got = tr.model(tok, tr.model.build_context(pos, AttnMeta.build(cu, causal=True)))
        want = theirs(input_ids=tok[None], position_ids=pos[None], attention_mask=mask, use_cache=False).logits[0]
    tr.close()
    assert torch.allclose(got.float(), want, atol=1e-5), (got - want).abs().max()


def test_a_training_step_has_the_librarys_loss_and_gradient_norm(tmp_path):
    """One optimizer step over two accumulated micro-batches through the Trainer (flat gradient buffers, sum / global
    token count, norm for clipping) against `loss.backward()` of the library's model on the same rows."""
    import transformers as T
    torch.manual_seed(0)
    hf_cfg = T.Qwen3MoeConfig(**DENSE, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, norm_topk_prob=True,
                              router_aux_loss_coef=0.0)
    hf_cfg._attn_implementation = "eager"
    theirs = T.Qwen3MoeForCausalLM(hf_cfg).train()
    folder = str(tmp_path / "hf")
    theirs.save_pretrained(folder, safe_serialization=True)
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path=folder, dump_folder=str(tmp_path / "run"), enable=True, initial_load_path=folder,
                             initial_load_in_hf=True, gradient_accumulation_steps=2, global_batch_size=4))
    tr = Trainer(cfg)
    assert tr.checkpointer.load()
    it = iter(tr.dataloader)
    rows = torch.cat([next(it)["input"] for _ in range(2)])
    tr.dataloader.cursor = 0
    step = tr.train_step()
    ours_after = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    tr.close()
    out = theirs(input_ids=rows, labels=rows)
    out.loss.backward()
    norm = torch.sqrt(sum(p.grad.float().square().sum() for p in theirs.parameters() if p.grad is not None))
    assert abs(step.loss - out.loss.item()) < 1e-5 and abs(step.grad_norm - norm.item()) < 1e-5 * max(1.0, norm.item())
    # the update: clip to max_norm, AdamW with the step's learning rate (decoupled weight decay on every tensor, like here)
    t, o = cfg.training, cfg.optimizer
    before = theirs.lm_head.weight.detach().clone()
    torch.nn.utils.clip_grad_norm_(theirs.parameters(), t.max_norm)
    torch.optim.AdamW(theirs.parameters(), lr=step.lr, betas=tuple(o.betas), eps=o.eps, weight_decay=o.weight_decay).step()
    moved = (theirs.lm_head.weight - before).abs().max().item()
    assert moved > 0 and norm.item() > t.max_norm                                     # the clip was active
    for name in ("lm_head.weight", "model.layers.1.self_attn.q_proj.weight", "model.norm.weight"):
        want = dict(theirs.named_parameters())[name]
        assert torch.allclose(ours_after[name], want, atol=moved * 1e-3), (name, (ours_after[name] - want).abs().max(), moved)
