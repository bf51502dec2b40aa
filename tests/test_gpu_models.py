"""Vision tower, vision-language wrapper and the delta-attention families on the sm_100a kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_vision_tower_matches_the_fp32_statement_and_trains():
    from torchllmtuner_b200.models.vision import VisionConfig, VisionTower
    dev = torch.device("cuda")
    cfg = VisionConfig(patch_size=14, hidden_size=256, intermediate_size=512, depth=2, num_heads=2, out_hidden_size=256)
    ref = VisionTower(cfg)
    ref.initialize_parameters(0)
    gpu = VisionTower(cfg, dtype=torch.bfloat16, device=dev)
    gpu.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
    grids = [(1, 8, 12), (1, 4, 4)]
    patches = torch.rand(sum(t * h * w for t, h, w in grids), cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = ref(patches, grids)
    got = gpu(patches.to(dev), grids)
    assert got.shape == want.shape == (24 + 4, 256)
    assert (want - got.float().cpu()).abs().max().item() < 0.03 * want.abs().max().item() + 1e-2
    got.float().square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in gpu.parameters())


def test_vision_language_wrapper_runs_forward_and_backward():
    from torchllmtuner_b200.datasets.multimodal import build_mrope_positions, insert_vision_placeholders
    from torchllmtuner_b200.models.qwen3 import Qwen3Config, Qwen3ForCausalLM
    from torchllmtuner_b200.models.vision import VisionConfig, VisionLanguageModel
    from torchllmtuner_b200.ops.attn_meta import AttnMeta
    from torchllmtuner_b200.ops.cuda_ext import check_status
    dev = torch.device("cuda")
    vcfg = VisionConfig(patch_size=14, hidden_size=256, intermediate_size=512, depth=2, num_heads=2, out_hidden_size=256)
    tcfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=128, tie_word_embeddings=False)
    vlm = VisionLanguageModel(Qwen3ForCausalLM(tcfg, dtype=torch.bfloat16, device=dev), vcfg, image_token_id=500,
                              dtype=torch.bfloat16, device=dev)
    vlm.initialize_parameters(0)
    grids = [(1, 8, 12), (1, 4, 4)]
    g = torch.Generator().manual_seed(2)
    patches = torch.rand(sum(t * h * w for t, h, w in grids), vcfg.patch_dim, generator=g)
    words = torch.randint(0, 400, (120,), generator=g).tolist()
    ids = insert_vision_placeholders(words[:40] + [500] + words[40:80] + [500] + words[80:], 500, grids)
    pos = build_mrope_positions(ids, 500, grids).to(dev)
    ids = torch.tensor(ids, device=dev)
    ctx = vlm.build_context(pos, AttnMeta.build(torch.tensor([0, ids.numel()]), device=dev))
    logits = vlm(ids, ctx, patches=patches.to(dev), grids=grids)
    loss = torch.nn.functional.cross_entropy(logits.float(), torch.roll(ids, -1))
    loss.backward()
    assert 5.0 < loss.item() < 8.0
    assert all(p.grad is None or torch.isfinite(p.grad).all() for p in vlm.parameters())
    assert all(p.grad is not None for p in vlm.visual.parameters())
    check_status("vision-language wrapper")


@pytest.mark.parametrize("family", ["qwen3_5", "kimi_linear", "kimi_k3", "deepseek_v4", "hybrid_gdn", "hybrid_kda_mla"])
def test_delta_attention_and_latent_attention_families_train(family):
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    cfg = LLMTunerConfig()
    cfg.apply_flat(dict(model_name_or_path=family, vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, global_batch_size=2, max_seq_len=1024, steps=3, seed=0,
                        dump_folder="/tmp/llmt_gpu_families", deterministic=False))
    cfg.model.arch_overrides = dict(head_dim=128, delta_heads=4, delta_head_dim=64, kv_lora_rank=128, qk_rope_dim=64)
    tr = Trainer(cfg)
    try:
        losses = []
        for _ in range(3):
            tr.dataloader.cursor = 0
            losses.append(tr.train_step().loss)
    finally:
        tr.close()
    assert losses[-1] < losses[0] - 0.5, losses


def test_graphed_block_replays_with_the_current_context():
    """A decoder block captured in a CUDA graph: a later call with other positions (same document layout) replays the graph
    on ITS rotary tables; another document layout is captured anew. Every output equals the plain block's."""
    from torchllmtuner_b200.models.qwen3 import Qwen3Config, Qwen3ForCausalLM
    from torchllmtuner_b200.ops.attn_meta import AttnMeta
    from torchllmtuner_b200.ops.cuda_ext import check_status
    from torchllmtuner_b200.parallel.graph_capture import GraphedInference
    dev = torch.device("cuda")
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=1, head_dim=128, tie_word_embeddings=False)
    m = Qwen3ForCausalLM(cfg, dtype=torch.bfloat16, device=dev)
    m.initialize_parameters(0)
    m.eval()
    blk = m.model.layers[0]
    g = GraphedInference(blk).eval()
    torch.manual_seed(0)
    with torch.no_grad():
        for n, (off, cu) in enumerate([(0, [0, 256]), (7, [0, 256]), (0, [0, 100, 256]), (3, [0, 100, 256])]):
            x = torch.randn(256, 256, device=dev).bfloat16()
            ctx = m.build_context(torch.arange(256, device=dev) + off, AttnMeta.build(torch.tensor(cu), device=dev))
            want = blk(x, ctx)
            got = g(x, ctx)
            assert torch.equal(got, want), n
    assert g.captures == 2
    torch.cuda.synchronize()
    check_status("graphed block")
