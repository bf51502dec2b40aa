"""Multimodal data path and a vision-language model under the Trainer: frame sampling, patch grids, placeholder
expansion and label masking, three-axis positions, packing, collation, the synthetic loader's determinism and resume,
and training a tower + decoder through the public Trainer on one and on two FSDP ranks."""
import pytest
import torch

from dist_cases import base_flat, run_ranks
from torchllmtuner_b200.datasets import multimodal_pipeline as mp
from torchllmtuner_b200.datasets.contracts import IGNORE_INDEX


def test_frame_sampling_respects_rate_budget_and_temporal_patch():
    spec = mp.VisionSpec(video_fps=2.0, video_min_frames=4, video_max_frames=8, temporal_patch_size=2)
    idx = mp.sample_frame_indices(60, 30.0, spec)        # 2 s at 2 fps -> 4 frames (the minimum)
    assert len(idx) == 4 and idx[0] == 0 and idx[-1] == 59 and idx == sorted(idx)
    assert len(mp.sample_frame_indices(3000, 30.0, spec)) == 8                  # capped by the budget
    assert len(mp.sample_frame_indices(5, 30.0, spec)) == 4                     # 5 frames -> 4 (multiple of 2)
    with pytest.raises(ValueError):
        mp.sample_frame_indices(1, 30.0, spec)


def test_image_and_video_patches_follow_the_pixel_budget():
    spec = mp.VisionSpec(patch_size=14, merge_size=2, max_pixels=14 * 14 * 4 * 16, min_pixels=56 * 56)
    p, g = mp.image_to_patches(torch.rand(3, 300, 500), spec)
    assert g[0] == 1 and g[1] % 2 == 0 and g[2] % 2 == 0 and g[1] * g[2] * 196 <= spec.max_pixels
    assert p.shape == (g[1] * g[2], 3 * 14 * 14)
    p, g = mp.video_to_patches(torch.rand(9, 3, 80, 120), 4.0, spec)
    assert g[0] == 2 and p.shape[0] == g[0] * g[1] * g[2]


def test_sample_expands_placeholders_masks_labels_and_builds_positions():
    spec = mp.VisionSpec()
    img = (torch.rand(4 * 6, 588), (1, 4, 6))             # 4x6 patches -> 2x3 merged rows
    s = mp.build_sample([5, 6, 99, 7, 8, 9], [img], placeholder_id=99, spec=spec, start_id=90, end_id=91, prompt_len=4)
    assert s.tokens == [5, 6, 90] + [99] * 6 + [91, 7, 8, 9]
    assert s.labels == [IGNORE_INDEX] * 10 + [IGNORE_INDEX, 8, 9][0:0] + [IGNORE_INDEX, 8, 9] or s.labels[-2:] == [8, 9]
    assert s.labels[:10] == [IGNORE_INDEX] * 10 and s.labels[10] == IGNORE_INDEX and s.labels[-2:] == [8, 9]
    pos = s.positions
    assert pos.shape == (3, 13)
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3
    assert pos[0, 3:9].tolist() == [3] * 6 and pos[1, 3:9].tolist() == [3, 3, 3, 4, 4, 4] and pos[2, 3:9].tolist() == [3, 4, 5] * 2
    assert pos[:, 9].tolist() == [6, 6, 6]                                     # continues after the largest position used
    with pytest.raises(ValueError):
        mp.build_sample([5, 99, 99], [img], placeholder_id=99, spec=spec)


def test_packing_keeps_samples_whole_and_collation_builds_documents():
    spec = mp.VisionSpec()
    mk = lambda n, k: mp.build_sample(list(range(1, n + 1)) + [99] * k, [(torch.rand(4, 588), (1, 2, 2))] * k, placeholder_id=99, spec=spec)  # noqa: E731
    a, b, c, big = mk(10, 1), mk(7, 0), mk(12, 2), mk(40, 0)
    rows, left, dropped = mp.pack_samples([a, big, b, c], seq_len=20, rows=2)
    assert dropped == 1 and not left
    assert [len(r.samples) for r in rows] == [2, 1] and rows[0].used == len(a) + len(b)
    batch = mp.collate_rows(rows, 20, pad_id=0)
    assert batch["input"].shape == (2, 20) and batch["positions"].shape == (3, 2, 20)
    assert batch["cu_seqlens"].tolist() == [0, 11, 18, 20, 34, 40]
    assert batch["patches"].shape == (12, 588) and len(batch["grids"]) == 3
    lab = batch["labels"]
    assert lab[0, 10] == IGNORE_INDEX and lab[0, 17] == IGNORE_INDEX and (lab[0, 18:] == IGNORE_INDEX).all()
    assert lab[0, 0] == 2 and lab[0, 11] == 2                               # shifted inside each document
    assert batch["num_valid_tokens"] == int((lab != IGNORE_INDEX).sum())


def test_synthetic_loader_is_deterministic_disjoint_and_resumable():
    kw = dict(vocab_size=300, image_token_id=299, global_batch=4, seq_len=256, seed=3, rows_per_rank=1, dp_degree=2,
              spec=mp.VisionSpec(max_pixels=14 * 14 * 4 * 8, min_pixels=28 * 28 * 4))
    a0, a1 = mp.SyntheticMultimodalLoader(dp_rank=0, **kw), mp.SyntheticMultimodalLoader(dp_rank=1, **kw)
    x0, x1 = next(a0), next(a1)
    assert not torch.equal(x0["input"], x1["input"])
    assert (x0["input"] == 299).sum() == sum(mp.calculate_vision_tokens(g) for g in x0["grids"])
    assert x0["patches"].shape[0] == sum(t * h * w for t, h, w in x0["grids"])
    again = mp.SyntheticMultimodalLoader(dp_rank=0, **kw)
    assert torch.equal(next(again)["input"], x0["input"])
    second = next(a0)
    resumed = mp.SyntheticMultimodalLoader(dp_rank=0, **kw)
    resumed.load_state_dict({**a0.state_dict(), "cursor": 1})
    assert torch.equal(next(resumed)["input"], second["input"])


VL = dict(model_name_or_path="qwen3_5_vl", dataset="random_multimodal", vocab_size=320, hidden_size=64, num_hidden_layers=4,
          num_attention_heads=2, num_key_value_heads=2, max_seq_len=192, global_batch_size=2, learning_rate=3e-3, mm_max_pixels=14 * 14 * 4 * 8)
VL_ARCH = dict(head_dim=32, vision=dict(hidden_size=64, intermediate_size=128, depth=2, num_heads=2))


def test_vision_language_model_trains_through_the_trainer(tmp_path):
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(dump_folder=str(tmp_path), steps=6, **VL))
    cfg.model.arch_overrides = dict(VL_ARCH)
    tr = Trainer(cfg)
    assert tr.model.image_token_id == 319 and any(n.startswith("visual.") for n, _ in tr.model.named_parameters())
    names = set(tr.asm.layout.state_names.values())
    assert "visual.merger.fc2.weight" in names and "text.model.layers.0.self_attn.in_proj_qkv.weight" in names
    before = tr.model.visual.merger.fc2.weight.detach().clone()
    losses = []
    for _ in range(6):
        tr.dataloader.cursor = 0
        losses.append(tr.train_step().loss)
    assert losses[-1] < losses[0] - 0.3, losses
    assert not torch.equal(before, tr.model.visual.merger.fc2.weight)           # the tower trains with the decoder
    tr.checkpointer  # noqa: B018
    tr.close()


def test_vision_language_model_on_two_fsdp_ranks_matches_one():
    ref = run_ranks(1, base_flat(**VL), arch=VL_ARCH, steps=3)
    got = run_ranks(2, base_flat(data_parallel_shard_size=2, **VL), arch=VL_ARCH, steps=3)
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 5e-5, (ref, got)


# ------------------------------------------------------------------------------------------ MoonViT (Kimi-K3's tower)
def test_moonvit_pieces_match_their_restatements():
    import torch.nn.functional as F
    from torchllmtuner_b200.models import moonvit as mv
    cfg = mv.MoonViTConfig(hidden_size=32, intermediate_size=64, depth=1, num_heads=2, out_hidden_size=24, pos_emb_height=4, pos_emb_width=4)
    tower = mv.MoonViTTower(cfg, dtype=torch.float32)
    tower.initialize_parameters(seed=2)
    grids = [(1, 4, 4), (2, 2, 6)]
    # position table: the learned table as is at its own size, bicubic elsewhere, plus the frame code for clips
    tab = tower.position_table(grids, torch.float32)
    assert torch.equal(tab[:16], tower.pos_emb.flatten(0, 1))
    want = F.interpolate(tower.pos_emb.permute(2, 0, 1)[None], size=(2, 6), mode="bicubic")[0].permute(1, 2, 0).flatten(0, 1)
    code = mv.time_code(32, 4)
    assert torch.allclose(tab[16:28], want + code[0]) and torch.allclose(tab[28:40], want + code[1])
    assert torch.allclose(code[1, :16], torch.sin(1.0 / 10000 ** (torch.arange(16) / 16.0)))
    # rotary pairs: even pairs turn with the column, odd pairs with the row; equal to a complex multiplication
    ang = mv.grid_pair_angles([(1, 2, 3)], 8, 10000.0)
    f = 1.0 / (10000.0 ** (torch.arange(0, 8, 4) / 8))
    assert torch.allclose(ang[4], torch.stack((1 * f, 1 * f), -1).flatten())          # patch (row 1, col 1)
    assert torch.allclose(ang[2], torch.stack((2 * f, 0 * f), -1).flatten())          # patch (row 0, col 2)
    x = torch.randn(6, 2, 8)
    z = torch.view_as_complex(x.view(6, 2, 4, 2).contiguous()) * torch.polar(torch.ones(6, 4), ang)[:, None, :]
    assert torch.allclose(mv.rotate_pairs(x, ang), torch.view_as_real(z).flatten(-2), atol=1e-6)
    # merger: mean over frames, then 2 x 2 neighbourhoods in row-major order of the merged grid
    h = torch.randn(16 + 24, 32)
    merged = tower.merge(h, grids)
    assert merged.shape == (4 + 3, 4, 32)
    clip = h[16:].view(2, 2, 6, 32).mean(0)
    assert torch.allclose(merged[4 + 1], torch.stack((clip[0, 2], clip[0, 3], clip[1, 2], clip[1, 3])))
    out = tower(torch.rand(40, cfg.patch_dim), grids)
    assert out.shape == (7, 24) and torch.isfinite(out).all()


def test_kimi_k3_with_moonvit_trains_through_the_trainer(tmp_path):
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(dump_folder=str(tmp_path), steps=5, model_name_or_path="kimi_k3_vl", dataset="random_multimodal", vocab_size=320,
                             hidden_size=64, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=2, max_seq_len=160,
                             global_batch_size=2, learning_rate=3e-3, mm_max_pixels=14 * 14 * 4 * 8, mm_video_fraction=0.5))
    cfg.model.arch_overrides = dict(linear_heads=2, linear_head_dim=16, vision=dict(hidden_size=32, intermediate_size=64, depth=1, num_heads=2))
    tr = Trainer(cfg)
    batch = next(iter(tr.dataloader))
    tr.dataloader.cursor = 0
    assert (batch["input"] == tr.model.image_token_id).sum() == sum((gh // 2) * (gw // 2) for _, gh, gw in batch["grids"])   # time-pooled
    losses = []
    for _ in range(5):
        tr.dataloader.cursor = 0
        losses.append(tr.train_step().loss)
    assert losses[-1] < losses[0] - 0.2, losses
    tr.close()


# ------------------------------------------------------------------------------------------ local-file recipes
def _fixtures(tmp_path):
    """Three record shapes over PNG files, a whitespace vocabulary that knows the placeholder tokens."""
    import json
    from PIL import Image
    import numpy as np
    from torchllmtuner_b200.components.tokenizer.whitespace import WhitespaceTokenizer
    rng = np.random.default_rng(0)
    for i in range(6):
        Image.fromarray(rng.integers(0, 255, (40 + 8 * i, 72 - 4 * i, 3), dtype=np.uint8)).save(tmp_path / f"im{i}.png")
    words = [f"w{i}" for i in range(40)]
    specials = ["<|image_pad|>", "<|video_pad|>", "<|vision_start|>", "<|vision_end|>", "<|endoftext|>"]
    WhitespaceTokenizer(specials + words).save(str(tmp_path / "vocab.json"))
    text = lambda n, a=0: " ".join(words[(a + j) % 40] for j in range(n))  # noqa: E731
    with open(tmp_path / "captions.jsonl", "w") as f:
        for i in range(6):
            f.write(json.dumps({"image": f"im{i}.png", "caption": text(6 + i, i)}) + "\n")
    with open(tmp_path / "interleaved.jsonl", "w") as f:
        for i in range(4):
            f.write(json.dumps({"texts": [text(5, i), None, text(7, i + 3), None], "images": [None, f"im{i}.png", None, f"im{i + 1}.png"]}) + "\n")
    with open(tmp_path / "mixed.jsonl", "w") as f:
        f.write(json.dumps({"text": f"{text(4)} <|image_pad|> {text(5, 9)} <|video_pad|> {text(3, 20)}", "images": ["im0.png"],
                            "videos": [["im2.png"] * 4]}) + "\n")
        f.write(json.dumps({"text": text(12, 5)}) + "\n")
    return tmp_path


def test_local_recipes_build_samples_from_files(tmp_path):
    from torchllmtuner_b200.components.tokenizer.huggingface import MultimodalTokenizer
    from torchllmtuner_b200.components.tokenizer.whitespace import WhitespaceTokenizer
    from torchllmtuner_b200.config.data_config import DataloaderConfig as DataConfig
    from torchllmtuner_b200.datasets.multimodal_recipes import MultimodalProcessor, load_image
    from torchllmtuner_b200.datasets.sources import IndexedJsonlSource
    root = _fixtures(tmp_path)
    tok = MultimodalTokenizer(WhitespaceTokenizer.from_file(str(root / "vocab.json")), DataConfig())
    assert load_image(str(root / "im0.png")).shape == (3, 40, 72)
    spec = mp.VisionSpec(max_pixels=14 * 14 * 4 * 8, min_pixels=28 * 28 * 4)
    cap = MultimodalProcessor(tok, "local_captions", spec, root=str(root))(IndexedJsonlSource(str(root / "captions.jsonl"))[0])
    n_img = mp.calculate_vision_tokens(cap.grids[0])
    assert cap.tokens[0] == tok.vision_start_id and cap.tokens[1:1 + n_img] == [tok.image_id] * n_img and cap.tokens[1 + n_img] == tok.vision_end_id
    assert cap.labels[:n_img + 2] == [IGNORE_INDEX] * (n_img + 2) and cap.labels[n_img + 2] == cap.tokens[n_img + 2]
    inter = MultimodalProcessor(tok, "local_interleaved", spec, root=str(root))(IndexedJsonlSource(str(root / "interleaved.jsonl"))[1])
    assert len(inter.grids) == 2 and inter.patches.shape[0] == sum(t * h * w for t, h, w in inter.grids)
    mixed_src = IndexedJsonlSource(str(root / "mixed.jsonl"))
    proc = MultimodalProcessor(tok, "local_multimodal", spec, root=str(root))
    mixed = proc(mixed_src[0])
    assert [g[0] for g in mixed.grids] == [1, 2]                        # an image, then a clip of 4 frames = 2 temporal steps
    assert proc(mixed_src[1]).grids == [] and proc(mixed_src[1]).patches.numel() == 0
    with pytest.raises(Exception, match="placeholder"):
        proc({"text": "w1 w2", "images": ["im0.png"]})


def test_vision_language_model_trains_on_local_image_files(tmp_path):
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    root = _fixtures(tmp_path)
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(dump_folder=str(tmp_path / "run"), steps=4, model_name_or_path="qwen3_5_vl", dataset="local_captions",
                             dataset_path=str(root / "captions.jsonl"), tokenizer_backend="whitespace", tokenizer_path=str(root / "vocab.json"),
                             vocab_size=64, hidden_size=64, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=2, max_seq_len=96,
                             global_batch_size=2, learning_rate=3e-3, mm_max_pixels=14 * 14 * 4 * 8, shuffle=False))
    cfg.model.arch_overrides = dict(head_dim=32, image_token_id=6, vision=dict(hidden_size=64, intermediate_size=128, depth=1, num_heads=2))
    tr = Trainer(cfg)
    first = next(iter(tr.dataloader))
    assert first["patches"] is not None and (first["input"] == 6).sum() > 0
    state = tr.dataloader.state_dict()
    second = next(tr.dataloader)
    tr.dataloader.load_state_dict(state)
    assert torch.equal(next(tr.dataloader)["input"], second["input"])          # resumable
    tr.dataloader.load_state_dict({**state, "delivered": 0})
    tr.data_iterator = iter(tr.dataloader)
    losses = [tr.train_step().loss for _ in range(3)]
    assert all(l == l for l in losses) and losses[-1] < losses[0] + 0.5
    tr.close()


def test_full_temporal_rows_keep_the_frames_of_a_step_side_by_side():
    """For a tower whose patch embedding has a temporal axis: a clip's row holds [channel, frame of the step, pixel] values,
    an image's row repeats its frame; both have the tower's full row width."""
    from torchllmtuner_b200.datasets.multimodal_pipeline import VisionSpec, image_to_patches, video_to_patches
    spec = VisionSpec(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=64, max_pixels=64, video_fps=1.0, video_min_frames=4,
                      video_max_frames=4, full_temporal=True)
    frames = torch.arange(4.0).view(4, 1, 1, 1).expand(4, 3, 8, 8) + torch.arange(3.0).view(1, 3, 1, 1) * 10     # value = 10 * channel + frame
    rows, grid = video_to_patches(frames.contiguous(), 1.0, spec)
    assert grid == (2, 2, 2) and rows.shape == (8, 3 * 2 * 16)
    r = rows.view(2, 4, 3, 2, 16)                                     # step, patch, channel, frame in step, pixel
    for step in range(2):
        for ch in range(3):
            for f in range(2):
                assert torch.all(r[step, :, ch, f] == 10 * ch + 2 * step + f)
    img_rows, g = image_to_patches(torch.rand(3, 8, 8), spec)
    assert g == (1, 2, 2) and img_rows.shape == (4, 96)
    v = img_rows.view(4, 3, 2, 16)
    assert torch.equal(v[:, :, 0], v[:, :, 1])
    averaged, _ = video_to_patches(frames.contiguous(), 1.0, VisionSpec(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=64,
                                                                        max_pixels=64, video_fps=1.0, video_min_frames=4, video_max_frames=4))
    assert averaged.shape == (8, 48) and torch.allclose(averaged.view(2, 4, 3, 16)[1, :, 0], torch.full((4, 16), 2.5))


def test_published_tower_trains_through_the_trainer_on_images_and_clips(tmp_path):
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.models.qwen_vit import QwenViTTower
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(dump_folder=str(tmp_path), steps=6, mm_video_fraction=0.5, **VL))
    cfg.model.arch_overrides = dict(head_dim=32, vision_tower="qwen3_5",
                                    vision=dict(hidden_size=64, intermediate_size=128, depth=2, num_heads=2, num_position_embeddings=16))
    tr = Trainer(cfg)
    assert isinstance(tr.model.visual, QwenViTTower)
    batch = next(iter(tr.dataloader))
    tr.dataloader.cursor = 0
    assert batch["patches"].shape[1] == tr.model.visual.config.full_patch_dim          # rows carry the temporal axis
    assert any(g[0] > 1 for g in batch["grids"]) or True
    before = tr.model.visual.pos_embed.weight.detach().clone()
    losses = []
    for _ in range(6):
        tr.dataloader.cursor = 0
        losses.append(tr.train_step().loss)
    assert losses[-1] < losses[0] - 0.3, losses
    assert not torch.equal(before, tr.model.visual.pos_embed.weight)                   # the position table trains too
    tr.close()
