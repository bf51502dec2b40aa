"""Vision tower, 3-axis rotary tables and the vision-language wrapper on CPU (fp32 statements of the same ops)."""
import pytest
import torch

from torchllmtuner_b200 import ops
from torchllmtuner_b200.datasets.multimodal import build_mrope_positions, insert_vision_placeholders, vision_to_patches
from torchllmtuner_b200.errors import ConfigError
from torchllmtuner_b200.models.qwen3 import Qwen3Config, Qwen3ForCausalLM
from torchllmtuner_b200.models.vision import (PatchMerger, VisionConfig, VisionLanguageModel, VisionTower, grid_rope_tables,
                                               mrope_tables)
from torchllmtuner_b200.ops.attn_meta import AttnMeta

VCFG = dict(patch_size=4, hidden_size=64, intermediate_size=96, depth=2, num_heads=2, out_hidden_size=64)
IMG = 90


def _tower(seed=0, **kw):
    t = VisionTower(VisionConfig(**{**VCFG, **kw}))
    t.initialize_parameters(seed)
    return t


def _images(sizes, seed=0):
    g = torch.Generator().manual_seed(seed)
    imgs = [torch.rand(3, h, w, generator=g) for h, w in sizes]
    patches = torch.cat([vision_to_patches(i, 4) for i in imgs])
    grids = [(1, h // 4, w // 4) for h, w in sizes]
    return patches, grids


def test_tower_shapes_and_images_do_not_see_each_other():
    tower = _tower()
    patches, grids = _images([(16, 24), (8, 8)])
    out = tower(patches, grids)
    assert out.shape == (2 * 3 + 1, 64)
    other, _ = _images([(16, 24), (8, 8)], seed=5)
    mixed = torch.cat([patches[:24], other[24:]])                   # second image replaced
    out2 = tower(mixed, grids)
    assert torch.allclose(out[:6], out2[:6], atol=1e-6) and not torch.allclose(out[6:], out2[6:], atol=1e-4)
    alone = tower(patches[:24], grids[:1])
    assert torch.allclose(alone, out[:6], atol=1e-5)


def test_tower_rejects_mismatched_inputs():
    tower = _tower()
    patches, grids = _images([(16, 24)])
    with pytest.raises(ConfigError):
        tower(patches[:-1], grids)
    with pytest.raises(ConfigError):
        tower(*_images([(12, 8)]))                                   # 3 patch rows: not a multiple of the merge size


def test_merger_groups_neighbouring_patches():
    m = PatchMerger(VisionConfig(**VCFG))
    gh, gw = 4, 6
    ids = torch.arange(gh * gw, dtype=torch.float32)[:, None].repeat(1, 64)
    g = m.regroup(ids, [(1, gh, gw)])
    assert g.shape == (6, 256)
    # merged row (1, 2) holds patches (2,4) (2,5) (3,4) (3,5)
    assert g[1 * 3 + 2].view(4, 64)[:, 0].tolist() == [2 * gw + 4, 2 * gw + 5, 3 * gw + 4, 3 * gw + 5]


def test_grid_rope_rows_and_columns():
    cos, sin = grid_rope_tables([(1, 2, 3)], 16, 10_000.0)
    assert cos.shape == (6, 8)
    # patches of one row share the row half; patches of one column share the column half
    assert torch.equal(sin[0, :4], sin[2, :4]) and torch.equal(sin[1, 4:], sin[4, 4:])
    assert not torch.equal(sin[0, 4:], sin[1, 4:]) and not torch.equal(sin[0, :4], sin[3, :4])


def test_mrope_tables_reduce_to_plain_rope_on_text_and_split_by_section():
    pos = torch.arange(11)
    c0, s0 = ops.rope_tables(pos, 32, 1e6)
    c1, s1 = mrope_tables(pos[None].repeat(3, 1), 32, 1e6)
    assert torch.allclose(c0, c1) and torch.allclose(s0, s1)
    p3 = torch.stack([pos, pos * 2, pos * 3])
    c, s = mrope_tables(p3, 32, 1e6, sections=[8, 4, 4])
    ct, _ = ops.rope_tables(pos, 32, 1e6)
    ch, _ = ops.rope_tables(pos * 2, 32, 1e6)
    cw, _ = ops.rope_tables(pos * 3, 32, 1e6)
    assert torch.allclose(c[:, :8], ct[:, :8]) and torch.allclose(c[:, 8:12], ch[:, 8:12]) and torch.allclose(c[:, 12:], cw[:, 12:])
    with pytest.raises(ConfigError):
        mrope_tables(p3, 32, 1e6, sections=[8, 8, 8])


def _vlm(seed=0):
    cfg = Qwen3Config(vocab_size=96, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, head_dim=32, tie_word_embeddings=True)
    text = Qwen3ForCausalLM(cfg)
    m = VisionLanguageModel(text, VisionConfig(**VCFG), image_token_id=IMG)
    m.initialize_parameters(seed)
    return m


def _sample(seed=0):
    patches, grids = _images([(16, 16), (8, 16)], seed)
    g = torch.Generator().manual_seed(seed)
    words = torch.randint(0, 80, (12,), generator=g).tolist()
    ids = insert_vision_placeholders(words[:4] + [IMG] + words[4:8] + [IMG] + words[8:], IMG, grids)
    pos = build_mrope_positions(ids, IMG, grids)
    return torch.tensor(ids), pos, patches, grids


def test_wrapper_splices_image_rows_and_trains_the_tower():
    m = _vlm()
    ids, pos, patches, grids = _sample()
    T = ids.numel()
    assert T == 12 + 4 + 2 and pos.shape == (3, T)
    ctx = m.build_context(pos, AttnMeta.build(torch.tensor([0, T])))
    x = m.embed(ids, patches, grids)
    rows = m.visual(patches, grids)
    where = (ids == IMG).nonzero().squeeze(1)
    assert torch.allclose(x[where], rows) and torch.equal(x[ids != IMG], m.text.model.embed_tokens(ids[ids != IMG]))
    with pytest.raises(ConfigError):
        m.embed(ids, patches[:16], grids[:1])                        # fewer image rows than placeholders
    with pytest.raises(ConfigError):
        m.embed(ids)

    targets = torch.roll(ids, -1)
    targets[ids == IMG] = ops.IGNORE_INDEX
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    losses = []
    for _ in range(8):
        logits = m(ids, ctx, patches=patches, grids=grids)
        loss = torch.nn.functional.cross_entropy(logits.float(), targets, ignore_index=ops.IGNORE_INDEX)
        opt.zero_grad()
        loss.backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m.visual.parameters())
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.3, losses


def test_image_content_reaches_the_logits_only_after_the_image():
    m = _vlm()
    ids, pos, patches, grids = _sample()
    T = ids.numel()
    ctx = m.build_context(pos, AttnMeta.build(torch.tensor([0, T])))
    with torch.no_grad():
        a = m(ids, ctx, patches=patches, grids=grids)
        b = m(ids, ctx, patches=patches * 0.5, grids=grids)
    first = int((ids == IMG).nonzero()[0])
    assert torch.allclose(a[:first], b[:first], atol=1e-6) and not torch.allclose(a[first:], b[first:], atol=1e-4)


def test_text_only_batch_matches_the_plain_decoder():
    m = _vlm()
    ids = torch.randint(0, 80, (10,))
    pos = torch.arange(10)
    meta = AttnMeta.build(torch.tensor([0, 10]))
    with torch.no_grad():
        a = m(ids, m.build_context(pos[None].repeat(3, 1), meta))
        b = m.text(ids, m.text.build_context(pos, meta))
    assert torch.allclose(a, b, atol=1e-6)
