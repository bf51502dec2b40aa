"""DeepSeek-V4 pieces against brute-force restatements written token by token: window pooling with and without
overlap, the indexer's causal top-k, window + entry attention with sinks, hyper-connection normalisation, hash routing,
and whole-model causality and document isolation."""
import math

import pytest
import torch

from torchllmtuner_b200.models import deepseek_v4 as v4
from torchllmtuner_b200.ops import AttnMeta


def _cfg(**kw):
    base = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=1,
                head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, shared_expert_intermediate_size=16,
                sliding_window=6, index_topk=2, qk_rope_head_dim=8)
    base.update(kw)
    return v4.DeepseekV4Config(**base)


def _ctx(model, lens):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    return model.build_context(pos, AttnMeta.build(cu, causal=True))


def _model(**kw):
    torch.manual_seed(0)
    m = v4.DeepseekV4ForCausalLM(_cfg(**kw), dtype=torch.float32)
    m.initialize_parameters(seed=1)
    with torch.no_grad():                      # make the zero-initialised pieces matter
        for mod in m.modules():
            if isinstance(mod, v4._WindowPool):
                mod.position_bias.normal_(0, 0.5)
            if isinstance(mod, v4.V4Attention):
                mod.sinks.normal_(0, 0.5)
            if isinstance(mod, (v4.HyperConnection,)):
                mod.base.normal_(0, 0.3)
        for p in m.parameters():
            if p.dim() >= 2:
                p.mul_(8.0)
    return m.eval()


def test_rotation_of_trailing_pairs_matches_complex_multiplication_and_inverts():
    x = torch.randn(5, 3, 12)
    pos = torch.tensor([0, 1, 5, 9, 2])
    cos, sin = v4.rope_tables_interleaved(pos, 8, 10000.0)
    y = v4.rotate_trailing_pairs(x, cos, sin)
    assert torch.equal(y[..., :4], x[..., :4])
    z = torch.view_as_complex(x[..., 4:].reshape(5, 3, 4, 2).contiguous()) * torch.polar(torch.ones(5, 4), pos[:, None] * (1.0 / 10000.0 ** (torch.arange(0, 8, 2) / 8)))[:, None, :]
    assert torch.allclose(y[..., 4:], torch.view_as_real(z).flatten(-2), atol=1e-5)
    assert torch.allclose(v4.rotate_trailing_pairs(y, cos, -sin), x, atol=1e-5)


def test_window_pool_without_and_with_overlap():
    m = _model()
    ctx = _ctx(m, [19, 9])
    x = torch.randn(28, 32)
    hca = m.model.layers[2].self_attn.compressor
    csa = m.model.layers[1].self_attn.compressor
    assert isinstance(hca, v4.HCACompressor) and isinstance(csa, v4.CSACompressor)
    for pool in (hca, csa):
        got = pool.pool(x, ctx)
        r, d = pool.rate, pool.width
        kv, gate = pool.kv_proj(x), pool.gate_proj(x)
        for (q0, L), e in zip(((0, 19), (19, 9)), got):
            assert e.shape == (L // r, d)
            for w in range(L // r):
                vals, logits = [], []
                if pool.overlap:
                    for j in range(r):              # first half of the previous window's features
                        if w > 0:
                            t = q0 + (w - 1) * r + j
                            vals.append(kv[t, :d])
                            logits.append(gate[t, :d] + pool.position_bias[j, :d])
                    for j in range(r):              # second half of this window's
                        t = q0 + w * r + j
                        vals.append(kv[t, d:])
                        logits.append(gate[t, d:] + pool.position_bias[j, d:])
                else:
                    for j in range(r):
                        t = q0 + w * r + j
                        vals.append(kv[t])
                        logits.append(gate[t] + pool.position_bias[j])
                p = torch.stack(logits).softmax(0)
                pooled = pool.kv_norm((torch.stack(vals) * p).sum(0, keepdim=True))
                cos, sin = v4.rope_tables_interleaved(torch.tensor([w * r]), pool.rope_dim, pool.theta)
                assert torch.allclose(e[w], v4.rotate_trailing_pairs(pooled, cos, sin)[0], atol=1e-5), (pool.overlap, w)


def test_indexer_selects_only_complete_windows_and_the_best_of_them():
    m = _model()
    ctx = _ctx(m, [23])
    x = torch.randn(23, 32)
    att = m.model.layers[1].self_attn
    idx = att.compressor.indexer
    q_res = att.q_a_norm(att.q_a_proj(x))
    (sel,) = idx.select(x, q_res, ctx)
    keys = idx.pool(x, ctx)[0]
    r = idx.rate
    cos, sin = ctx.rope["compress"]
    q = v4.rotate_trailing_pairs(idx.q_b_proj(q_res).view(23, idx.heads, idx.width), cos, sin)
    hw = idx.weights_proj(x) * idx.heads ** -0.5
    for t in range(23):
        visible = (t + 1) // r
        scores = [sum(float(torch.relu(q[t, h] @ keys[w]) * idx.width ** -0.5 * hw[t, h]) for h in range(idx.heads)) for w in range(visible)]
        got = [int(i) for i in sel[t] if i >= 0]
        assert len(got) == len(set(got)) == min(idx.topk, visible) and all(i < visible for i in got), (t, got)
        # ties (several keys scoring exactly zero after the relu) may resolve either way: compare the scores reached
        assert sorted(scores[i] for i in got) == pytest.approx(sorted(scores, reverse=True)[:idx.topk][::-1], abs=1e-6), (t, got, scores)


@pytest.mark.parametrize("layer", [0, 1, 2])
def test_attention_matches_a_per_query_softmax_over_its_visible_keys(layer):
    m = _model()
    lens = [21, 10]
    ctx = _ctx(m, lens)
    x = torch.randn(sum(lens), 32)
    att = m.model.layers[layer].self_attn
    got = att(x, ctx)
    # restatement
    T, H, d = x.shape[0], att.H, att.d
    cos, sin = ctx.rope[att.rope_kind]
    q_res = att.q_a_norm(att.q_a_proj(x))
    q = v4.rotate_trailing_pairs(v4.unweighted_rms_norm(att.q_b_proj(q_res).view(T, H, d), att.eps), cos, sin)
    kv = v4.rotate_trailing_pairs(att.kv_norm(att.kv_proj(x)), cos, sin)
    comp = att.compressor(x, q_res, ctx) if att.compressor is not None else None
    out = torch.zeros(T, H, d)
    q0 = 0
    for di, L in enumerate(lens):
        for i in range(L):
            keys = [kv[q0 + j] for j in range(max(0, i - att.window + 1), i + 1)]
            if comp is not None:
                e, bias = comp[di]
                keys += [e[w] for w in range(e.shape[0]) if bias[i, w] == 0]
            K = torch.stack(keys)
            for h in range(H):
                logits = torch.cat((K @ q[q0 + i, h] * att.scale, att.sinks[h:h + 1]))
                p = logits.softmax(0)[:-1]
                out[q0 + i, h] = p @ K
        q0 += L
    out = v4.rotate_trailing_pairs(out, cos, -sin)
    want = att.o_b_proj(att.o_a_proj(out.reshape(T, att.groups, -1)).reshape(T, -1))
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()


def test_hyper_connection_mixing_is_doubly_normalised_and_collapse_is_a_weighted_sum():
    cfg = _cfg(hc_mult=3, hc_sinkhorn_iters=30)
    hc = v4.HyperConnection(cfg, dtype=torch.float32)
    with torch.no_grad():
        hc.fn.normal_(0, 0.3)
        hc.base.normal_(0, 0.3)
        hc.scale.fill_(1.0)
    s = torch.randn(7, 3, 32)
    post, comb, x = hc(s)
    assert post.shape == (7, 3) and comb.shape == (7, 3, 3) and x.shape == (7, 32)
    assert torch.allclose(comb.sum(-1), torch.ones(7, 3), atol=1e-3) and torch.allclose(comb.sum(-2), torch.ones(7, 3), atol=1e-3)
    assert (post > 0).all() and (post < 2).all()
    # the write consumes the matrix transposed
    y = torch.randn(7, 32)
    new = v4.write_streams(post, comb, y, s)
    for t in range(7):
        for mi in range(3):
            want = post[t, mi] * y[t] + sum(comb[t, n, mi] * s[t, n] for n in range(3))
            assert torch.allclose(new[t, mi], want, atol=1e-5)


def test_hash_routed_layer_takes_its_experts_from_the_table():
    m = _model()
    layer = m.model.layers[0]
    assert layer.is_hash and not m.model.layers[1].is_hash
    ids = torch.tensor([3, 9, 3, 60])
    x = torch.randn(4, 32)
    w, idx, counts, _ = layer.mlp.router(x, None, token_ids=ids)
    assert torch.equal(idx, layer.mlp.router.tid2eid[ids]) and torch.equal(idx[0], idx[2])
    assert (idx[:, 0] != idx[:, 1]).all()
    assert torch.allclose(w.sum(-1), torch.full((4,), m.config.routed_scaling_factor), atol=1e-5)
    assert counts.sum() == 8
    with pytest.raises(ValueError):
        layer.mlp(x)


def test_model_is_causal_and_documents_do_not_see_each_other():
    m = _model()
    lens = [17, 12]
    tok = torch.randint(0, 64, (29,))
    with torch.no_grad():
        base = m(tok, _ctx(m, lens), skip_lm_head=True)
        t2 = tok.clone()
        t2[11] = (t2[11] + 1) % 64
        pert = m(t2, _ctx(m, lens), skip_lm_head=True)
        assert torch.equal(base[:11], pert[:11]) and not torch.allclose(base[11:17], pert[11:17])
        assert torch.equal(base[17:], pert[17:])                       # the second document never sees the first
        alone = m(tok[17:], _ctx(m, [12]), skip_lm_head=True)
        assert torch.allclose(alone, base[17:], atol=1e-5)


def test_schedule_and_geometry_are_validated_before_anything_is_allocated():
    with pytest.raises(ValueError, match="layer_types"):
        _cfg(layer_types=["sliding_attention"])
    with pytest.raises(ValueError, match="not one of"):
        _cfg(mlp_layer_types=["moe", "dense", "moe"])
    with pytest.raises(ValueError, match="compress_rates"):
        _cfg(compress_rates={"compressed_sparse_attention": 0, "heavily_compressed_attention": 8})
    with pytest.raises(ValueError, match="o_groups"):
        _cfg(o_groups=3)


def test_trains_through_the_trainer_and_round_trips_its_checkpoint_names(tmp_path):
    from dist_cases import base_flat
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.components.checkpointer.reference_layout import export_reference_layout
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path="deepseek_v4", num_hidden_layers=3, max_seq_len=64, steps=6, dump_folder=str(tmp_path),
                             enable=True, interval=100))
    tr = Trainer(cfg)
    losses = []
    for _ in range(6):
        tr.dataloader.cursor = 0
        losses.append(tr.train_step().loss)
    assert losses[-1] < losses[0] - 0.5, losses
    tr.checkpointer.save(6, force=True)
    tr.checkpointer.wait()
    tr.close()
    info = export_reference_layout(str(tmp_path / "checkpoint" / "step-6"), str(tmp_path / "ref"))
    keys = set(info["keys"])
    for k in ("model.layers.0.mlp.gate.weight", "model.layers.1.mlp.experts.gate_up_proj", "model.layers.1.self_attn.compressor.indexer.scorer.weights_proj.weight",
              "model.layers.2.self_attn.compressor.position_bias", "model.layers.0.attn_hc.fn", "model.hc_head.hc_fn", "model.layers.0.self_attn.sinks",
              "model.layers.0.self_attn.o_a_proj.weight"):
        assert k in keys, (k, sorted(keys)[:30])


def test_two_fsdp_ranks_match_one():
    """The stream-collapsing head belongs to no decoder block; its shard must be gathered again after every step."""
    from dist_cases import base_flat, run_ranks
    base = dict(model_name_or_path="deepseek_v4", num_hidden_layers=3, max_seq_len=64)
    ref = run_ranks(1, base_flat(**base), steps=4)
    got = run_ranks(2, base_flat(data_parallel_shard_size=2, **base), steps=4)
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 5e-5, (ref, got)


def test_sequence_parallel_ranks_reproduce_one_rank(tmp_path):
    """Two ranks each hold half of every sequence: the shared key/value head and the compressor inputs are gathered, every
    rank pools all windows, queries stay local. First Adam moments (0.1 x gradient) and losses agree with one rank."""
    import os
    import torch.distributed.checkpoint as dcp
    from dist_cases import base_flat, run_ranks
    base = dict(model_name_or_path="deepseek_v4", num_hidden_layers=3, max_seq_len=64, enable=True)
    one, two = str(tmp_path / "one"), str(tmp_path / "two")
    ref = run_ranks(1, base_flat(dump_folder=one, _save_at=1, **base), steps=3)
    got = run_ranks(2, base_flat(dump_folder=two, _save_at=1, data_parallel_shard_size=1, context_parallel_kv_allgather_size=2, **base), steps=3)
    assert abs(ref["loss"][0] - got["loss"][0]) < 1e-5, (ref, got)
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 1e-4, (ref, got)

    def moments(folder):
        path = os.path.join(folder, "checkpoint", "step-1")
        md = dcp.FileSystemReader(path).read_metadata().state_dict_metadata
        want = {k: torch.empty(tuple(v.size), dtype=v.properties.dtype) for k, v in md.items() if k.endswith(".exp_avg")}
        dcp.load(want, checkpoint_id=path, no_dist=True)
        return want
    a, b = moments(one), moments(two)
    scale = max(t.abs().max().item() for t in a.values())
    for k in a:
        assert (a[k] - b[k]).abs().max().item() <= 1e-4 * a[k].abs().max().item() + 1e-7 * scale, k
