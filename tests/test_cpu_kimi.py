"""Kimi-Linear / Kimi-K3 pieces against step-by-step restatements: document-aware short convolution, the KDA recurrence
with per-channel decay, latent attention without rotary, grouped sigmoid routing, attention residuals, SituGLU, and the
whole decoder's causality; sequence parallelism (convolution history and recurrent state handed across ranks)."""
import math

import pytest
import torch
import torch.nn.functional as F

from dist_cases import base_flat, run_ranks
from torchllmtuner_b200.models import kimi_k3 as km
from torchllmtuner_b200.ops import AttnMeta


def _cfg(**kw):
    base = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=2, num_key_value_heads=2,
                head_dim=16, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16, linear_heads=2, linear_head_dim=8,
                kda_chunk_size=4)
    base.update(kw)
    return km.KimiConfig(**base)


def _ctx(model, lens):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return model.build_context(torch.cat([torch.arange(n) for n in lens]), AttnMeta.build(cu, causal=True))


def _model(**kw):
    torch.manual_seed(0)
    m = km.KimiForCausalLM(_cfg(**kw), dtype=torch.float32)
    m.initialize_parameters(seed=3)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2 and p.shape[-1] > 4:
                p.mul_(6.0)
    return m.eval()


def test_short_convolution_restarts_at_documents_and_matches_conv1d():
    conv = km.CausalConvolution(6, 4, dtype=torch.float32)
    with torch.no_grad():
        conv.weight.normal_()
    lens = [5, 1, 9]
    x = torch.randn(sum(lens), 6)
    pos = torch.cat([torch.arange(n) for n in lens])
    got = conv(x, pos)
    a = 0
    for n in lens:
        want = F.silu(F.conv1d(x[a:a + n].t()[None], conv.weight, padding=3, groups=6)[0, :, :n].t())
        assert torch.allclose(got[a:a + n], want, atol=1e-6)
        a += n


def test_kda_layer_matches_the_token_by_token_recurrence():
    m = _model()
    layer = m.model.layers[0].self_attn
    assert isinstance(layer, km.KimiDeltaAttention)
    lens = [11, 6]
    ctx = _ctx(m, lens)
    x = torch.randn(sum(lens), 32)
    got = layer(x, ctx)
    H, d = layer.H, layer.d
    outs = []
    a = 0
    for n in lens:
        xs, pos = x[a:a + n], torch.arange(n)
        q, k, v = (getattr(layer, f"{c}_conv1d")(getattr(layer, f"{c}_proj")(xs), pos).view(n, H, d) for c in "qkv")
        q = q / torch.sqrt(q.square().sum(-1, keepdim=True) + 1e-6)
        k = k / torch.sqrt(k.square().sum(-1, keepdim=True) + 1e-6)
        raw = layer.f_b_proj(layer.f_a_proj(xs)).view(n, H, d) + layer.dt_bias.view(H, d)
        decay = (-layer.A_log.exp().view(1, H, 1) * F.softplus(raw)).exp()
        beta = layer.b_proj(xs).sigmoid()
        S = torch.zeros(H, d, d)
        o = []
        for t in range(n):
            S = S * decay[t].unsqueeze(-1)
            resid = v[t] - (k[t].unsqueeze(-1) * S).sum(-2)
            S = S + k[t].unsqueeze(-1) * (resid * beta[t].unsqueeze(-1)).unsqueeze(-2)
            o.append((q[t].unsqueeze(-1) * S).sum(-2) * d ** -0.5)
        o = torch.stack(o)
        gate = layer.g_b_proj(layer.g_a_proj(xs)).view(n, H, d)
        o = o * torch.rsqrt(o.square().mean(-1, keepdim=True) + layer.eps) * layer.o_norm.weight * gate.sigmoid()
        outs.append(layer.o_proj(o.reshape(n, H * d)))
        a += n
    assert torch.allclose(got, torch.cat(outs), atol=2e-5), (got - torch.cat(outs)).abs().max()


def test_bounded_decay_form():
    m = _model(gate_lower_bound=-3.0)
    layer = m.model.layers[0].self_attn
    x = torch.randn(5, 32)
    ld = layer.log_decay(x)
    assert (ld <= 0).all() and (ld >= -3.0).all()
    with pytest.raises(ValueError):
        _model(gate_lower_bound=-9.0)


def test_latent_attention_has_no_rotary_and_handles_narrow_values():
    m = _model(v_head_dim=8, mla_use_output_gate=True, q_lora_rank=12)
    att = m.model.layers[3].self_attn
    assert isinstance(att, km.KimiLatentAttention)
    lens = [7, 5]
    x = torch.randn(12, 32)
    got = att(x, _ctx(m, lens))
    # the same document at another place of the batch gives the same rows: nothing depends on absolute position
    alone = att(x[7:], _ctx(m, [5]))
    assert torch.allclose(got[7:], alone, atol=1e-5)
    q = att.q_b_proj(att.q_a_layernorm(att.q_a_proj(x))).view(12, 2, att.dq)
    ckv = att.kv_a_proj_with_mqa(x)
    kv = att.kv_b_proj(att.kv_a_layernorm(ckv[:, :att.rank])).view(12, 2, att.dn + att.dv)
    out = torch.zeros(12, 2, att.dv)
    a = 0
    for n in lens:
        for i in range(n):
            for h in range(2):
                keys = torch.cat((kv[a:a + i + 1, h, :att.dn], ckv[a:a + i + 1, att.rank:]), -1)
                p = (keys @ q[a + i, h] * att.scale).softmax(0)
                out[a + i, h] = p @ kv[a:a + i + 1, h, att.dn:]
        a += n
    want = att.o_proj(out.reshape(12, -1) * att.g_proj(x).sigmoid())
    assert torch.allclose(got, want, atol=1e-5)


def test_grouped_sigmoid_routing_selects_inside_the_best_groups():
    m = _model(num_expert_group=4, topk_group=2, routed_scaling_factor=2.5)
    moe = m.model.layers[1].mlp
    assert isinstance(moe, km.KimiMoE)
    with torch.no_grad():
        moe.expert_bias_E.copy_(torch.linspace(-0.2, 0.2, 8))
    x = torch.randn(9, 32)
    w, idx, counts, _ = moe.router(x, moe.expert_bias_E)
    scores = (x @ moe.router.weight.t()).sigmoid()
    choice = scores + moe.expert_bias_E
    for t in range(9):
        group_score = choice[t].view(4, 2).topk(2, -1).values.sum(-1)
        keep = set(group_score.topk(2).indices.tolist())
        allowed = [e for e in range(8) if e // 2 in keep]
        want = sorted(allowed, key=lambda e: -float(choice[t, e]))[:2]
        assert set(idx[t].tolist()) == set(want), (t, idx[t], want)
        sel = scores[t, idx[t]]
        assert torch.allclose(w[t], sel / sel.sum() * 2.5, atol=1e-6)          # weights from the scores without the bias
    with pytest.raises(ValueError, match="groups"):
        _cfg(num_expert_group=3)
    with pytest.raises(ValueError, match="retained groups"):
        _cfg(num_expert_group=8, topk_group=1)


def test_latent_experts_project_into_and_out_of_a_narrow_space():
    m = _model(routed_expert_hidden_size=16)
    moe = m.model.layers[1].mlp
    assert moe.routed.experts.w1_EFD.shape == (8, 16, 16) and moe.routed_expert_down_proj.weight.shape == (16, 32)
    x = torch.randn(6, 32)
    got = moe(x)
    w, idx, _, _ = moe.router(x, moe.expert_bias_E)
    z = moe.routed_expert_down_proj(x)
    ex = moe.routed.experts
    acc = torch.zeros(6, 16)
    for t in range(6):
        for j in range(2):
            e = int(idx[t, j])
            h = F.silu(z[t] @ ex.w1_EFD[e].t()) * (z[t] @ ex.w3_EFD[e].t())
            acc[t] += w[t, j] * (h @ ex.w2_EDF[e].t())
    want = moe.routed_expert_up_proj(moe.routed_expert_norm(acc)) + moe.shared_experts(x)
    assert torch.allclose(got, want, atol=1e-5)


def test_situ_glu_and_attention_residual_formulas():
    g, u = torch.randn(4, 6), torch.randn(4, 6)
    act = km.SituGLU(2.0, 3.0)
    assert torch.allclose(act(g, u), 2.0 * torch.tanh(g / 2.0) * g.sigmoid() * 3.0 * torch.tanh(u / 3.0), atol=1e-6)
    with pytest.raises(ValueError):
        km.SituGLU(0.0)
    prefix, blocks = torch.randn(3, 8), torch.randn(3, 2, 8)
    pw, nw = torch.randn(1, 8), torch.rand(8) + 0.5
    got = km.attention_residual(prefix, blocks, pw, nw, 1e-6)
    for t in range(3):
        cand = torch.cat((blocks[t], prefix[t][None]))
        score = torch.stack([((c / torch.sqrt(c.square().mean() + 1e-6)) * nw * pw[0]).sum() for c in cand])
        assert torch.allclose(got[t], (score.softmax(0)[:, None] * cand).sum(0), atol=1e-5)


@pytest.mark.parametrize("extra", [dict(), dict(attn_res_block_size=2, hidden_act="situ", activation_situ_beta=4.0, routed_expert_hidden_size=16,
                                               num_expert_group=4, topk_group=2, mla_use_output_gate=True)])
def test_decoder_is_causal_and_documents_are_isolated(extra):
    m = _model(**extra)
    lens = [13, 8]
    tok = torch.randint(0, 64, (21,))
    with torch.no_grad():
        base = m(tok, _ctx(m, lens), skip_lm_head=True)
        t2 = tok.clone()
        t2[9] = (t2[9] + 1) % 64
        pert = m(t2, _ctx(m, lens), skip_lm_head=True)
        assert torch.allclose(base[:9], pert[:9], atol=1e-6) and not torch.allclose(base[9:13], pert[9:13])
        assert torch.allclose(base[13:], pert[13:], atol=1e-6)
        alone = m(tok[13:], _ctx(m, [8]), skip_lm_head=True)
        assert torch.allclose(alone, base[13:], atol=1e-5)


def test_layer_schedule_follows_the_published_one_based_lists():
    c = _cfg(num_hidden_layers=8, kda_layers=[1, 2, 3, 5, 6, 7], first_k_dense_replace=2, moe_layer_freq=2)
    assert [c.is_kda_layer(i) for i in range(8)] == [True, True, True, False, True, True, True, False]
    assert [c.is_moe_layer(i) for i in range(8)] == [False, False, True, False, True, False, True, False]


@pytest.mark.parametrize("family", ["kimi_linear", "kimi_k3"])
def test_sequence_parallel_gives_the_gradients_of_one_rank(family, tmp_path):
    """Two ranks each hold half of every sequence: the convolutions fetch their history from the rank before, the
    recurrence hands its state on, the latent attention gathers keys and values. After one step the first Adam moment
    (0.1 x the gradient) of every parameter must agree with the single-rank run, and the loss curve follows (which also
    needs the parameters that no decoder block owns, the output mixing of the attention residuals, to be refreshed on
    every rank after each optimizer step)."""
    import os
    import torch.distributed.checkpoint as dcp
    arch = dict(head_dim=16, linear_heads=2, linear_head_dim=8, kda_chunk_size=8)
    base = dict(model_name_or_path=family, num_hidden_layers=4, enable=True)
    one, two = str(tmp_path / "one"), str(tmp_path / "two")
    ref = run_ranks(1, base_flat(dump_folder=one, _save_at=1, **base), arch=arch, steps=3)
    got = run_ranks(2, base_flat(dump_folder=two, _save_at=1, data_parallel_shard_size=1, context_parallel_kcp_size=2, **base), arch=arch, steps=3)
    assert abs(ref["loss"][0] - got["loss"][0]) < 1e-5 and abs(ref["grad_norm"][0] - got["grad_norm"][0]) < 1e-4, (ref, got)
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 5e-5, (ref, got)

    def moments(folder):
        path = os.path.join(folder, "checkpoint", "step-1")
        md = dcp.FileSystemReader(path).read_metadata().state_dict_metadata
        want = {k: torch.empty(tuple(v.size), dtype=v.properties.dtype) for k, v in md.items() if k.endswith(".exp_avg")}
        dcp.load(want, checkpoint_id=path, no_dist=True)
        return want
    a, b = moments(one), moments(two)
    assert a.keys() == b.keys() and len(a) > 20
    scale = max(t.abs().max().item() for t in a.values())
    for k in a:
        tol = 1e-4 * a[k].abs().max().item() + 1e-7 * scale
        assert (a[k] - b[k]).abs().max().item() <= tol, (k, (a[k] - b[k]).abs().max().item(), a[k].abs().max().item())


def test_hf_export_uses_the_published_names_and_imports_back(tmp_path):
    import json
    import os
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.components.checkpointer.hf import load_hf_checkpoint, save_hf_checkpoint
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(model_name_or_path="kimi_k3", num_hidden_layers=4, dump_folder=str(tmp_path / "run")))
    cfg.model.arch_overrides = dict(head_dim=16, linear_heads=2, linear_head_dim=8)
    tr = Trainer(cfg)
    tr.train_step()
    out = str(tmp_path / "hf")
    save_hf_checkpoint(tr, out, "float32")
    wm = json.load(open(os.path.join(out, "model.safetensors.index.json")))["weight_map"]
    for k in ("model.layers.1.block_sparse_moe.gate.weight", "model.layers.1.block_sparse_moe.experts.7.w2.weight",
              "model.layers.1.block_sparse_moe.shared_experts.gate_proj.weight", "model.layers.1.block_sparse_moe.routed_expert_down_proj.weight",
              "model.layers.0.mlp.gate_proj.weight", "model.layers.0.self_attn.q_conv1d.weight", "model.layers.0.self_attn.A_log",
              "model.layers.3.self_attn.kv_a_proj_with_mqa.weight", "model.layers.2.mlp_res_proj.weight", "model.output_attn_res_proj.weight"):
        assert k in wm, (k, sorted(wm)[:40])
    hf_cfg = json.load(open(os.path.join(out, "config.json")))
    assert hf_cfg["model_type"] == "kimi_linear" and hf_cfg["linear_attn_config"]["kda_layers"] == [1, 2, 3]
    before = [u.master.clone() for u in tr.asm.fsdp.units]
    for u in tr.asm.fsdp.units:
        u.master.zero_()
    load_hf_checkpoint(tr, out)
    for a, u in zip(before, tr.asm.fsdp.units):
        assert torch.equal(a[:u.numel], u.master[:u.numel])
    tr.close()


@pytest.mark.parametrize("lower", [None, -5.0, -2.0])
def test_decay_gate_forms_match_the_flash_linear_attention_references(lower):
    """log decay = -exp(A_log) * softplus(f(x) + dt_bias), or lower_bound * sigmoid(exp(A_log) * (f(x) + dt_bias)): the
    module's two forms against the plain-PyTorch gate references of the `fla` package."""
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        gate = pytest.importorskip("fla.ops.kda.gate")
    cfg = _cfg(gate_lower_bound=lower)
    torch.manual_seed(1)
    m = km.KimiDeltaAttention(cfg)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.5)
    x = torch.randn(13, cfg.hidden_size)
    raw = m.f_b_proj(m.f_a_proj(x)).float().view(1, 13, m.H, m.d)
    if lower is None:
        want = gate.naive_kda_gate(raw, m.A_log, m.dt_bias)
    else:
        want = gate.naive_kda_lowerbound_gate(raw, m.A_log, m.dt_bias, lower_bound=lower)
    assert torch.allclose(m.log_decay(x), want[0], atol=1e-6)
