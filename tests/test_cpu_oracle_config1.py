"""The CPU oracle configuration: tiny Qwen3 dense on CPU, single process, fp32, 20 AdamW steps on uniform random tokens from
seed 0. The oracle is an independent plain-PyTorch statement of the same architecture (`baseline/stock_arm.py::Model`,
library `nn.Linear` / `F.scaled_dot_product_attention` / `nn.RMSNorm`), started from the same weights and fed the same
batches; thresholds are the reference's acceptance numbers (per-step loss absolute error <= 0.02, relative <= 0.005)."""
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from torchllmtuner_b200 import LLMTunerConfig, Trainer  # noqa: E402

ARCH = dict(vocab_size=32000, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=768,
            num_hidden_layers=4, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)


def _oracle_hidden(m, ids):
    """The stand-in model's forward with fp32 rotary tables and no activation checkpointing."""
    S, d = ids.shape[1], 64
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.arange(S, dtype=torch.float32)[:, None] * inv[None]
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x = m.embed_tokens(ids)
    for layer in m.layers:
        x = layer(x, cos, sin)
    return m.norm(x)


def test_twenty_steps_match_the_plain_pytorch_oracle(monkeypatch):
    from baseline.stock_arm import Model
    monkeypatch.setenv("LLMTUNER_DEVICE", "cpu")
    torch.manual_seed(0)
    cfg = LLMTunerConfig()
    cfg.apply_flat(dict(model_name_or_path="qwen3", vocab_size=32000, hidden_size=256, intermediate_size=768, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, global_batch_size=4, max_seq_len=512, steps=20,
                        learning_rate=3e-4, seed=0, dump_folder="/tmp/llmt_oracle_out", compute_dtype="float32"))
    cfg.model.arch_overrides = dict(head_dim=64, tie_word_embeddings=True, rope_theta=1e6)
    tr = Trainer(cfg)
    assert tr.model.config.tie_word_embeddings and tr.model.lm_head.weight is tr.model.model.embed_tokens.weight
    # oracle with the same starting weights
    oracle = Model(dict(ARCH)).float()
    oracle.lm_head.weight = oracle.embed_tokens.weight
    mine = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    with torch.no_grad():
        for n, p in oracle.named_parameters():
            src = "model." + n if not n.startswith("lm_head") else n
            src = src.replace("layers.", "layers.").replace(".q_proj", ".self_attn.q_proj").replace(".k_proj", ".self_attn.k_proj") \
                     .replace(".v_proj", ".self_attn.v_proj").replace(".o_proj", ".self_attn.o_proj") \
                     .replace(".q_norm", ".self_attn.q_norm").replace(".k_norm", ".self_attn.k_norm") \
                     .replace(".gate_proj", ".mlp.gate_proj").replace(".up_proj", ".mlp.up_proj").replace(".down_proj", ".mlp.down_proj")
            assert src in mine, (n, src)
            p.copy_(mine[src].float())
    opt = torch.optim.AdamW(oracle.parameters(), lr=3e-4, weight_decay=0.0, betas=(0.9, 0.999), eps=1e-8)
    ours, ref = [], []
    for step in range(20):
        batch = tr.fetch_batch()
        ids, labels = batch["input"], batch["labels"]
        h = _oracle_hidden(oracle, ids)
        logits = h @ oracle.lm_head.weight.t()
        loss = F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=-100, reduction="sum") / float(batch["num_valid_tokens"])
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(oracle.parameters(), 1.0)
        opt.step()
        ref.append(float(loss))
        ours.append(tr.train_step(batches=[batch]).loss)
    tr.close()
    for a, b in zip(ours, ref):
        assert abs(a - b) <= 0.02 and abs(a - b) / abs(b) <= 0.005, (ours, ref)
    assert ours[-1] < ours[0]
