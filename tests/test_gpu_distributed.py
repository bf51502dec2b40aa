"""Multi-GPU equivalence (needs >= 2 GPUs): sharded arm on NCCL vs single GPU, bf16 tolerances."""
import pytest
import torch

from dist_cases import base_flat, run_ranks

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _flat(**kw):
    return base_flat(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, max_seq_len=256,
                     vocab_size=1024, **kw)


def test_fsdp2_gpu_matches_single_gpu():
    _need(2)
    ref = run_ranks(1, _flat(), device="cuda")
    for impl in ("custom", "native"):
        got = run_ranks(2, _flat(data_parallel_shard_size=2, activation_checkpoint_mode="full", fsdp_implementation=impl), device="cuda")
        assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 3e-2, (impl, ref, got)
        assert max(abs(a - b) / max(a, 1e-6) for a, b in zip(ref["grad_norm"], got["grad_norm"])) < 5e-2, (impl, ref, got)


def test_fsdp2_with_blocks_of_different_sizes_fuses_the_common_size():
    """Kimi-Linear blocks come in three sizes (dense first layer, KDA + sparse, latent attention + sparse). The most common
    size rides the peer-memory collectives, the odd units take NCCL in the same runtime; two GPUs reproduce one."""
    _need(2)
    arch = dict(linear_heads=4, linear_head_dim=64, kda_chunk_size=16, qk_nope_head_dim=32, qk_rope_head_dim=32, v_head_dim=64, kv_lora_rank=64)
    base = dict(model_name_or_path="kimi_linear", num_hidden_layers=6)
    ref = run_ranks(1, _flat(**base), arch=arch, device="cuda")
    got = run_ranks(2, _flat(data_parallel_shard_size=2, **base), arch=arch, device="cuda")
    assert got.get("fsdp_fused_units", 0) >= 3 and got["fsdp_fused_units"] < got["fsdp_block_units"], got
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 4e-2, (ref, got)


MOE = dict(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128)


@pytest.mark.parametrize("name,flat,arch", [
    ("tp2", dict(tensor_parallel_size=2, data_parallel_shard_size=1), None),
    ("cp_ulysses2", dict(context_parallel_ulysses_size=2, data_parallel_shard_size=1), None),
    ("cp_kv2_headtail", dict(context_parallel_kv_allgather_size=2, context_parallel_load_balancer="headtail", data_parallel_shard_size=1), None),
    ("ep2", dict(model_name_or_path="qwen3_moe", expert_parallel_size=2, data_parallel_shard_size=2), MOE),
    ("tp2_moe", dict(model_name_or_path="qwen3_moe", tensor_parallel_size=2, data_parallel_shard_size=1), MOE),
])
def test_parallel_modes_gpu_match_single_gpu(name, flat, arch):
    _need(2)
    base = dict(model_name_or_path=flat.get("model_name_or_path", "qwen3"))
    ref = run_ranks(1, _flat(**base), arch=arch, device="cuda")
    got = run_ranks(2, _flat(**flat), arch=arch, device="cuda")
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 4e-2, (name, ref, got)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_tp_gemms_match_nccl_reference(world):
    """all-gather -> GEMM and GEMM -> reduce-scatter over peer memory, forward and backward, with slot reuse."""
    _need(world)
    from fused_tp_cases import run_fused_tp
    res = run_fused_tp(world)
    for k in ("ag", "rs", "ag_bwd", "rs_bwd"):
        assert res[k] < 2e-2, res
    assert res["stats"]["ag_fused"] > 0 and res["stats"]["rs_fused"] > 0


@pytest.mark.parametrize("world", [2, 8])
def test_vocab_parallel_head_and_embedding_match_the_full_vocabulary(world):
    """Vocabulary-sharded head: gather riding on the logits GEMM, one (max, sum-exp, target) exchange per token inside the
    loss kernel, reduce-scatter riding on the input-gradient GEMM; embedding rows written into the owners' token shards."""
    _need(world)
    from fused_tp_cases import run_vocab_parallel
    res = run_vocab_parallel(world)
    assert res["loss"] < 2e-3 and res["dh"] < 3e-2 and res["dw"] < 3e-2 and res["emb"] == 0.0 and res["demb"] < 2e-2, res
    assert res["stats"].get("ag_fused", 0) > 0 and res["stats"].get("rs_fused", 0) > 0, res


def test_tp2_model_uses_fused_collectives():
    _need(2)
    flat = _flat(tensor_parallel_size=2, data_parallel_shard_size=1)
    flat["max_seq_len"] = 512
    ref = run_ranks(1, dict(_flat(), max_seq_len=512), device="cuda")
    got = run_ranks(2, flat, device="cuda")
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 4e-2, (ref, got)
    assert got.get("tp_fused", {}).get("ag_fused", 0) > 0, got


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_ep_dispatcher_matches_nccl_dispatcher(world):
    """Device-side count exchange, P2P row pushes and pulls against the NCCL all-to-all dispatcher, values and gradients."""
    _need(world)
    from fused_ep_cases import run_fused_ep
    res = run_fused_ep(world)
    for k in ("out", "dx", "dw", "dparam"):
        assert res[k] < 2e-2, res
    assert res["stats"]["dispatches"] > 0 and res["stats"]["combines"] > 0


@pytest.mark.parametrize("name,flat,arch", [
    ("tp2_fsdp2", dict(tensor_parallel_size=2, data_parallel_shard_size=2, activation_checkpoint_mode="full"), None),
    ("ep2_fsdp4", dict(model_name_or_path="qwen3_moe", expert_parallel_size=2, data_parallel_shard_size=4, activation_checkpoint_mode="full"), MOE),
    ("hsdp2x2", dict(data_parallel_replicate_size=2, data_parallel_shard_size=2), None),
])
def test_mixed_parallel_modes_on_four_gpus(name, flat, arch):
    """Fused FSDP collectives together with fused TP / EP exchanges, each on its own sub-group arena."""
    _need(4)
    base = dict(model_name_or_path=flat.get("model_name_or_path", "qwen3"))
    ref = run_ranks(1, _flat(**base), arch=arch, device="cuda")
    got = run_ranks(4, _flat(**flat), arch=arch, device="cuda")
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 4e-2, (name, ref, got)


def test_peer_ep_capacity_overflow_is_reported_not_written():
    """All copies routed to one rank with a receive buffer sized for the average: rows that do not fit are dropped, the
    status word says so, and the context stays usable."""
    _need(2)
    from fused_ep_cases import run_fused_ep
    res = run_fused_ep(2, iters=1, overflow=True)
    assert res["overflow_seen"] == 1.0, res


def test_peer_ep_default_capacity_takes_every_token_on_one_rank():
    """Default (worst-case) receive buffers: every copy of every rank routed to rank 0's experts is exchanged without a
    drop and matches the NCCL all-to-all dispatcher."""
    _need(2)
    from fused_ep_cases import run_fused_ep
    res = run_fused_ep(2, iters=2, skew=True)
    assert res["out"] < 2e-2 and res["dx"] < 2e-2 and res["dw"] < 2e-2 and res["dparam"] < 3e-2, res


def test_peer_that_never_arrives_becomes_an_error_on_every_rank():
    """Failure detection on the device without a fault: a host rank skips its launch, the waiting kernel gives up after
    its poll limit, and both ranks raise through the error-coordination boundary; the symmetric arena is untouched."""
    _need(2)
    from fused_tp_cases import run_absent_peer
    (v0, ok0), (v1, ok1) = run_absent_peer(2)
    assert v0.startswith("own:") and "flag" in v0 and "7401" in v0, (v0, v1)
    assert v1.startswith("peer:") and "all-gather of step 7" in v1, (v0, v1)
    assert ok0 and ok1


HYBRID = dict(head_dim=64, delta_heads=4, delta_head_dim=64, kv_lora_rank=64, qk_rope_dim=32)


@pytest.mark.parametrize("name,flat", [
    ("kda_mla_kcp2", dict(model_name_or_path="hybrid_kda_mla", context_parallel_kcp_size=2, data_parallel_shard_size=1)),
    ("gdn_tp2", dict(model_name_or_path="hybrid_gdn", tensor_parallel_size=2, data_parallel_shard_size=1)),
    ("kda_mla_tp2", dict(model_name_or_path="hybrid_kda_mla", tensor_parallel_size=2, data_parallel_shard_size=1)),
])
def test_hybrid_families_sequence_and_tensor_parallel_on_gpus(name, flat):
    """Delta-rule state handed across ranks (kcp) and the mixers' own tensor-parallel cuts, on NCCL and the CUDA kernels."""
    _need(2)
    base = dict(model_name_or_path=flat["model_name_or_path"], num_hidden_layers=4)
    ref = run_ranks(1, _flat(**base), arch=HYBRID, device="cuda")
    got = run_ranks(2, _flat(num_hidden_layers=4, **flat), arch=HYBRID, device="cuda")
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 4e-2, (name, ref, got)


FAITHFUL = dict(head_dim=64, linear_heads=4, linear_head_dim=64, kda_chunk_size=16, qk_nope_head_dim=32, qk_rope_head_dim=32, v_head_dim=64,
                kv_lora_rank=64, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=64, linear_value_head_dim=64,
                linear_chunk_size=32)


@pytest.mark.parametrize("name,flat", [
    ("kimi_linear_kcp2", dict(model_name_or_path="kimi_linear", context_parallel_kcp_size=2, data_parallel_shard_size=1)),
    ("kimi_k3_kcp2", dict(model_name_or_path="kimi_k3", context_parallel_kcp_size=2, data_parallel_shard_size=1)),
    ("qwen3_5_moe_kv2", dict(model_name_or_path="qwen3_5_moe", context_parallel_kv_allgather_size=2, data_parallel_shard_size=1)),
    ("deepseek_v4_kv2", dict(model_name_or_path="deepseek_v4", context_parallel_kv_allgather_size=2, data_parallel_shard_size=1)),
    ("deepseek_v4_ep2", dict(model_name_or_path="deepseek_v4", expert_parallel_size=2, data_parallel_shard_size=2)),
])
def test_model_families_sequence_and_expert_parallel_on_gpus(name, flat):
    """The families' own sequence-parallel paths on NCCL and the CUDA kernels: convolution history and recurrent state
    handed across ranks (Kimi, Qwen3.5), the gathered shared key/value head and compressor inputs (DeepSeek-V4), and
    hash-routed plus biased top-k experts under expert parallelism."""
    _need(2)
    arch = {k: v for k, v in FAITHFUL.items() if v is not None}
    if flat["model_name_or_path"] == "deepseek_v4":
        arch = dict(head_dim=64, qk_rope_head_dim=16, index_head_dim=32, q_lora_rank=64, o_lora_rank=32, sliding_window=32)
    base = dict(model_name_or_path=flat["model_name_or_path"], num_hidden_layers=4)
    ref = run_ranks(1, _flat(**base), arch=arch, device="cuda")
    got = run_ranks(2, _flat(num_hidden_layers=4, **flat), arch=arch, device="cuda")
    assert max(abs(a - b) for a, b in zip(ref["loss"], got["loss"])) < 5e-2, (name, ref, got)
