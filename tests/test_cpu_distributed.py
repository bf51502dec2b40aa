"""Two-arm equivalence on CPU/gloo ranks: the sharded/parallel arm must reproduce the single-rank loss curve."""
import pytest

from dist_cases import base_flat, run_ranks


def _close(a, b, tol):
    assert len(a) == len(b)
    assert max(abs(x - y) for x, y in zip(a, b)) < tol, (a, b)


def test_fsdp2_matches_single_rank():
    ref = run_ranks(1, base_flat())
    for ac in ("none", "full"):
        got = run_ranks(2, base_flat(data_parallel_shard_size=2, activation_checkpoint_mode=ac))
        _close(ref["loss"], got["loss"], 2e-5)
        _close(ref["grad_norm"], got["grad_norm"], 2e-4)


def test_hsdp_and_accumulation_match_single_rank():
    ref = run_ranks(1, base_flat())
    got = run_ranks(4, base_flat(data_parallel_replicate_size=2, data_parallel_shard_size=2))
    _close(ref["loss"], got["loss"], 2e-5)
    got = run_ranks(2, base_flat(data_parallel_shard_size=2, gradient_accumulation_steps=2))
    _close(ref["loss"], got["loss"], 2e-5)


def test_tp2_matches_single_rank():
    ref = run_ranks(1, base_flat())
    got = run_ranks(2, base_flat(tensor_parallel_size=2, data_parallel_shard_size=1))
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


def test_tp2_dp2_matches_single_rank():
    ref = run_ranks(1, base_flat())
    got = run_ranks(4, base_flat(tensor_parallel_size=2, data_parallel_shard_size=2, activation_checkpoint_mode="full"))
    _close(ref["loss"], got["loss"], 5e-5)


def test_fsdp_ignored_modules_are_reduced_and_stepped():
    """Parameters named by `fsdp_ignored_modules` stay whole on every rank; their gradient is summed over the data ranks
    and the optimizer steps them, so the curve equals the fully sharded one (and differs from a run that froze them)."""
    ref = run_ranks(1, base_flat())
    got = run_ranks(2, base_flat(data_parallel_shard_size=2, fsdp_ignored_modules=["layers\\.1\\.mlp", "norm"]))
    _close(ref["loss"], got["loss"], 2e-5)
    _close(ref["grad_norm"], got["grad_norm"], 2e-4)


def test_fsdp_pattern_units_match_single_rank():
    """`fsdp_apply_modules`: selected modules become sharding units of their own (two same-size projections of one block
    included); the curve is unchanged, with and without activation checkpointing."""
    ref = run_ranks(1, base_flat())
    pats = ["model.layers.{0-1}.mlp.gate_proj", "model.layers.{0-1}.mlp.up_proj", "model.layers.*.self_attn"]
    for ac in ("none", "full"):
        got = run_ranks(2, base_flat(data_parallel_shard_size=2, fsdp_apply_modules=pats, activation_checkpoint_mode=ac))
        _close(ref["loss"], got["loss"], 2e-5)
        _close(ref["grad_norm"], got["grad_norm"], 2e-4)


def test_single_rank_accumulation_matches_one_large_batch():
    """One shard rank with gradient accumulation accumulates in fp32: four micro-batches equal one batch of four rows."""
    ref = run_ranks(1, base_flat())
    got = run_ranks(1, base_flat(gradient_accumulation_steps=4))
    _close(ref["loss"], got["loss"], 2e-5)
    _close(ref["grad_norm"], got["grad_norm"], 2e-4)


MOE = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)


def test_ep2_matches_single_rank():
    ref = run_ranks(1, base_flat(model_name_or_path="qwen3_moe"), arch=MOE)
    got = run_ranks(2, base_flat(model_name_or_path="qwen3_moe", expert_parallel_size=2, data_parallel_shard_size=2), arch=MOE)
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


def test_balance_loss_weight_is_independent_of_dp_and_accumulation():
    """The load-balance loss is a per-token-stream objective of weight `coef`: two micro-batches accumulated on one rank and
    the same two micro-batches on two data-parallel ranks give the same loss curve and the same gradient norm."""
    flat = dict(model_name_or_path="qwen3_moe", router_aux_loss_coef=0.5, learning_rate=1e-2)
    one = run_ranks(1, base_flat(gradient_accumulation_steps=2, **flat), arch=MOE)
    two = run_ranks(2, base_flat(data_parallel_shard_size=2, **flat), arch=MOE)
    _close(one["loss"], two["loss"], 5e-5)
    _close(one["grad_norm"], two["grad_norm"], 5e-4)
    off = run_ranks(1, base_flat(gradient_accumulation_steps=2, model_name_or_path="qwen3_moe", learning_rate=1e-2), arch=MOE)
    assert abs(off["grad_norm"][0] - one["grad_norm"][0]) > 1e-3        # the balance term does reach the gradient


def test_tp2_moe_matches_single_rank():
    """MoE block under tensor parallelism: rows gathered in, experts' intermediate dimension sharded, partial sums
    reduce-scattered out."""
    ref = run_ranks(1, base_flat(model_name_or_path="qwen3_moe"), arch=MOE)
    got = run_ranks(2, base_flat(model_name_or_path="qwen3_moe", tensor_parallel_size=2, data_parallel_shard_size=1), arch=MOE)
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


@pytest.mark.parametrize("flat", [dict(context_parallel_ulysses_size=2), dict(context_parallel_kv_allgather_size=2),
                                  dict(context_parallel_kv_allgather_size=2, context_parallel_load_balancer="headtail")])
def test_cp2_matches_single_rank(flat):
    ref = run_ranks(1, base_flat())
    got = run_ranks(2, base_flat(data_parallel_shard_size=1, **flat))
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


@pytest.mark.parametrize("schedule", ["GPipe", "1F1B", "Interleaved1F1B"])
def test_pipeline_two_stages_match_single_rank(schedule):
    from dist_cases import run_pp
    ref = run_ranks(1, base_flat(num_hidden_layers=4))
    got = run_pp(2, base_flat(num_hidden_layers=4, pipeline_parallel_size=2, data_parallel_shard_size=1), schedule)
    _close(ref["loss"], got["loss"], 5e-5)


def test_stage_split_rule():
    from torchllmtuner_b200.experiments.pipeline_parallel import split_layers
    assert split_layers(6, 2) == [(0, 3), (3, 6)]
    assert split_layers(7, 2) == [(0, 4), (4, 7)]          # the remainder goes to the first stage
    assert [b - a for a, b in split_layers(10, 4)] == [2, 3, 3, 2]


def test_interleaved_schedule_orders_messages_consistently():
    """Per direction of the pipeline, every rank's send order equals its neighbour's receive order, and a run with
    asynchronous sends / blocking receives never waits on a message that was not sent (simulated, no processes)."""
    from torchllmtuner_b200.experiments.pipeline_parallel.schedules import build_schedule, stages_per_rank
    for name, pp, M in [("1f1b", 4, 8), ("interleaved1f1b", 2, 4), ("interleaved1f1b", 4, 8), ("interleaved1f1b", 3, 6)]:
        V = stages_per_rank(name)
        S = pp * V
        acts = [build_schedule(name, r, pp, M) for r in range(pp)]
        sends, recvs = {}, {}
        for r in range(pp):
            for kind, c, mb in acts[r]:
                g = c * pp + r
                if kind == "F":
                    if g > 0:
                        recvs.setdefault(((g - 1) % pp, r, "f"), []).append((g - 1, mb))
                    if g < S - 1:
                        sends.setdefault((r, (g + 1) % pp, "f"), []).append((g, mb))
                else:
                    if g < S - 1:
                        recvs.setdefault(((g + 1) % pp, r, "b"), []).append((g + 1, mb))
                    if g > 0:
                        sends.setdefault((r, (g - 1) % pp, "b"), []).append((g, mb))
        assert sends == recvs, (name, pp, M)
        pos, done_f, done_b, moved = [0] * pp, set(), set(), True
        while moved:
            moved = False
            for r in range(pp):
                if pos[r] >= len(acts[r]):
                    continue
                kind, c, mb = acts[r][pos[r]]
                g = c * pp + r
                ready = (g == 0 or (g - 1, mb) in done_f) if kind == "F" else ((g, mb) in done_f and (g == S - 1 or (g + 1, mb) in done_b))
                if ready:
                    (done_f if kind == "F" else done_b).add((g, mb))
                    pos[r] += 1
                    moved = True
        assert all(pos[r] == len(acts[r]) for r in range(pp)) and len(done_b) == S * M, (name, pp, M)


@pytest.mark.parametrize("lb", [None, "headtail"])
def test_hybrid_context_parallel_kv_times_ulysses_matches_single_rank(lb):
    """cp = cp_kv x cp_ulysses: heads exchanged inside the ulysses axis, keys / values gathered over the other one."""
    flat = dict(context_parallel_kv_allgather_size=2, context_parallel_ulysses_size=2, data_parallel_shard_size=1)
    if lb:
        flat["context_parallel_load_balancer"] = lb
    ref = run_ranks(1, base_flat())
    got = run_ranks(4, base_flat(**flat))
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


def test_dist_muon_two_ranks_match_single_rank():
    """Muon needs whole matrices: owners gather their gradients, orthogonalise, and scatter the updates back."""
    ref = run_ranks(1, base_flat(optimizer_type="DistMuon", learning_rate=2e-2))
    got = run_ranks(2, base_flat(optimizer_type="DistMuon", learning_rate=2e-2, data_parallel_shard_size=2))
    _close(ref["loss"], got["loss"], 2e-3)


@pytest.mark.parametrize("family,flat", [("hybrid_kda_mla", dict(context_parallel_kcp_size=2)),
                                         ("hybrid_gdn", dict(context_parallel_kv_allgather_size=2))])
def test_delta_attention_families_under_sequence_parallelism(family, flat):
    """Delta-rule layers hand their recurrent state from rank to rank; the softmax / latent attention layers of the same
    model gather keys and values over the same axis."""
    arch = dict(head_dim=16, delta_heads=2, delta_head_dim=8, kv_lora_rank=16, qk_rope_dim=8, delta_chunk_size=8)
    base = dict(model_name_or_path=family, num_hidden_layers=4)
    ref = run_ranks(1, base_flat(**base), arch=arch)
    got = run_ranks(2, base_flat(data_parallel_shard_size=1, **base, **flat), arch=arch)
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


@pytest.mark.parametrize("family", ["hybrid_gdn", "hybrid_kda_mla"])
def test_hybrid_families_under_tensor_parallelism(family):
    """Every mixer names its own cut (delta rule: all projections by heads; latent attention: per-head projections cut,
    latent down-projection and rotary key whole; gated attention: q/k/v/gate by heads)."""
    arch = dict(head_dim=16, delta_heads=2, delta_head_dim=8, kv_lora_rank=16, qk_rope_dim=8, delta_chunk_size=8)
    base = dict(model_name_or_path=family, num_hidden_layers=4)
    ref = run_ranks(1, base_flat(**base), arch=arch)
    got = run_ranks(2, base_flat(tensor_parallel_size=2, data_parallel_shard_size=1, **base), arch=arch)
    _close(ref["loss"], got["loss"], 5e-5)
    _close(ref["grad_norm"], got["grad_norm"], 5e-4)


def test_dist_muon_plan_balances_work_and_prefers_the_storing_rank():
    from torchllmtuner_b200.components.optimizer.muon import MuonJob, ns_cost, plan_owners
    jobs = [MuonJob("a", 0, 1, 64, 64, (64, 64)), MuonJob("b", 4096, 1, 64, 64, (64, 64)), MuonJob("c", 8192, 1, 64, 256, (64, 256)),
            MuonJob("d", 24576, 1, 32, 32, (32, 32)), MuonJob("e", 25600, 1, 32, 32, (32, 32))]
    owners, loads = plan_owners(jobs, 2, 13312, 5)
    assert owners[2] == 1                                   # the largest job goes first; the tie goes to the rank storing more of it
    assert owners[0] == owners[1] == 0                      # the two mid-size matrices balance it on the other rank
    assert max(loads) - min(loads) <= ns_cost(64, 64, 1, 5)
    again, carried = plan_owners(jobs[:1], 2, 13312, 5, loads)
    assert again == [loads.index(min(loads))] and sum(carried) == sum(loads) + ns_cost(64, 64, 1, 5)


def test_dist_muon_orthogonalises_expert_matrices_and_fused_qkv_row_blocks():
    """Packed expert tensors are Muon matrices too (one per expert, runs of experts placed as jobs); with a fused QKV
    projection the query, key and value rows are orthogonalised separately. Two ranks reproduce one."""
    moe = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)
    base = dict(model_name_or_path="qwen3_moe", optimizer_type="DistMuon", learning_rate=2e-2, qkv_projection="fused")
    ref = run_ranks(1, base_flat(**base), arch=moe)
    got = run_ranks(2, base_flat(data_parallel_shard_size=2, **base), arch=moe)
    ep = run_ranks(2, base_flat(data_parallel_shard_size=2, expert_parallel_size=2, **base), arch=moe)
    _close(ref["loss"], got["loss"], 2e-3)
    _close(ref["loss"], ep["loss"], 2e-3)
    assert ref["loss"][-1] < ref["loss"][0]
