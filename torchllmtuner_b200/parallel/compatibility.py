"""Compatibility matrix: which feature combinations are supported, checked before any mutation of the model
(reference: llmtuner/parallel/compatibility.py:108-373). Each entry is (name, predicate(ctx) -> bool violated, message)."""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import UnsupportedCombinationError


@dataclass
class CompatContext:
    config: object
    topo: object
    model_config: object      # the architecture config (e.g. Qwen3Config)


def _has_moe(ctx) -> bool:
    return getattr(ctx.model_config, "num_experts", 0) > 0


ENTRIES = (
    ("ep_without_experts", lambda c: c.topo.ep > 1 and not _has_moe(c), "expert_parallel_size > 1 needs a model with routed experts"),
    ("ep_divides_experts", lambda c: c.topo.ep > 1 and _has_moe(c) and c.model_config.num_experts % c.topo.ep != 0,
     "expert_parallel_size must divide num_experts"),
    ("tp_divides_heads", lambda c: c.topo.tp > 1 and (c.model_config.num_attention_heads % c.topo.tp or c.model_config.num_key_value_heads % c.topo.tp),
     "tensor_parallel_size must divide the query and key/value head counts"),
    ("ulysses_divides_heads", lambda c: c.topo.cp_ulysses > 1 and ((c.model_config.num_key_value_heads // max(1, c.topo.tp)) % c.topo.cp_ulysses),
     "ulysses degree must divide the per-rank key/value head count"),
    ("kcp_needs_delta_attention", lambda c: c.topo.kcp > 1 and getattr(c.model_config, "model_type", "") not in ("kimi_linear", "kimi_k3", "hybrid_kda_mla"),
     "context_parallel_kcp_size > 1 is defined for delta-attention models only"),
    ("ptrr_backstop", lambda c: c.config.parallel.cp_config.context_parallel_load_balancer == "ptrr", "ptrr load balancing is not supported"),
    ("headtail_needs_kv_allgather", lambda c: c.config.parallel.cp_config.context_parallel_load_balancer == "headtail" and c.topo.cp_ulysses > 1 and c.topo.cp_kv == 1,
     "headtail balancing applies to the kv_allgather axis; the ulysses axis keeps contiguous shards"),
    ("shared_expert_tp", lambda c: c.topo.tp > 1 and c.topo.ep > 1 and getattr(c.model_config, "shared_expert_intermediate_size", 0) > 0,
     "shared experts under TP together with EP are not supported"),
    ("quantile_routing_bias", lambda c: getattr(c.model_config, "moe_quantile_balancing", False) and getattr(c.model_config, "router_bias_update_coeff", 0) > 0,
     "quantile balancing and aux-loss-free bias balancing are mutually exclusive"),
    ("chunked_loss_tied_tp", lambda c: c.config.training.chunked_loss_num_chunks > 0 and c.topo.tp > 1 and getattr(c.model_config, "tie_word_embeddings", False),
     "chunked loss with tied embeddings under tensor parallelism is not supported"),
    ("validation_pp", lambda c: c.topo.pp > 1 and c.config.training.validation_config is not None, "validation inside the pipeline experiment is not supported"),
    ("domino_needs_ep", lambda c: c.config.parallel.ep_config.ep_token_dispatcher == "domino" and c.topo.ep == 1,
     "the domino dispatcher overlaps expert-parallel traffic and needs expert_parallel_size > 1"),
    ("cpu_offload_host_moments", lambda c: c.config.parallel.fsdp_config.fsdp_cpu_offload and c.config.optimizer.state_residency == "host",
     "fsdp_cpu_offload already keeps the optimizer state on the host"),
)


def check_compatibility(config, topo, model_config) -> None:
    ctx = CompatContext(config, topo, model_config)
    for name, violated, msg in ENTRIES:
        try:
            bad = violated(ctx)
        except AttributeError:
            bad = False
        if bad:
            raise UnsupportedCombinationError(f"[{name}] {msg}")
