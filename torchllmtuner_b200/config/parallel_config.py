"""Parallelism config groups (reference: llmtuner/config/parallel_config.py:39-473)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..errors import ConfigError
from .utils import require_bool, require_choice, require_integer_at_least, require_string_patterns

CP_STRATEGIES = ("kv_allgather", "ulysses", "kcp")
CP_LOAD_BALANCERS = (None, "headtail", "ptrr")
EP_DISPATCHERS = ("alltoall", "fused", "torchao", "domino", "mc2", "deepep", "hybridep")
EP_DISPATCHER_GAPS = ("deepep", "hybridep", "mc2", "torchao")


@dataclass
class FSDPConfig:
    fsdp_reshard_after_forward: str = "default"          # default | always | never
    fsdp_reduce_dtype: str = "float32"                   # float32 | bfloat16 | float64
    fsdp_cpu_offload: bool = False
    fsdp_cpu_offload_pin_memory: bool = True
    fsdp_forward_prefetch_count: int = 0
    fsdp_backward_prefetch_count: int = 0
    fsdp_apply_modules: dict[str, dict[str, Any]] = field(default_factory=dict)
    fsdp_ignored_modules: list[str] = field(default_factory=list)
    fsdp_implementation: str = "native"                  # native (fused P2P kernels) | custom (NCCL arm)
    enable_fsdp_symm_mem: bool = False
    fsdp_symm_mem_scope: str = "all"                     # all | dense
    fsdp_expert_reduce_layout: str = "storage"           # storage | split
    fsdp_expert_reduce_workspace_limit_bytes: int = 0

    def __post_init__(self):
        require_choice("fsdp_reshard_after_forward", self.fsdp_reshard_after_forward, ("default", "always", "never"))
        require_choice("fsdp_reduce_dtype", self.fsdp_reduce_dtype, ("float32", "bfloat16", "float64"))
        require_bool("fsdp_cpu_offload", self.fsdp_cpu_offload)
        require_integer_at_least("fsdp_forward_prefetch_count", self.fsdp_forward_prefetch_count, 0)
        require_integer_at_least("fsdp_backward_prefetch_count", self.fsdp_backward_prefetch_count, 0)
        require_choice("fsdp_implementation", self.fsdp_implementation, ("native", "custom"))
        require_choice("fsdp_symm_mem_scope", self.fsdp_symm_mem_scope, ("all", "dense"))
        require_choice("fsdp_expert_reduce_layout", self.fsdp_expert_reduce_layout, ("storage", "split"))
        require_string_patterns("fsdp_ignored_modules", self.fsdp_ignored_modules)
        if self.fsdp_cpu_offload and self.enable_fsdp_symm_mem:
            raise ConfigError("enable_fsdp_symm_mem cannot be combined with fsdp_cpu_offload")


@dataclass
class TensorParallelConfig:
    enable_sequence_parallel: bool = True
    tp_colwise_modules: list[str] = field(default_factory=list)
    tp_rowwise_modules: list[str] = field(default_factory=list)
    tp_sequence_modules: list[str] = field(default_factory=list)
    # Shard the head over the vocabulary like the embedding (vocabulary-parallel cross-entropy). False keeps the head
    # replicated with its gradient all-reduced over the TP group, which is the only layout the reference accepts under
    # sequence-parallel TP.
    tp_vocab_parallel_head: bool = True

    def __post_init__(self):
        require_bool("enable_sequence_parallel", self.enable_sequence_parallel)
        require_bool("tp_vocab_parallel_head", self.tp_vocab_parallel_head)
        for n in ("tp_colwise_modules", "tp_rowwise_modules", "tp_sequence_modules"):
            require_string_patterns(n, getattr(self, n))


@dataclass
class ContextParallelConfig:
    context_parallel_strategy: str = "kv_allgather"
    context_parallel_load_balancer: str | None = None

    def __post_init__(self):
        require_choice("context_parallel_strategy", self.context_parallel_strategy, CP_STRATEGIES)
        require_choice("context_parallel_load_balancer", self.context_parallel_load_balancer, CP_LOAD_BALANCERS)
        if self.context_parallel_load_balancer == "ptrr":
            raise ConfigError("context_parallel_load_balancer='ptrr' is not supported")


@dataclass
class ExpertParallelConfig:
    router_aux_loss_coef: float | None = None
    moe_quantile_balancing: bool = False
    fixed_router: bool = False
    ep_token_dispatcher: str = "alltoall"
    # Receive-buffer size of the peer-memory dispatcher as a multiple of the balanced load (token copies per rank).
    # None (default) sizes the buffers for the worst case, expert_parallel_size times the balanced load (every token of
    # every rank routed to one rank), so no routing skew can drop a row: at EP=8, 4096 tokens, top-8 and hidden 2048 that is
    # 1 GiB per buffer. A smaller factor saves memory; rows beyond it are dropped and reported through the kernel status
    # word (the step then raises).
    ep_capacity_factor: float | None = None
    ep_torchao_pad_multiple: int = 16

    def __post_init__(self):
        require_choice("ep_token_dispatcher", self.ep_token_dispatcher, EP_DISPATCHERS)
        if self.ep_token_dispatcher in EP_DISPATCHER_GAPS:
            raise ConfigError(f"ep_token_dispatcher={self.ep_token_dispatcher!r} is a registered gap on this platform; "
                              "use 'alltoall', 'fused' or 'domino'")
        if self.router_aux_loss_coef is not None and not (self.router_aux_loss_coef >= 0):
            raise ConfigError("router_aux_loss_coef must be >= 0")
        require_integer_at_least("ep_torchao_pad_multiple", self.ep_torchao_pad_multiple, 1)
        if self.ep_capacity_factor is not None and not (self.ep_capacity_factor >= 1.0):
            raise ConfigError("ep_capacity_factor must be >= 1")


@dataclass
class ParallelConfig:
    fsdp_config: FSDPConfig = field(default_factory=FSDPConfig)
    tp_config: TensorParallelConfig = field(default_factory=TensorParallelConfig)
    cp_config: ContextParallelConfig = field(default_factory=ContextParallelConfig)
    ep_config: ExpertParallelConfig = field(default_factory=ExpertParallelConfig)
    data_parallel_replicate_size: int = 1
    data_parallel_shard_size: int = -1
    tensor_parallel_size: int = 1
    context_parallel_kv_allgather_size: int = 1
    context_parallel_ulysses_size: int = 1
    context_parallel_kcp_size: int = 1
    expert_parallel_size: int = 1
    pipeline_parallel_size: int = 1              # experiment axis (outermost); 1 in production runs
    train_timeout_seconds: int = 100

    def __post_init__(self):
        for n in ("data_parallel_replicate_size", "tensor_parallel_size", "context_parallel_kv_allgather_size",
                  "context_parallel_ulysses_size", "context_parallel_kcp_size", "expert_parallel_size",
                  "pipeline_parallel_size", "train_timeout_seconds"):
            require_integer_at_least(n, getattr(self, n), 1)
        if self.data_parallel_shard_size != -1:
            require_integer_at_least("data_parallel_shard_size", self.data_parallel_shard_size, 1)
        if self.tensor_parallel_size > 1 and not self.tp_config.enable_sequence_parallel:
            raise ConfigError("tensor parallelism is sequence-parallel here: enable_sequence_parallel must stay True when tp > 1")

    @property
    def cp_size(self) -> int:
        return (self.context_parallel_kv_allgather_size * self.context_parallel_ulysses_size
                * self.context_parallel_kcp_size)

    def derive_dp(self, world_size: int) -> tuple[int, int]:
        """(dp_replicate, dp_shard) for `world_size`; dp_shard=-1 takes what is left."""
        fixed = self.data_parallel_replicate_size * self.cp_size * self.tensor_parallel_size * self.pipeline_parallel_size
        shard = self.data_parallel_shard_size
        if shard == -1:
            if world_size % fixed:
                raise ConfigError(f"world size {world_size} is not divisible by dp_replicate*cp*tp*pp = {fixed}")
            shard = world_size // fixed
        if fixed * shard != world_size:
            raise ConfigError(f"dp_replicate*dp_shard*cp*tp*pp = {fixed * shard} != world size {world_size}")
        return self.data_parallel_replicate_size, shard
