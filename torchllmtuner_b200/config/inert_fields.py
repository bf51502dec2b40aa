"""Flags that are accepted so that a command line written for the reference still parses, but that select something this
platform does not have (another vendor's back end, a tracing compiler, an optional third-party library). Setting one of
them to a non-default value has no effect; the trainer says so once at start-up instead of staying silent."""
from __future__ import annotations

import dataclasses

INERT_FIELDS: dict[str, str] = {
    "norm_backend": "RMSNorm always runs the in-tree sm_100a kernel (CUDA) or the PyTorch statement (CPU)",
    "attention_backend": "attention always runs the in-tree tcgen05 kernel (CUDA) or the PyTorch statement (CPU)",
    "linear_attention_backend": "delta-attention mixers use the in-tree PyTorch statement",
    "router_compute_dtype": "router logits and scores are always fp32",
    "rotary_init_device": "rotary tables are built on the compute device",
    "rotary_compute_dtype": "rotary tables are always fp32",
    "rotary_cache_dtype": "rotary tables are always fp32",
    "fsdp_cpu_offload_pin_memory": "host-resident optimizer state is always pinned",
    "enable_fsdp_symm_mem": "the native FSDP runtime always uses its own symmetric arena on CUDA (LLMT_DISABLE_FUSED_COMM=1 turns it off)",
    "fsdp_symm_mem_scope": "see enable_fsdp_symm_mem",
    "fsdp_expert_reduce_workspace_limit_bytes": "expert gradients are reduced in storage order, without a workspace",
    "tp_sequence_modules": "sequence boundaries are placed by the model's TP plan",
    "context_parallel_strategy": "the strategy follows from which context-parallel degree is > 1",
    "ep_torchao_pad_multiple": "the torchao dispatcher is not available; segments are padded to 128 rows",
    "swap_prefetch": "host-resident moments are streamed through two device slots: the upload of the next slice always overlaps the current update",
    "swap_memory_fraction": "the slice size comes from swap_max_device_bytes",
    "swap_max_host_bytes": "pinned host memory for the moments is not capped",
    "compute_sharding_by_fqn": "Muon jobs are placed by cost (longest first on the least loaded rank, ties to the storing rank)",
    "bucket_configs": "Muon redistribution is one all-to-all per sharding unit each way",
    "sharded_expert_parallel": "checkpoints always hold whole tensors written as boxes, which resume at any EP degree",
    "sharded_tensor_parallel": "checkpoints always hold whole tensors written as boxes, which resume at any TP degree",
    "global_context_rows": "rows are assigned to data-parallel ranks by contiguous slices",
    "streaming_shuffle_buffer_size": "only used by `datasets.sources.StreamingSource` when a recipe builds one",
    "mm_pad_token": "multimodal padding uses the tokenizer's pad id",
    "disable_color_printing": "console output is never coloured",
    "npu_profiler_level": "no NPU profiler on this platform",
    "profiler_skip_first_wait": "the profiler schedule has no separate first-cycle wait",
    "enable_async_tensor_parallel": "TP collectives are fused into the GEMM kernels, there is no compiler pass to enable",
    "determinism_check": "activation recomputation is bitwise deterministic by construction (same kernels, same order)",
}

# Flags whose non-default value would CHANGE what is trained or how gradients are formed, and that this platform does not
# implement: setting one raises instead of being ignored. Value: (accepted default values, reason).
UNSUPPORTED_FIELDS: dict[str, tuple[tuple, str]] = {
    "grad_norm_precision": (("float32",), "the gradient norm is accumulated in fp32 over the fp32 gradient shards; a norm "
                                           "taken in the parameter dtype is not implemented"),
    "fsdp_expert_reduce_layout": (("storage",), "expert gradients are reduced in storage order; the split gate / up / down "
                                                 "reduce layout is not implemented"),
}


def _walk(obj, prefix=""):
    if not dataclasses.is_dataclass(obj):
        return
    for f in dataclasses.fields(obj):
        v = getattr(obj, f.name)
        if dataclasses.is_dataclass(v):
            yield from _walk(v, prefix + f.name + ".")
        else:
            yield f, v


def check_unsupported_fields(config) -> None:
    """Raises `UnsupportedCombinationError` for the first semantics-changing flag set to a value this platform lacks."""
    from ..errors import UnsupportedCombinationError
    for f, v in _walk(config):
        rule = UNSUPPORTED_FIELDS.get(f.name)
        if rule is not None and v not in rule[0] and v not in (None, [], ()):
            raise UnsupportedCombinationError(f"--{f.name}={v!r} is not supported: {rule[1]}")


def inert_fields_set(config) -> list[tuple[str, str]]:
    """(field, reason) for every inert field whose value differs from its default."""
    out = []
    for f, v in _walk(config):
        if f.name not in INERT_FIELDS:
            continue
        default = f.default if f.default is not dataclasses.MISSING else (f.default_factory() if f.default_factory is not dataclasses.MISSING else None)
        if v != default:
            out.append((f.name, INERT_FIELDS[f.name]))
    return out
