"""Execution layout: what one rank's forward pass consumes and produces under the resolved parallel plans
(reference: llmtuner/parallel/execution.py:21-158).

Resolved once, together with the stage plans and before any model mutation, from the configuration, the topology and the
plans. The trainer reads it instead of re-deriving the same facts in several places:
  * `sequence_shard_axes`: the mesh axes that cut the token dimension of the activations a rank holds (context parallel
    first, then tensor parallel, which is sequence-parallel here); `tokens_per_rank(seq)` follows from them;
  * `output_kind`: "hidden" when the loss consumes hidden states (chunked head + CE, always with a vocabulary-sharded
    head) or "logits";
  * `vocabulary_sharded`: the head is cut over the tensor-parallel group. The reference rejects that layout under
    sequence-parallel TP (execution.py:127-132); here it is the default, because the loss kernel exchanges its per-token
    statistics over the same group and the gather / reduce-scatter ride on the head's GEMMs;
  * `loss_chunks`: token chunks of the head + CE.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError, UnsupportedCombinationError


@dataclass(frozen=True)
class ExecutionLayout:
    output_kind: str                      # "hidden" | "logits"
    sequence_shard_axes: tuple[str, ...]  # subset of ("cp", "tp"), outermost first
    sequence_shards: int                  # product of the degrees of those axes
    vocabulary_sharded: bool
    loss_chunks: int
    load_balancer: str | None = None      # "headtail" cuts the sequence into 2 * cp chunks

    def __post_init__(self):
        if self.output_kind not in ("hidden", "logits"):
            raise ValueError(f"output_kind {self.output_kind!r}")
        if self.vocabulary_sharded and self.output_kind != "hidden":
            raise UnsupportedCombinationError("a vocabulary-sharded head produces no full logits: the loss has to take hidden states")

    def tokens_per_rank(self, tokens: int) -> int:
        if tokens % self.sequence_shards:
            raise ConfigError(f"{tokens} tokens do not divide over {self.sequence_shards} sequence shards {self.sequence_shard_axes}")
        return tokens // self.sequence_shards

    def validate_sequence_length(self, seq_len: int, cp: int) -> None:
        quantum = self.sequence_shards * (2 if self.load_balancer == "headtail" and cp > 1 else 1)
        if seq_len % quantum:
            raise ConfigError(f"max_seq_len {seq_len} must be a multiple of {quantum} "
                              f"(sequence shards {self.sequence_shard_axes}" + (", head-tail balance" if quantum != self.sequence_shards else "") + ")")


def resolve_execution_layout(config, topo, model, plans: dict | None = None) -> ExecutionLayout:
    plans = plans or {}
    axes = tuple(a for a, d in (("cp", topo.cp), ("tp", topo.tp)) if d > 1)
    shards = (topo.cp if topo.cp > 1 else 1) * (topo.tp if topo.tp > 1 else 1)
    tp_plan = plans.get("tp")
    vocab = bool(tp_plan is not None and any(t.kind == "head" and t.layout == "vocab" for t in tp_plan.targets))
    chunks = int(config.training.chunked_loss_num_chunks)
    kind = "hidden" if (chunks > 0 or vocab) else "logits"
    lb = config.parallel.cp_config.context_parallel_load_balancer if topo.cp > 1 else None
    layout = ExecutionLayout(kind, axes, shards, vocab, max(1, chunks) if kind == "hidden" else 0, lb)
    layout.validate_sequence_length(config.training.max_seq_len, topo.cp)
    return layout
