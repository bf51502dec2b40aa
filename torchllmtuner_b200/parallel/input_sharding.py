"""Context- and tensor-parallel sharding of model inputs
(reference: llmtuner/parallel/context_parallel/input_sharding.py:22-270).

CP first, then TP. CP cuts the packed row axis of every sequence into `cp` contiguous chunks, or with `headtail`
balancing into `2*cp` chunks of which rank r owns chunks r and 2cp-1-r. TP (sequence parallel) cuts tokens and
targets into `tp` contiguous parts in mesh-rank order; positions stay whole for the rows a rank's attention sees.
Document boundaries travel as global `cu_seqlens`, which is what lets packed rows be used under CP.
"""
from __future__ import annotations

import torch

from ..errors import ConfigError


def headtail_chunks(seq_len: int, cp: int, rank: int) -> list[tuple[int, int]]:
    if seq_len % (2 * cp):
        raise ConfigError(f"headtail load balancing needs seq_len ({seq_len}) divisible by 2*cp ({2 * cp})")
    c = seq_len // (2 * cp)
    return [(rank * c, (rank + 1) * c), ((2 * cp - 1 - rank) * c, (2 * cp - rank) * c)]


def contiguous_chunk(seq_len: int, n: int, rank: int) -> tuple[int, int]:
    if seq_len % n:
        raise ConfigError(f"sequence length {seq_len} is not divisible by {n}")
    c = seq_len // n
    return rank * c, (rank + 1) * c


def cp_row_index(batch: int, seq: int, cp: int, rank: int, load_balancer: str | None) -> torch.Tensor:
    """Global packed-row indices (into [B*S]) owned by CP rank `rank`, in local order."""
    if load_balancer == "headtail":
        spans = headtail_chunks(seq, cp, rank)
    else:
        spans = [contiguous_chunk(seq, cp, rank)]
    per_seq = torch.cat([torch.arange(a, b) for a, b in spans])
    return (torch.arange(batch)[:, None] * seq + per_seq[None, :]).reshape(-1)


def shard_model_inputs(inputs: dict, parallel_dims) -> dict:
    """`inputs` as produced by `prepare_inputs` (host tensors). `parallel_dims` is a dict-like with keys
    cp, cp_rank, tp, tp_rank, load_balancer (or None for no sharding)."""
    if parallel_dims is None:
        return inputs
    cp, tp = int(parallel_dims.get("cp", 1)), int(parallel_dims.get("tp", 1))
    if cp == 1 and tp == 1:
        return inputs
    out = dict(inputs)
    B, S = inputs["batch"], inputs["seq"]
    rows = torch.arange(B * S)
    if cp > 1:
        kv, ul = int(parallel_dims.get("cp_kv", 1)), int(parallel_dims.get("cp_ulysses", 1))
        if kv > 1 and ul > 1:
            # two levels: the key/value axis cuts the sequences (optionally head-tail balanced); the ulysses axis cuts each
            # rank's rows of that level into contiguous parts, so that its all-to-all restores exactly those rows
            rows_kv = cp_row_index(B, S, kv, int(parallel_dims["cp_kv_rank"]), parallel_dims.get("load_balancer"))
            if rows_kv.numel() % ul:
                raise ConfigError(f"{rows_kv.numel()} rows per key/value rank are not divisible by the ulysses degree {ul}")
            n = rows_kv.numel() // ul
            u = int(parallel_dims["cp_ulysses_rank"])
            rows = rows_kv[u * n:(u + 1) * n]
        else:
            rows = cp_row_index(B, S, cp, int(parallel_dims["cp_rank"]), parallel_dims.get("load_balancer"))
        out["cp_rows"] = rows                      # which global rows this rank's queries are
        out["global_cu_seqlens"] = inputs["cu_seqlens"]
        out["global_rows"] = B * S
    out["positions"] = inputs["positions"][rows]
    tok, tgt = inputs["tokens"][rows], inputs["targets"][rows]
    if tp > 1:
        a, b = contiguous_chunk(tok.shape[0], tp, int(parallel_dims["tp_rank"]))
        tok, tgt = tok[a:b], tgt[a:b]
        out["tp_span"] = (a, b)
    out["tokens"], out["targets"] = tok, tgt
    return out
