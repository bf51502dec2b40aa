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
