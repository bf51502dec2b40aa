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
