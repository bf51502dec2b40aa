"""Batch services of a step (reference: llmtuner/trainer/runtime/batch.py:34-330): reading a micro-batch with a
three-state agreement between ranks, counting the valid tokens of the optimizer step over the data-parallel ranks, and
moving a trainer batch to the compute device."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...datasets.contracts import DataloaderExhaustedError

READY, EXHAUSTED, FAILED = 2, 1, 0


def fetch_batch(data_iterator, env):
    """Read one micro-batch; all ranks agree on (ready / exhausted / error) with one MIN all-reduce, so that no rank
    enters the step's collectives alone."""
    state, batch, err = READY, None, None
    try:
        batch = next(data_iterator)
    except (StopIteration, DataloaderExhaustedError):
        state = EXHAUSTED
    except Exception as e:  # noqa: BLE001
        state, err = FAILED, e
    if dist.is_initialized() and env.world_size > 1:
        dev = env.device if env.device.type == "cuda" else torch.device("cpu")
        s = torch.tensor([state], dtype=torch.int32, device=dev)
        dist.all_reduce(s, op=dist.ReduceOp.MIN)
        agreed = int(s.item())
    else:
        agreed = state
    if agreed == FAILED:
        raise err if err is not None else RuntimeError("a peer rank failed while reading data")
    if agreed == EXHAUSTED:
        raise DataloaderExhaustedError("the data loader is exhausted on at least one rank")
    return batch


def global_valid_tokens(batches, device, reductions) -> torch.Tensor:
    """Scalar fp32 device tensor: valid target tokens of the whole optimizer step, summed over the data-parallel ranks.
    The loss of every rank is its sum of token losses divided by this number."""
    local_valid = sum(int(b["num_valid_tokens"]) for b in batches)
    gv = torch.tensor([float(local_valid)], dtype=torch.float32, device=device)
    if reductions.dp_group is not None:
        dist.all_reduce(gv, group=reductions.dp_group)
    return gv.reshape(())
