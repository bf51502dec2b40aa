"""Whole-tensor checkpoints written from flat shards, without ever building a whole tensor
(reference: llmtuner/components/checkpointer/core/chunked_tensor.py:26-216 reaches the same end with a tensor subclass that
carries local chunks under a global shape).

A rank of this framework owns, for each parameter, a range [lo, hi) of the flattened local tensor. On disk the
parameter is one N-D tensor with the reference's metadata: global shape plus a list of rectangular chunks. The bridge is
geometric: a flat range of a row-major tensor is the union of at most 2·N − 1 boxes (a ragged head, whole slabs, a
ragged tail, recursively per dimension), each of which is ALSO a contiguous run of the flat range, so a box's data is a
plain view of the shard, no copy. A tensor-, expert- or vocabulary-parallel cut is an offset of those boxes inside the
global tensor; rows that exist only as padding of a cut (a padded vocabulary) are clipped away.

`BoxSavePlanner` turns `{key#i: view}` entries plus a side table of (tensor name, global shape, box offsets) into torch
DCP write items that all point at the same tensor name; `BoxLoadPlanner` asks DCP's resharding helper which stored chunks
intersect each local box and reads straight into the views. The result resumes at any data-, expert- or tensor-parallel
degree, along any cut dimension, and any DCP reader (the reference's included) sees ordinary N-D tensors.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
from torch.distributed.checkpoint.metadata import (ChunkStorageMetadata, MetadataIndex, TensorProperties,
                                                   TensorStorageMetadata)
from torch.distributed.checkpoint.planner import LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType
from torch.distributed.checkpoint.planner_helpers import _create_read_items, _create_write_items, create_read_items_for_chunk_list

from ...errors import ConfigError, LLMTunerError

BOX_SEP = "#box"


class CheckpointIOError(LLMTunerError, RuntimeError):
    """A distributed-checkpoint save or load failed on at least one rank."""


@contextlib.contextmanager
def dcp_errors(what: str):
    """torch's `CheckpointException` derives from `BaseException`, so it slips past every `except Exception` between the
    checkpointer and the training loop's cleanup. Inside this block it is turned into this framework's errors: a
    `ConfigError` raised by a planner comes out as itself, anything else as `CheckpointIOError` naming the ranks."""
    from torch.distributed.checkpoint.api import CheckpointException
    try:
        yield
    except CheckpointException as e:
        failures = getattr(e, "failures", {}) or {}
        for rank in sorted(failures):
            cause = failures[rank]
            cause = cause[0] if isinstance(cause, tuple) else cause
            if isinstance(cause, LLMTunerError):
                raise cause from None
        ranks = sorted(failures)
        first = failures[ranks[0]] if ranks else e
        first = first[0] if isinstance(first, tuple) else first
        raise CheckpointIOError(f"{what} failed on ranks {ranks}: {type(first).__name__}: {first}") from None


def _prod(xs) -> int:
    n = 1
    for x in xs:
        n *= int(x)
    return n


def flat_range_boxes(lo: int, hi: int, shape) -> list[tuple[tuple[int, ...], tuple[int, ...], int]]:
    """Boxes (offsets, sizes, start) whose row-major concatenation, in order, is the flat range [lo, hi) of a tensor of
    `shape`; `start` is the position of the box's first element relative to `lo`."""
    shape = tuple(int(s) for s in shape)
    if not (0 <= lo <= hi <= _prod(shape)):
        raise ValueError(f"flat range [{lo}, {hi}) outside a tensor of shape {shape}")
    out: list[tuple[tuple[int, ...], tuple[int, ...], int]] = []

    def rec(lo_, hi_, dims, prefix_off, prefix_size, start):
        if hi_ <= lo_:
            return
        if len(dims) == 1:
            out.append((prefix_off + (lo_,), prefix_size + (hi_ - lo_,), start))
            return
        stride = _prod(dims[1:])
        r0, r1 = lo_ // stride, (hi_ - 1) // stride
        if r0 == r1:
            rec(lo_ - r0 * stride, hi_ - r0 * stride, dims[1:], prefix_off + (r0,), prefix_size + (1,), start)
            return
        first_full, last_full = r0, r1
        if lo_ % stride:
            rec(lo_ % stride, stride, dims[1:], prefix_off + (r0,), prefix_size + (1,), start)
            first_full = r0 + 1
        if hi_ % stride:
            last_full = r1 - 1
        if last_full >= first_full:
            out.append((prefix_off + (first_full,) + (0,) * (len(dims) - 1), prefix_size + (last_full - first_full + 1,) + dims[1:],
                        start + first_full * stride - lo_))
        if hi_ % stride:
            rec(0, hi_ % stride, dims[1:], prefix_off + (r1,), prefix_size + (1,), start + r1 * stride - lo_)

    if not shape:
        return [((), (), 0)] if hi > lo else []
    rec(lo, hi, shape, (), (), 0)
    return out


@dataclass(frozen=True)
class Box:
    name: str                      # tensor name on disk
    global_shape: tuple[int, ...]
    offsets: tuple[int, ...]       # of this box inside the global tensor
    sizes: tuple[int, ...]
    start: int                     # first element of the box inside the rank's flat slice of this parameter
    numel: int


def boxes_of_slice(name: str, lo: int, hi: int, local_shape, global_shape, cut_offsets) -> list[Box]:
    """The flat range [lo, hi) of a rank's local tensor (shape `local_shape`, placed at `cut_offsets` inside the global
    tensor) as boxes of the global tensor. Boxes that reach past the global extent in the outermost dimension are
    clipped (padding rows of a vocabulary cut); a box entirely in padding is dropped."""
    gs = tuple(int(x) for x in global_shape)
    out = []
    for off, size, start in flat_range_boxes(lo, hi, local_shape):
        goff = tuple(o + c for o, c in zip(off, cut_offsets))
        size = list(size)
        if goff and goff[0] + size[0] > gs[0]:
            size[0] = gs[0] - goff[0]
            if size[0] <= 0:
                continue
        if any(o + s > g for o, s, g in zip(goff, size, gs)):
            raise ConfigError(f"{name}: box at {goff} of size {tuple(size)} does not fit the global shape {gs}")
        out.append(Box(name, gs, goff, tuple(size), start, _prod(size)))
    return out


class BoxSavePlanner(DefaultSavePlanner):
    """State-dict keys `"<name>#box<i>"` hold box views; `table[key]` says where each belongs. Other entries (whole
    tensors, byte blobs) follow the default rules."""

    def __init__(self, table: dict[str, Box]):
        super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False, dedup_replicated_tensors=None)
        self.table = table
        self._by_index: dict[tuple[str, tuple[int, ...]], str] = {}

    def create_local_plan(self) -> SavePlan:
        items = []
        for key, obj in self.state_dict.items():
            box = self.table.get(key)
            if box is None:
                items += _create_write_items(key, obj)
                continue
            if tuple(obj.shape) != box.sizes:
                raise ConfigError(f"{key}: view of shape {tuple(obj.shape)} for a box of size {box.sizes}")
            self._by_index[(box.name, box.offsets)] = key
            items.append(WriteItem(index=MetadataIndex(box.name, torch.Size(box.offsets)), type=WriteItemType.SHARD,
                                   tensor_data=TensorWriteData(chunk=ChunkStorageMetadata(offsets=torch.Size(box.offsets), sizes=torch.Size(box.sizes)),
                                                               properties=TensorProperties.create_from_tensor(obj),
                                                               size=torch.Size(box.global_shape))))
        self.plan = SavePlan(items)
        return self.plan

    def lookup_object(self, index: MetadataIndex):
        key = self._by_index.get((index.fqn, tuple(index.offset))) if index.offset is not None else None
        if key is not None:
            return self.state_dict[key]
        return super().lookup_object(index)


class BoxLoadPlanner(DefaultLoadPlanner):
    """Destination views under `"<name>#box<i>"` keys are filled from whichever stored chunks of `<name>` intersect them.
    `missing` collects tensor names the checkpoint does not hold (the caller decides whether that is an error);
    a box that the stored chunks cover only in part is an error here."""

    def __init__(self, table: dict[str, Box], optional: set[str] | None = None):
        super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False, allow_partial_load=True)
        self.table = table
        self.optional = optional or set()
        self.missing: set[str] = set()
        self._by_index: dict[tuple[str, tuple[int, ...]], str] = {}

    def create_local_plan(self) -> LoadPlan:
        md_all = self.metadata.state_dict_metadata
        reqs = []
        for key, obj in self.state_dict.items():
            box = self.table.get(key)
            if box is None:
                md = md_all.get(key)
                if md is None:
                    self.missing.add(key)
                    continue
                reqs += _create_read_items(key, md, obj)
                continue
            md = md_all.get(box.name)
            if md is None:
                self.missing.add(box.name)
                continue
            if not isinstance(md, TensorStorageMetadata):
                raise ConfigError(f"checkpoint entry {box.name} is not a tensor")
            if tuple(md.size) != box.global_shape:
                raise ConfigError(f"checkpoint holds {box.name} with shape {tuple(md.size)}; this model expects {box.global_shape}")
            self._by_index[(box.name, box.offsets)] = key
            items = create_read_items_for_chunk_list(box.name, md, [ChunkStorageMetadata(torch.Size(box.offsets), torch.Size(box.sizes))])
            covered = sum(_prod(it.lengths) for it in items)
            if covered != box.numel:
                raise ConfigError(f"checkpoint covers {covered} of {box.numel} elements of {box.name} at {box.offsets}+{box.sizes}")
            reqs += items
        return LoadPlan(reqs)

    def lookup_tensor(self, index: MetadataIndex) -> torch.Tensor:
        key = self._by_index.get((index.fqn, tuple(index.offset))) if index.offset is not None else None
        if key is not None:
            return self.state_dict[key]
        return super().lookup_tensor(index)
