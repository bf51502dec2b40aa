"""Hugging Face safetensors import / export (reference: llmtuner/components/checkpointer/model_state.py:30-283,
hf/hf_storage.py:38-190, hf/hf_expert_storage.py:22-131).

Import: every rank opens the indexed safetensors files lazily and copies exactly the element ranges its flat shards
own (per-expert HF tensors are stitched into the packed native expert tensors on the fly).
Export: every rank writes the HF tensors (or contiguous parts of them) it owns into its own
`model-<rank>-of-<world>.safetensors`... which HF cannot read when a tensor is split, so instead the ranks hand their
ranges to rank 0 tensor by tensor (point-to-point gathers of one parameter at a time), and rank 0 writes complete
tensors into size-bounded shards, then publishes `model.safetensors.index.json` and `config.json` atomically by
renaming a `.export-<id>` staging folder."""
from __future__ import annotations

import json
import os
import shutil
import uuid

import torch
import torch.distributed as dist

from ...errors import ConfigError, UnsupportedCombinationError
from ...models.state import get_state_format
from .dcp_manager import _global_positions, iter_pieces

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def read_hf_weight_map(path: str) -> dict[str, str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return json.load(f)["weight_map"]
    single = os.path.join(path, "model.safetensors")
    if os.path.exists(single):
        from safetensors import safe_open
        with safe_open(single, "pt") as f:
            return {k: "model.safetensors" for k in f.keys()}
    raise ConfigError(f"{path} holds neither model.safetensors.index.json nor model.safetensors")


def resolve_hf_name(fmt, name: str, stored) -> str | None:
    """The key of `stored` (a weight map or any container of names) that holds the tensor `name`: itself, else the first
    of the state format's aliases that is there."""
    if name in stored:
        return name
    return next((a for a in fmt.hf_aliases(name) if a in stored), None)


def _param_index(trainer):
    if hasattr(trainer.asm.fsdp, "sync_optimizer"):
        trainer.asm.fsdp.sync_optimizer()
    out = {}
    tp_rank = trainer.env.topo.coord("tp")
    for p in trainer.model.parameters():
        if hasattr(p, "tp_shard_dim"):
            p._tp_rank = tp_rank                  # iter_pieces places a tensor-parallel cut through this
    for u in trainer.asm.fsdp.units:
        for p, s in zip(u.params, u.slots):
            out[s.fqn.replace(".inner.", ".")] = (p, s)
    return out


def _full_shape(p, s):
    shape = list(s.shape)
    if getattr(p, "ep_sharded", False):
        shape[0] = p.ep_full_experts
    if hasattr(p, "tp_full_shape") and not getattr(p, "ep_sharded", False):
        shape = list(p.tp_full_shape)
    return shape


def load_hf_checkpoint(trainer, path: str) -> None:
    from safetensors import safe_open
    fmt = get_state_format(getattr(trainer.model, "state_format", "qwen3"))
    wmap = read_hf_weight_map(path)
    handles: dict[str, object] = {}

    def tensor(name):
        stored = resolve_hf_name(fmt, name, wmap)
        if stored is None:
            raise ConfigError(f"HF checkpoint {path} lacks tensor {name}")
        fn, name = wmap[stored], stored
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), "pt")
        return handles[fn].get_tensor(name)

    pidx = _param_index(trainer)
    with torch.no_grad():
        for fqn, tag, glo, ghi, u, slo in iter_pieces(trainer.asm.fsdp):
            p, s = pidx[fqn]
            full_shape = _full_shape(p, s)
            variants = fmt.hf_piece_variants(fqn, full_shape)
            pieces = next((v for v in variants if all(resolve_hf_name(fmt, pc.name, wmap) is not None for pc in v)), variants[0])
            if tag:
                # a row-parallel weight (cut on dimension 1): this rank's flat range maps to scattered positions of the
                # full tensor, which is stored whole under one HF name
                if len(full_shape) != 2 or len(pieces) != 1:
                    raise ConfigError(f"HF import of {fqn}: only 2-D tensors may be cut along dimension 1")
                pos = _global_positions(tag, glo, ghi, full_shape[1])
                src = tensor(pieces[0].name).reshape(-1)
                u.master[slo: slo + (ghi - glo)].copy_(src[pos - pieces[0].native_lo + pieces[0].ref_lo].float())
                continue
            for piece in pieces:
                a, b = max(glo, piece.native_lo), min(ghi, piece.native_lo + piece.n)
                if b <= a:
                    continue
                off = piece.ref_lo - piece.native_lo
                src = tensor(piece.name).reshape(-1)[a + off:b + off]
                u.master[slo + (a - glo): slo + (b - glo)].copy_(src.float())
        for u in trainer.asm.fsdp.units:
            if u.separate_master:
                u.shard_lowp.copy_(u.master)
            if u.world > 1:
                u.gathered = False
                if getattr(u, "persistent", False):
                    trainer.asm.fsdp.unshard(u)


def save_hf_checkpoint(trainer, out_dir: str, export_dtype: str = "bfloat16", max_shard_bytes: int = 5 << 30) -> None:
    from safetensors.torch import save_file
    from .storage import is_remote
    if is_remote(out_dir):
        raise UnsupportedCombinationError(f"safetensors export writes local files; {out_dir} is a URI (export locally, then copy)")
    rank, world = trainer.env.rank, trainer.env.world_size
    fmt = get_state_format(getattr(trainer.model, "state_format", "qwen3"))
    dt = _DT[export_dtype]
    pidx = _param_index(trainer)
    mine: dict[str, list] = {}
    for fqn, tag, glo, ghi, u, slo in iter_pieces(trainer.asm.fsdp):
        mine.setdefault(fqn, []).append((glo, ghi, u.master[slo:slo + ghi - glo], tag))
    # which canonical FQNs exist anywhere, with their full shapes (identical on all ranks except expert slices)
    table = {fqn: _full_shape(*pidx[fqn]) for fqn in pidx}
    if world > 1:
        tables = [None] * world
        dist.all_gather_object(tables, table)
        for t in tables:
            table.update(t)
    stage = f"{out_dir}.export-{uuid.uuid4().hex[:8]}" if rank == 0 else None
    if rank == 0:
        os.makedirs(stage, exist_ok=True)
    shard, shard_bytes, shard_files, weight_map = {}, 0, [], {}
    partial: dict[str, tuple] = {}

    def flush():
        nonlocal shard, shard_bytes
        if shard:
            name = f"model-{len(shard_files) + 1:05d}.safetensors"
            save_file(shard, os.path.join(stage, name), metadata={"format": "pt"})
            shard_files.append((name, list(shard)))
            shard, shard_bytes = {}, 0

    for fqn in sorted(table):
        shape = table[fqn]
        numel = 1
        for x in shape:
            numel *= x
        parts = [(lo, hi, t.detach().to("cpu", torch.float32), tag) for lo, hi, t, tag in mine.get(fqn, [])]
        if world > 1:
            gathered = [None] * world if rank == 0 else None
            dist.gather_object(parts, gathered, dst=0)
            parts = [x for g in gathered for x in g] if rank == 0 else []
        if rank != 0:
            continue
        full = torch.zeros(numel, dtype=torch.float32)
        seen = 0
        for lo, hi, t, tag in parts:
            if tag:            # cut on dimension 1: scatter through positions in the full tensor
                full[_global_positions(tag, lo, hi, shape[1])] = t
                seen += hi - lo
                continue
            hi = min(hi, numel)
            if hi > lo:
                full[lo:hi] = t[:hi - lo]
                seen += hi - lo
        if seen < numel:
            raise ConfigError(f"export of {fqn}: gathered {seen} of {numel} elements")
        for piece in fmt.hf_pieces(fqn, shape):
            numel_hf = 1
            for x in piece.shape:
                numel_hf *= x
            if piece.n == numel_hf:
                t = full[piece.native_lo:piece.native_lo + piece.n].to(dt).view(*piece.shape).contiguous()
            else:                        # an HF tensor filled from several native tensors: hold it until it is complete
                buf, filled = partial.get(piece.name, (None, 0))
                if buf is None:
                    buf = torch.zeros(numel_hf, dtype=dt)
                buf[piece.ref_lo:piece.ref_lo + piece.n] = full[piece.native_lo:piece.native_lo + piece.n].to(dt)
                filled += piece.n
                if filled < numel_hf:
                    partial[piece.name] = (buf, filled)
                    continue
                partial.pop(piece.name, None)
                t = buf.view(*piece.shape)
            nbytes = t.numel() * t.element_size()
            if shard_bytes + nbytes > max_shard_bytes:
                flush()
            shard[piece.name] = t
            shard_bytes += nbytes
    if rank == 0:
        if partial:
            raise ConfigError(f"HF export: tensors left incomplete: {sorted(partial)[:5]}")
        flush()
        total = len(shard_files)
        for i, (name, keys) in enumerate(shard_files):
            final = f"model-{i + 1:05d}-of-{total:05d}.safetensors"
            os.replace(os.path.join(stage, name), os.path.join(stage, final))
            for k in keys:
                weight_map[k] = final
        with open(os.path.join(stage, "config.json"), "w") as f:
            json.dump(fmt.hf_config_of(trainer.model), f, indent=1)
        with open(os.path.join(stage, "model.safetensors.index.json.tmp"), "w") as f:
            json.dump({"metadata": {"format": "pt"}, "weight_map": weight_map}, f, indent=1)
        os.replace(os.path.join(stage, "model.safetensors.index.json.tmp"), os.path.join(stage, "model.safetensors.index.json"))
        if os.path.isdir(out_dir):
            shutil.rmtree(out_dir)
        os.replace(stage, out_dir)
    if world > 1:
        dist.barrier()
