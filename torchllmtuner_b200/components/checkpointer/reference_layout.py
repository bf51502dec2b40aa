"""Checkpoints in the reference's distributed-checkpoint key layout, read and written
(reference: llmtuner/components/checkpointer/backends/distributed_checkpoint.py:835-856 merges the model's entries, keyed
by bare parameter names, with the other state categories; llmtuner/components/optimizer/state_dict.py:168-190 flattens
the optimizer to `state.<fqn>.<name>` and `param_groups.<fqn>.<option>` under `optimizer`).

A checkpoint of this framework already uses that key layout, with this framework's parameter names and packing
(`...mlp.routed.experts.w1_EFD`); the converters here translate names and packing to and from those of the reference's
module classes (`...mlp.experts.gate_up_proj`). They work on folders, in one process on the host, one tensor at a time:

  export_reference_layout(step_dir, out_dir)    native names -> the reference's names
        <name>                                   model weights (names and packing of the reference's module classes)
        optimizer.state.<name>.exp_avg|exp_avg_sq|momentum_buffer|step
        optimizer.param_groups.<name>.<option>   lr, betas, eps, weight_decay, ... of the group that owns <name>
        lr_scheduler.last_epoch, train_state.<field>
  import_reference_layout(ref_dir, step_dir, shapes, state_format)
        the inverse: writes every native tensor whole, which this framework's loader then cuts for whatever data-,
        expert- or tensor-parallel degree resumes from it.

Two native tensors may share one reference tensor (gate and up rows of the packed experts); a reference tensor is
therefore assembled from every native piece that maps into it before it is written.
"""
from __future__ import annotations

import os

import torch
import torch.distributed.checkpoint as dcp

from ...errors import ConfigError
from ...models.state import get_state_format
from .boxes import dcp_errors
from .dcp_manager import _PIECE_RE, _global_positions, _pack, _unpack, FORMAT_VERSION

_MOMENTS = ("exp_avg", "exp_avg_sq", "momentum_buffer")


def _numel(shape) -> int:
    n = 1
    for x in shape:
        n *= int(x)
    return n


class _PieceReader:
    """Assembles whole flat tensors from the pieces of a native checkpoint folder."""

    def __init__(self, path: str):
        self.path = path
        self.reader = dcp.FileSystemReader(path)
        self.meta = self.reader.read_metadata().state_dict_metadata
        self.pieces: dict[str, list[tuple[str, str, int, int]]] = {}
        for key in self.meta:
            m = _PIECE_RE.match(key)
            if m:
                tag = f"@tp{m['dim']}.{m['r']}of{m['n']}" if m["dim"] is not None else ""
                self.pieces.setdefault(m["base"], []).append((key, tag, int(m["lo"]), int(m["hi"])))

    def obj(self, name: str):
        md = self.meta.get(f"obj.{name}")
        if md is None:
            return None
        want = {f"obj.{name}": torch.empty(md.size, dtype=torch.uint8)}
        dcp.load(want, checkpoint_id=self.path, storage_reader=self.reader, no_dist=True)
        return _unpack(want[f"obj.{name}"])

    def full(self, base: str, shape) -> torch.Tensor | None:
        parts = self.pieces.get(base)
        if not parts:
            # format 3 stores whole tensors under bare names (`model.` prefix only existed for pieces)
            key = base[len("model."):] if base.startswith("model.") and base not in self.meta else base
            md = self.meta.get(key)
            if md is None or not hasattr(md, "size"):
                return None
            if tuple(md.size) != tuple(int(x) for x in shape):
                raise ConfigError(f"{self.path}: {key} has shape {tuple(md.size)}, the format record says {tuple(shape)}")
            want = {key: torch.empty(tuple(md.size), dtype=torch.float32)}
            dcp.load(want, checkpoint_id=self.path, storage_reader=self.reader, no_dist=True)
            return want[key].reshape(-1)
        numel = _numel(shape)
        want = {key: torch.empty(hi - lo, dtype=torch.float32) for key, _, lo, hi in parts}
        dcp.load(want, checkpoint_id=self.path, storage_reader=self.reader, no_dist=True)
        out = torch.zeros(numel, dtype=torch.float32)
        seen = 0
        for key, tag, lo, hi in parts:
            if tag:
                if len(shape) != 2:
                    raise ConfigError(f"{base}: piece {key} is cut along a later dimension of a tensor that is not 2-D")
                out[_global_positions(tag, lo, hi, int(shape[1]))] = want[key]
                seen += hi - lo
            else:
                hi = min(hi, numel)                 # a padded vocabulary slice may reach past the real rows
                if hi > lo:
                    out[lo:hi] = want[key][:hi - lo]
                    seen += hi - lo
        if seen < numel:
            raise ConfigError(f"{self.path}: pieces of {base} cover {seen} of {numel} elements")
        return out


@dcp_errors("exporting a checkpoint to the reference layout")
def export_reference_layout(step_dir: str, out_dir: str, state_format: str | None = None) -> dict:
    """Returns {"tensors": count, "keys": sorted list of the keys written}."""
    src = _PieceReader(step_dir)
    fmt_obj = src.obj("format")
    if not isinstance(fmt_obj, dict) or "shapes" not in fmt_obj:
        raise ConfigError(f"{step_dir} does not record parameter shapes (written by an older version); re-save it first")
    fmt = get_state_format(state_format or fmt_obj.get("state_format", "native"))
    shapes = fmt_obj["shapes"]
    steps = src.obj("optimizer.step") or [0]
    groups = src.obj("optimizer.param_groups") or []
    option_of: dict[str, dict] = {}
    step_of: dict[str, int] = {}
    for oi, opt_groups in enumerate(groups):
        for g in opt_groups:
            opts = {k: v for k, v in g.items() if k not in ("param_names", "params", "name")}
            for n in g.get("param_names", []):
                option_of[n] = opts
                step_of[n] = int(steps[min(oi, len(steps) - 1)])

    def assemble(prefix: str, suffix: str = "") -> dict[str, torch.Tensor]:
        out: dict[str, torch.Tensor] = {}
        for fqn, shape in shapes.items():
            flat = src.full(f"{prefix}{fqn}{suffix}", shape)
            if flat is None:
                continue
            for pc in fmt.to_reference(fqn, shape):
                dst = out.get(pc.name)
                if dst is None:
                    dst = out[pc.name] = torch.zeros(_numel(pc.shape), dtype=torch.float32)
                dst[pc.ref_lo:pc.ref_lo + pc.n] = flat[pc.native_lo:pc.native_lo + pc.n]
        return out

    state: dict = {}
    ref_shape: dict[str, tuple] = {}
    owner: dict[str, str] = {}
    for fqn, shape in shapes.items():
        for pc in fmt.to_reference(fqn, shape):
            ref_shape[pc.name] = tuple(pc.shape)
            owner.setdefault(pc.name, fqn)
    for name, t in assemble("model.").items():
        state[name] = t.view(ref_shape[name])
    opt_state: dict = {}
    for k in _MOMENTS:
        for name, t in assemble("optimizer.state.", f".{k}").items():
            opt_state.setdefault(name, {})[k] = t.view(ref_shape[name])
    for name, st in opt_state.items():
        st["step"] = torch.tensor(float(step_of.get(owner[name], steps[0])), dtype=torch.float32)
    param_groups = {name: dict(option_of[owner[name]]) for name in ref_shape if owner[name] in option_of}
    if opt_state or param_groups:
        state["optimizer"] = {"state": opt_state, "param_groups": param_groups}
    sched = src.obj("lr_scheduler")
    if isinstance(sched, dict):
        state["lr_scheduler"] = sched
    prog = src.obj("train_state")
    if isinstance(prog, dict):
        state["train_state"] = prog
    collisions = [k for k in ("optimizer", "lr_scheduler", "train_state") if k in ref_shape]
    if collisions:
        raise ConfigError(f"model tensors named like state categories: {collisions}")
    os.makedirs(out_dir, exist_ok=True)
    dcp.save(state, checkpoint_id=out_dir, no_dist=True)
    keys = sorted(dcp.FileSystemReader(out_dir).read_metadata().state_dict_metadata)
    return {"tensors": len(ref_shape), "keys": keys}


@dcp_errors("importing a reference-layout checkpoint")
def import_reference_layout(ref_dir: str, step_dir: str, shapes: dict[str, list[int]], state_format: str = "native",
                            model_only: bool = False) -> dict:
    """`shapes`: canonical native fqn -> whole shape of the model that will load the result (`native_shapes(model)` gives
    it from a model built on any device, the meta device included)."""
    fmt = get_state_format(state_format)
    reader = dcp.FileSystemReader(ref_dir)
    meta = reader.read_metadata().state_dict_metadata
    cache: dict[str, torch.Tensor] = {}

    def ref_tensor(key: str, shape) -> torch.Tensor | None:
        md = meta.get(key)
        if md is None:
            return None
        if key not in cache:
            if tuple(md.size) != tuple(shape):
                raise ConfigError(f"{ref_dir}: {key} has shape {tuple(md.size)}, the model expects {tuple(shape)}")
            want = {key: torch.empty(tuple(md.size), dtype=md.properties.dtype)}
            dcp.load(want, checkpoint_id=ref_dir, storage_reader=reader, no_dist=True)
            if len(cache) > 8:
                cache.clear()
            cache[key] = want[key].reshape(-1).float()
        return cache[key]

    out: dict[str, torch.Tensor] = {}
    missing = []
    step = None
    for fqn, shape in shapes.items():
        numel = _numel(shape)
        pcs = fmt.to_reference(fqn, shape)
        flat = torch.empty(numel, dtype=torch.float32)
        ok = True
        for pc in pcs:
            t = ref_tensor(pc.name, pc.shape)
            if t is None:
                ok = False
                break
            flat[pc.native_lo:pc.native_lo + pc.n] = t[pc.ref_lo:pc.ref_lo + pc.n]
        if not ok:
            missing.append(fqn)
            continue
        out[fqn] = flat.view(tuple(int(x) for x in shape))
        if model_only:
            continue
        for k in _MOMENTS:
            flat = torch.empty(numel, dtype=torch.float32)
            ok = True
            for pc in pcs:
                t = ref_tensor(f"optimizer.state.{pc.name}.{k}", pc.shape)
                if t is None:
                    ok = False
                    break
                flat[pc.native_lo:pc.native_lo + pc.n] = t[pc.ref_lo:pc.ref_lo + pc.n]
            if ok:
                out[f"optimizer.state.{fqn}.{k}"] = flat.view(tuple(int(x) for x in shape))
        if step is None:
            sk = f"optimizer.state.{pcs[0].name}.step"
            if sk in meta:
                want = {sk: torch.empty((), dtype=torch.float32)}
                dcp.load(want, checkpoint_id=ref_dir, storage_reader=reader, no_dist=True)
                step = int(want[sk].item())
    if missing:
        raise ConfigError(f"{ref_dir} lacks tensors for {missing[:5]}{'...' if len(missing) > 5 else ''}")
    objs = {"format": {"version": FORMAT_VERSION, "state_format": state_format, "shapes": {k: list(v) for k, v in shapes.items()},
                       "imported_from": "reference layout"}}
    if not model_only and step is not None:
        objs["optimizer.step"] = [step]
        objs["lr_scheduler"] = {"last_epoch": step}
        prog = _load_plain(ref_dir, reader, meta, "train_state.")
        prog.setdefault("step", step)
        objs["train_state"] = prog
    out.update({f"obj.{k}": _pack(v) for k, v in objs.items()})
    os.makedirs(step_dir, exist_ok=True)
    dcp.save(out, checkpoint_id=step_dir, no_dist=True)
    return {"tensors": len(shapes), "step": step}


def _load_plain(path, reader, meta, prefix: str) -> dict:
    """Non-tensor leaves under `prefix` (DCP stores them as pickled bytes) and scalar tensors, one level deep."""
    from torch.distributed.checkpoint.metadata import BytesStorageMetadata
    want = {}
    for key, md in meta.items():
        if key.startswith(prefix) and "." not in key[len(prefix):]:
            want[key] = None if isinstance(md, BytesStorageMetadata) else torch.empty(tuple(md.size), dtype=md.properties.dtype)
    if not want:
        return {}
    dcp.load(want, checkpoint_id=path, storage_reader=reader, no_dist=True)
    return {k[len(prefix):]: (v.item() if isinstance(v, torch.Tensor) and v.numel() == 1 else v) for k, v in want.items()}


def native_shapes(model) -> dict[str, list[int]]:
    from .dcp_manager import canonical_fqn
    return {canonical_fqn(n): [int(x) for x in getattr(p, "_meta_shape", p.shape)] for n, p in model.named_parameters()}
