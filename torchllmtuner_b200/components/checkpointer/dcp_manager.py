"""Distributed checkpoint manager on torch DCP (reference: llmtuner/components/checkpointer/core/base.py:76-972,
backends/distributed_checkpoint.py:102-899, core/format_state.py, core/random_state.py, storage/checkpoint_writer.py).

State categories, in order: format, model, optimizer, lr_scheduler, [ema], train_state, dataloader, rng.

Tensor state lives in flat shards (see parallel/fsdp.py). On disk every parameter is ONE N-D tensor under its
wrapper-free name (`model.layers.0.self_attn.q_proj.weight`), its moments under `optimizer.state.<fqn>.exp_avg` /
`.exp_avg_sq` / `.momentum_buffer`, its average under `ema.ema_params.<fqn>`: the key layout of the reference. Each rank
contributes the rectangular boxes that make up the flat range it owns (components/checkpointer/boxes.py), placed inside
the global tensor by its tensor-, expert- or vocabulary-parallel cut, so the files are independent of every parallel
degree of the run that wrote them and a reader loads exactly the boxes it owns. Format 2 of this framework (1-D pieces
keyed `model.<fqn>@<lo>:<hi>`) is still read: `_load_pieces` is the migration path.

Publication is atomic: a save writes into `step-N.tmp-<id>/` and renames it to `step-N/` after DCP has written its
`.metadata`; `load` only considers folders that contain `.metadata`. A purge thread keeps the newest K resumable
checkpoints (exports are kept separately). Async modes stage the shards to (pinned) host memory and write from a
background thread over a gloo group.
"""
from __future__ import annotations

import dataclasses
import io
import os
import queue
import re
import threading
import time
import uuid

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from ...errors import ConfigError
from .manager import CheckpointManager
from .storage import is_remote, storage_for

FORMAT_VERSION = 3
READABLE_VERSIONS = (2, 3)
_CATEGORIES = ("optimizer", "ema", "obj")
_STEP_RE = re.compile(r"^step-(\d+)$")
_TMP_RE = re.compile(r"^step-(\d+)\.tmp-[0-9a-f]+$")
_PIECE_RE = re.compile(r"^(?P<base>.+?)(?:@tp(?P<dim>\d+)\.(?P<r>\d+)of(?P<n>\d+))?@(?P<lo>\d+):(?P<hi>\d+)$")


def _pack(obj) -> torch.Tensor:
    """Python state (dicts, lists, RNG tensors) travels as one opaque uint8 tensor so that DCP neither flattens nor
    re-keys it."""
    buf = io.BytesIO()
    torch.save(obj, buf)
    return torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).clone()


def _unpack(t: torch.Tensor):
    """Only plain containers, numbers, strings and tensors come back: a checkpoint cannot make the reader run code."""
    return torch.load(io.BytesIO(t.numpy().tobytes()), weights_only=True)


def validate_step_counter(value, *, key: str) -> int:
    """An optimizer step counter read from a checkpoint must be one finite, non-negative whole number (plain or a
    one-element tensor); anything else would silently corrupt bias correction
    (reference: llmtuner/components/optimizer/state_dict.py:237-265)."""
    if isinstance(value, torch.Tensor):
        if value.numel() != 1:
            raise ConfigError(f"{key}: step counter must hold exactly one value, got {value.numel()}")
        value = value.item()
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{key}: step counter must be a number, got {type(value).__name__}")
    if value != value or value in (float("inf"), float("-inf")) or value < 0 or float(value) != int(value):
        raise ConfigError(f"{key}: step counter must be a finite non-negative integer, got {value!r}")
    return int(value)


def canonical_fqn(fqn: str) -> str:
    """Names are those of the unwrapped model: parallelism wrappers (`.inner`) do not show in checkpoints."""
    return fqn.replace(".inner.", ".")


def _global_cut(p):
    """(tag, flat offset of the local parameter inside the full one, full numel). tag is '' when local flat ranges
    map to contiguous global flat ranges (uncut or cut on dim 0), else the local-coordinate tag."""
    shape = getattr(p, "_meta_shape", p.shape)
    numel = shape.numel()
    row = numel // shape[0] if len(shape) else 1
    off, full, tag = 0, numel, ""
    if getattr(p, "ep_sharded", False):
        off += p.ep_rank * shape[0] * row
        full = p.ep_full_experts * row
    d = getattr(p, "tp_shard_dim", None)
    if d is not None and hasattr(p, "tp_full_shape") and not getattr(p, "tp_vocab", False):
        fs = p.tp_full_shape
        n = fs[d] // shape[d] if shape[d] else 1
        r = getattr(p, "_tp_rank", None)
        if d == 0 and not getattr(p, "ep_sharded", False):
            if r is None:
                return None
            off += r * shape[0] * row
            full = fs[0] * row
        else:
            if r is None:
                return None
            tag = f"@tp{d}.{r}of{n}"
    elif getattr(p, "tp_vocab", False):
        r = getattr(p, "_tp_rank", 0)
        off += r * shape[0] * row
        full = max(p.tp_full_shape[0] * row, off + numel)
    return tag, off, full


def iter_pieces(rt):
    """Yield (fqn, tag, global_lo, global_hi, unit, shard_lo) for every parameter range this rank owns."""
    by_fqn = {}
    for u in rt.units:
        for p, s in zip(u.params, u.slots):
            by_fqn[s.fqn] = p
    for u in rt.units:
        for fqn, _shape, lo, hi, shard_lo in u.shard_slices():
            p = by_fqn[fqn]
            cut = _global_cut(p)
            if cut is None:
                raise ConfigError(f"{fqn}: tensor-parallel cut without a recorded rank")
            tag, off, _full = cut
            yield canonical_fqn(fqn), tag, off + lo, off + hi, u, shard_lo


def piece_params(rt) -> dict:
    """canonical fqn -> parameter object (for shapes and cut attributes) of everything this runtime owns."""
    out = {}
    for u in rt.units:
        for p_, s_ in zip(u.params, u.slots):
            out[canonical_fqn(s_.fqn)] = p_
    return out


def cut_geometry(p):
    """(local shape, global shape, offsets of the local tensor inside the global one) from the cut attributes that the
    tensor-, expert- and vocabulary-parallel stages leave on a parameter."""
    local = tuple(int(x) for x in getattr(p, "_meta_shape", p.shape))
    glob = list(local)
    off = [0] * len(local)
    d = getattr(p, "tp_shard_dim", None)
    if hasattr(p, "tp_full_shape") and (d is not None or getattr(p, "tp_vocab", False)):
        fs = tuple(int(x) for x in p.tp_full_shape)
        d = 0 if d is None else d
        r = getattr(p, "_tp_rank", None)
        if r is None:
            raise ConfigError("tensor-parallel cut without a recorded rank")
        glob[d] = fs[d]
        off[d] = r * local[d]
    if getattr(p, "ep_sharded", False):
        glob[0] = int(p.ep_full_experts)
        off[0] = int(p.ep_rank) * local[0]
    return local, tuple(glob), tuple(off)


def iter_boxes(rt):
    """Yield (fqn, Box list, unit, shard_lo) for every parameter range this rank owns; box names are the bare fqn."""
    from .boxes import boxes_of_slice
    params = piece_params(rt)
    for u in rt.units:
        for fqn, _shape, lo, hi, shard_lo in u.shard_slices():
            name = canonical_fqn(fqn)
            local, glob, off = cut_geometry(params[name])
            yield name, boxes_of_slice(name, lo, hi, local, glob, off), u, shard_lo


_TAG_RE = re.compile(r"^@tp(?P<dim>\d+)\.(?P<r>\d+)of(?P<n>\d+)$")


def _global_positions(tag: str, lo: int, hi: int, full_cols: int) -> torch.Tensor:
    """Flat positions inside the full 2-D tensor of the flat range [lo, hi) of a piece. Untagged pieces are already in
    full coordinates; a `@tp1.rofn` piece counts inside rank r's column block of width full_cols / n."""
    idx = torch.arange(lo, hi, dtype=torch.int64)
    if not tag:
        return idx
    m = _TAG_RE.match(tag)
    r, n = int(m["r"]), int(m["n"])
    c = full_cols // n
    return (idx // c) * full_cols + r * c + idx % c


def _intersections(need_lo: int, need_hi: int, have: list[tuple[int, int]]):
    for lo, hi in have:
        a, b = max(lo, need_lo), min(hi, need_hi)
        if b > a:
            yield lo, hi, a, b


class DistributedCheckpointManager(CheckpointManager):
    enabled = True

    def __init__(self, config, trainer):
        self.cfg = config.training.checkpoint_config
        self.config, self.trainer = config, trainer
        self.store = storage_for(self.cfg.folder if is_remote(self.cfg.folder) else config.training.dump_folder)
        self.root = self.store.join(config.training.dump_folder, self.cfg.folder)     # a URI in `folder` stands alone
        self.rank = trainer.env.rank
        self.world = trainer.env.world_size
        self._stamp_tp_ranks()
        self._async_future = None
        self._gloo = None
        self._purge_q: queue.Queue = queue.Queue()
        self._purge_thread = None
        if self.cfg.keep_latest_k > 0 and self.rank == 0:
            self._purge_thread = threading.Thread(target=self._purge_loop, daemon=True)
            self._purge_thread.start()
        if self.cfg.async_mode != "disabled" and dist.is_initialized():
            self._gloo = dist.new_group(backend="gloo")

    def _stamp_tp_ranks(self) -> None:
        topo = self.trainer.env.topo
        for p in self.trainer.model.parameters():
            if hasattr(p, "tp_shard_dim"):
                p._tp_rank = topo.coord("tp")

    # ------------------------------------------------------------------ state assembly
    def _tensor_state(self, model_only: bool = False):
        """({key: view or tensor}, {key: Box}): box views of this rank's shards plus whole buffers from their owner."""
        tr = self.trainer
        out: dict[str, torch.Tensor] = {}
        table: dict = {}

        def add(name, boxes, flat, slo):
            for b in boxes:
                key = f"{name}#box{len(table)}"
                table[key] = b if b.name == name else dataclasses.replace(b, name=name)
                out[key] = flat[slo + b.start: slo + b.start + b.numel].view(b.sizes)
        for rt, opt in zip([tr.asm.fsdp], tr.optimizers.optimizers):
            moments = getattr(opt, "state", {})
            for fqn, boxes, u, slo in iter_boxes(rt):
                if fqn.split(".")[0] in _CATEGORIES:
                    raise ConfigError(f"parameter {fqn} is named like a checkpoint state category")
                add(fqn, boxes, u.master, slo)
                if model_only:
                    continue
                st = moments.get(u.name)
                if st is not None:
                    for k in ("exp_avg", "exp_avg_sq", "momentum_buffer"):
                        if k in st:
                            add(f"optimizer.state.{fqn}.{k}", boxes, st[k], slo)
                if tr.ema is not None:
                    add(f"ema.ema_params.{fqn}", boxes, tr.ema.ema_params[u.name], slo)
        for name, buf in tr.model.named_buffers():
            if buf is not None and self._owns_replicated():
                out[canonical_fqn(name)] = buf.detach()
        if tr.ema is not None and not model_only and self._owns_replicated():
            for name, avg in tr.ema.ema_buffers.items():          # averaged buffers sit beside the averaged parameters
                out[f"ema.ema_params.{name}"] = avg
        return out, table

    def _full_shapes(self) -> dict[str, list[int]]:
        """canonical fqn -> shape of the whole (unsharded, all experts) parameter; what a converter needs to turn the
        flat pieces back into tensors."""
        out = {}
        for fqn, p in piece_params(self.trainer.asm.fsdp).items():
            shape = list(getattr(p, "_meta_shape", p.shape))
            if hasattr(p, "tp_full_shape") and not getattr(p, "ep_sharded", False):
                shape = list(p.tp_full_shape)
            if getattr(p, "ep_sharded", False):
                shape[0] = p.ep_full_experts
            out[fqn] = [int(x) for x in shape]
        return out

    def _owns_replicated(self) -> bool:
        t = self.trainer.env.topo
        return t.coord("dp") == 0 and t.coord("cp") == 0 and t.coord("tp") == 0

    def _object_state(self) -> dict:
        tr = self.trainer
        t = tr.env.topo
        obj = {}
        if self.rank == 0:
            obj["format"] = {"version": FORMAT_VERSION, "topology": t.snapshot(), "model": type(tr.model).__name__,
                             "arch": {k: v for k, v in vars(tr.model.config).items() if isinstance(v, (int, float, str, bool, list))},
                             "state_format": getattr(tr.model, "state_format", "native"), "shapes": self._full_shapes()}
            obj["optimizer.step"] = [getattr(o, "step_count", 0) for o in tr.optimizers.optimizers]
            obj["optimizer.param_groups"] = [[dict(g, param_names=[canonical_fqn(n) for n in g.get("param_names", [])])
                                              for g in o.param_groups] for o in tr.optimizers.optimizers]
            obj["lr_scheduler"] = tr.lr_schedulers.state_dict()
            obj["train_state"] = tr.progress.state_dict()
            if tr.ema is not None:
                obj["ema.num_updates"] = tr.ema.num_updates
        if t.coord("cp") == 0 and t.coord("tp") == 0:
            obj[f"dataloader.dp{t.coord('dp')}"] = tr.dataloader.state_dict()
        rng = {"cpu": torch.get_rng_state()}
        if torch.cuda.is_available() and tr.env.device.type == "cuda":
            rng["cuda"] = torch.cuda.get_rng_state(tr.env.device)
        obj[f"rng.rank{self.rank}"] = rng
        return {f"obj.{k}": _pack(v) for k, v in obj.items()}

    # ------------------------------------------------------------------ save
    def _should_save(self, step: int, last_step: bool) -> bool:
        if last_step:
            return True
        if step == 1 and self.cfg.enable_first_step_checkpoint:
            return True
        return step % self.cfg.interval == 0

    def _check_layout(self, what: str) -> None:
        """Optimizer and EMA state are keyed by parameter names: refuse to write or read them when the model's parameters
        are no longer the ones those consumers were built against."""
        tr = self.trainer
        rt = getattr(getattr(tr, "asm", None), "fsdp", None)
        if rt is not None and hasattr(rt, "sync_optimizer"):
            rt.sync_optimizer()                   # a parameter update may still be running on the optimizer's stream
        layout = getattr(getattr(tr, "asm", None), "layout", None)
        if layout is None:
            return
        layout.validate(tr.model)
        for consumer, obj in (("optimizer", getattr(tr, "optimizers", None)), ("ema", getattr(tr, "ema", None))):
            snap = getattr(obj, "layout_snapshot", None)
            if snap is not None:
                snap.validate(layout, consumer=f"checkpoint {what}: {consumer}")

    def save(self, step: int, last_step: bool = False, force: bool = False) -> None:
        if not (force or self._should_save(step, last_step)):
            return
        self.wait()
        self._check_layout("save")
        model_only = last_step and self.cfg.last_save_model_only and not force and step != 0
        if last_step and self.cfg.last_save_in_hf:
            from .hf import save_hf_checkpoint
            save_hf_checkpoint(self.trainer, self.store.join(self.root, "model-export"), self.cfg.export_dtype)
            return
        save_id = uuid.uuid4().hex[:8]
        if dist.is_initialized():
            ids = [save_id]
            dist.broadcast_object_list(ids, src=0)
            save_id = ids[0]
        final = self.store.join(self.root, f"step-{step}")
        tmp = f"{final}.tmp-{save_id}"
        from .boxes import BoxSavePlanner, dcp_errors
        state, table = self._tensor_state(model_only=model_only)
        state.update(self._object_state())
        if self.cfg.async_mode == "disabled":
            with dcp_errors(f"saving {tmp}"):
                dcp.save(state, storage_writer=self.store.writer(tmp), planner=BoxSavePlanner(table))
            self._publish(tmp, final, step)
        else:
            pin = self.cfg.async_mode == "async_with_pinned_mem" and torch.cuda.is_available()
            staged = {}
            for k, v in state.items():
                if isinstance(v, torch.Tensor):
                    c = torch.empty(v.shape, dtype=v.dtype, device="cpu", pin_memory=pin)
                    c.copy_(v, non_blocking=True)
                    staged[k] = c
                else:
                    staged[k] = v
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            fut = dcp.async_save(staged, storage_writer=self.store.writer(tmp), process_group=self._gloo, planner=BoxSavePlanner(table))
            self._async_future = (fut, tmp, final, step)

    def _publish(self, tmp: str, final: str, step: int) -> None:
        """Atomic publication by rank 0 inside an error-coordination boundary: if the rename fails, every rank raises
        and the previously published step stays the latest one."""
        from ...accelerator.collectives import synchronize_local_errors
        if dist.is_initialized():
            dist.barrier()
        with synchronize_local_errors("checkpoint-publish"):
            if self.rank == 0:
                if self.store.isdir(final):
                    self.store.rmtree(final)
                self.store.rename(tmp, final)
                self._purge_q.put(step)

    def latest_step(self) -> int:
        """Highest published step of this run folder, -1 when there is none."""
        steps = self._existing_steps()
        return max(steps) if steps else -1

    def maybe_wait_for_staging(self) -> None:
        """Called once per training step. Staging copies are synchronised inside `save()`; what is left is publication of
        a background write: as soon as EVERY rank's write has finished (MIN all-reduce of the done flags over the gloo
        group, so all ranks take the same branch) the folder is renamed to `step-N`. A crash in a later step then resumes
        from it instead of one interval earlier (reference: the DCP backend publishes when the background save completes,
        llmtuner/components/checkpointer/backends/distributed_checkpoint.py:328-457)."""
        if self._async_future is None:
            return
        fut = self._async_future[0]
        done = 1 if fut.done() else 0
        if dist.is_initialized() and self._gloo is not None:
            flag = torch.tensor([done], dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self._gloo)
            done = int(flag.item())
        if done:
            self.wait()

    def wait(self) -> None:
        if self._async_future is not None:
            from .boxes import dcp_errors
            fut, tmp, final, step = self._async_future
            self._async_future = None                         # a failed write is reported once, not at every later step
            with dcp_errors(f"saving {tmp}"):
                fut.result()
            self._publish(tmp, final, step)

    # ------------------------------------------------------------------ purge
    def _purge_loop(self) -> None:
        while True:
            item = self._purge_q.get()
            if item is None:
                return
            try:
                steps = sorted(self._existing_steps())
                exempt = self.cfg.purge_exempt or (lambda s: False)
                for s in steps[:-self.cfg.keep_latest_k]:
                    if not exempt(s):
                        self.store.rmtree(self.store.join(self.root, f"step-{s}"))
            except Exception:                # purging is best effort on every store; the next publication retries
                pass

    def _adopt_finished_writes(self) -> None:
        """A run that died after a background write finished but before its rename leaves `step-N.tmp-<id>` with a
        `.metadata` file (the coordinator writes it last, after every rank's shards). Such a folder is a complete
        checkpoint: rank 0 publishes it under its final name unless that step was published already."""
        st = self.store
        if self.rank != 0 or not st.isdir(self.root):
            return
        for name in sorted(st.listdir(self.root)):
            m = _TMP_RE.match(name)
            if not m:
                continue
            src, dst = st.join(self.root, name), st.join(self.root, f"step-{m.group(1)}")
            if st.exists(st.join(src, ".metadata")) and not st.isdir(dst):
                try:
                    st.rename(src, dst)
                except OSError:
                    pass

    def _existing_steps(self) -> list[int]:
        st = self.store
        if not st.isdir(self.root):
            return []
        out = []
        for name in st.listdir(self.root):
            m = _STEP_RE.match(name)
            if m and st.exists(st.join(self.root, name, ".metadata")):
                out.append(int(m.group(1)))
        return out

    # ------------------------------------------------------------------ load
    def _resolve_load_source(self, step: int):
        """An existing step folder of this run wins over `initial_load_path`."""
        self._adopt_finished_writes()
        if dist.is_initialized():
            dist.barrier()
        steps = self._existing_steps()
        if steps:
            s = max(steps) if step == -1 else step
            if s not in steps:
                raise ConfigError(f"checkpoint step {s} not found under {self.root} (have {sorted(steps)})")
            return self.store.join(self.root, f"step-{s}"), False, False
        if self.cfg.initial_load_path:
            return self.cfg.initial_load_path, self.cfg.initial_load_model_only, self.cfg.initial_load_in_hf
        return None, False, False

    def load(self, step: int = -1) -> bool:
        path, model_only, in_hf = self._resolve_load_source(step)
        if dist.is_initialized():
            agreed = [None] * self.world
            dist.all_gather_object(agreed, (path, model_only, in_hf))
            if any(a != agreed[0] for a in agreed):
                raise ConfigError(f"ranks disagree on the checkpoint to load: {agreed}")
        if path is None:
            return False
        if in_hf:
            from .hf import load_hf_checkpoint
            load_hf_checkpoint(self.trainer, path)
            return True
        self._load_dcp(path, model_only)
        return True

    def _load_dcp(self, path: str, model_only: bool) -> None:
        self._check_layout("load")
        reader = storage_for(path).reader(path)           # `initial_load_path` may live on another store than this run
        meta = reader.read_metadata()
        if any(_PIECE_RE.match(k) for k in meta.state_dict_metadata):
            self._load_pieces(path, model_only, reader, meta)       # written by format 2
        else:
            self._load_boxes(path, model_only, reader, meta)

    def _object_wants(self, meta, model_only: bool, exclude) -> dict:
        obj_keys = ["format"]
        if not model_only:
            t = self.trainer.env.topo
            obj_keys += ["optimizer.step", "lr_scheduler", "train_state", "ema.num_updates", f"dataloader.dp{t.coord('dp')}",
                         f"rng.rank{self.rank}"]
        want = {}
        for k in obj_keys:
            md = meta.state_dict_metadata.get(f"obj.{k}")
            if md is not None and k.split(".")[0] not in exclude:
                want[f"obj.{k}"] = torch.empty(md.size, dtype=torch.uint8)
        return want

    def _load_boxes(self, path: str, model_only: bool, reader, meta) -> None:
        from .boxes import BoxLoadPlanner, dcp_errors
        tr = self.trainer
        exclude = set(self.cfg.exclude_from_loading)
        want: dict[str, torch.Tensor] = {}
        table: dict = {}
        staged = []                  # (device view, host tensor): DCP reads into host memory, one copy to the device follows

        def add(name, boxes, flat, slo):
            for b in boxes:
                key = f"{name}#box{len(table)}"
                table[key] = dataclasses.replace(b, name=name)
                dst = flat[slo + b.start: slo + b.start + b.numel].view(b.sizes)
                if dst.device.type != "cpu":
                    host = torch.empty(b.sizes, dtype=dst.dtype)
                    staged.append((dst, host, key))
                    dst = host
                want[key] = dst
        required = set()
        for rt, opt in zip([tr.asm.fsdp], tr.optimizers.optimizers):
            for fqn, boxes, u, slo in iter_boxes(rt):
                if "model" not in exclude:
                    add(fqn, boxes, u.master, slo)
                    required.add(fqn)
                if model_only or "optimizer" in exclude:
                    continue
                st = getattr(opt, "state", {}).get(u.name, {})
                for k in ("exp_avg", "exp_avg_sq", "momentum_buffer"):
                    if k in st:
                        add(f"optimizer.state.{fqn}.{k}", boxes, st[k], slo)
                if tr.ema is not None and "ema" not in exclude:
                    add(f"ema.ema_params.{fqn}", boxes, tr.ema.ema_params[u.name], slo)
        buf_dst = {}
        for name, buf in tr.model.named_buffers():
            key = canonical_fqn(name)
            md = meta.state_dict_metadata.get(key)
            if md is not None and "model" not in exclude and tuple(md.size) == tuple(buf.shape):
                want[key] = torch.empty(buf.shape, dtype=buf.dtype)
                buf_dst[key] = buf
        ema_buf_dst = {}
        if tr.ema is not None and not model_only and "ema" not in exclude:
            for name, avg in tr.ema.ema_buffers.items():
                key = f"ema.ema_params.{name}"
                md = meta.state_dict_metadata.get(key)
                if md is not None and tuple(md.size) == tuple(avg.shape):
                    want[key] = torch.empty(avg.shape, dtype=avg.dtype)
                    ema_buf_dst[key] = avg
        obj_want = self._object_wants(meta, model_only, exclude)
        want.update(obj_want)
        planner = BoxLoadPlanner(table)
        with dcp_errors(f"loading {path}"):
            dcp.load(want, checkpoint_id=path, storage_reader=reader, planner=planner, no_dist=True)
        lacking = sorted(required & planner.missing)
        if lacking:
            raise ConfigError(f"checkpoint {path} lacks model tensors: {lacking[:5]}{'...' if len(lacking) > 5 else ''}")
        with torch.no_grad():
            for dst, host, key in staged:
                if table[key].name not in planner.missing:
                    dst.copy_(host)
            for key, buf in buf_dst.items():
                buf.copy_(want[key])
            for key, avg in ema_buf_dst.items():
                avg.copy_(want[key])
        self._after_tensor_load()
        self._restore_objects({k[4:]: _unpack(v) for k, v in obj_want.items()}, model_only)

    def _after_tensor_load(self) -> None:
        with torch.no_grad():
            for rt in [self.trainer.asm.fsdp]:
                for u in rt.units:
                    if u.separate_master:
                        u.shard_lowp.copy_(u.master)
                    if u.world > 1:
                        u.gathered = False
                        if getattr(u, "persistent", False):
                            rt.unshard(u)

    def _load_pieces(self, path: str, model_only: bool, reader, meta) -> None:
        """Format 2: 1-D pieces in global flat coordinates, `model.<fqn>@<lo>:<hi>`."""
        tr = self.trainer
        have: dict[tuple[str, str], list[tuple[int, int]]] = {}
        for key in meta.state_dict_metadata:
            m = _PIECE_RE.match(key)
            if m:
                tag = f"@tp{m['dim']}.{m['r']}of{m['n']}" if m["dim"] is not None else ""
                have.setdefault((m["base"], tag), []).append((int(m["lo"]), int(m["hi"])))
        exclude = set(self.cfg.exclude_from_loading)
        want: dict[str, torch.Tensor] = {}
        copies = []        # (dst view, key, src offset, n)

        def request(base, tag, glo, ghi, dst):
            pieces = have.get((base, tag))
            if pieces is None:
                return False
            covered = 0
            for lo, hi, a, b in _intersections(glo, ghi, pieces):
                key = f"{base}{tag}@{lo}:{hi}"
                if key not in want:
                    want[key] = torch.empty(hi - lo, dtype=torch.float32)
                copies.append((dst[a - glo:b - glo], key, a - lo, b - a))
                covered += b - a
            if covered != ghi - glo:
                raise ConfigError(f"checkpoint {path} covers {covered} of {ghi - glo} elements of {base}{tag}[{glo}:{ghi}]")
            return True

        have_by_base: dict[str, list[tuple[str, int, int]]] = {}
        for (base_, tag_), ranges in have.items():
            for lo_, hi_ in ranges:
                have_by_base.setdefault(base_, []).append((tag_, lo_, hi_))
        indexed = []       # (dst view, key, dst positions, src positions): pieces saved under another tensor-parallel cut

        def request_resharded(base, tag, glo, ghi, dst, p) -> bool:
            """The checkpoint holds this tensor under another cut of dimension 1 (row-parallel weights saved at a
            different tensor-parallel degree): match element by element through positions in the full tensor."""
            pieces = have_by_base.get(base)
            full_shape = tuple(getattr(p, "tp_full_shape", getattr(p, "_meta_shape", p.shape)))
            if not pieces or len(full_shape) != 2 or getattr(p, "ep_sharded", False):
                return False
            if any(t and (_TAG_RE.match(t) is None or int(_TAG_RE.match(t)["dim"]) != 1) for t, _, _ in pieces) or \
                    (tag and int(_TAG_RE.match(tag)["dim"]) != 1):
                return False
            C = full_shape[1]
            need = _global_positions(tag, glo, ghi, C)
            covered = 0
            for t, lo, hi in pieces:
                src = _global_positions(t, lo, hi, C)
                # both position lists are sorted: locate the needed positions inside this piece
                loc = torch.searchsorted(src, need)
                hit = (loc < src.numel()) & (src[loc.clamp_max(src.numel() - 1)] == need)
                if hit.any():
                    key = f"{base}{t}@{lo}:{hi}"
                    if key not in want:
                        want[key] = torch.empty(hi - lo, dtype=torch.float32)
                    indexed.append((dst, key, hit.nonzero().squeeze(1), loc[hit]))
                    covered += int(hit.sum())
            if covered != ghi - glo:
                raise ConfigError(f"checkpoint {path} covers {covered} of {ghi - glo} elements of {base}{tag}[{glo}:{ghi}]")
            return True

        missing = []
        for rt, opt in zip([tr.asm.fsdp], tr.optimizers.optimizers):
            params = piece_params(rt)
            for fqn, tag, glo, ghi, u, slo in iter_pieces(rt):
                n = ghi - glo

                def fetch(base, dst, _fqn=fqn, _tag=tag, _glo=glo, _ghi=ghi):
                    return request(base, _tag, _glo, _ghi, dst) or request_resharded(base, _tag, _glo, _ghi, dst, params[_fqn])
                if "model" not in exclude and not fetch(f"model.{fqn}", u.master[slo:slo + n]):
                    missing.append(fqn)
                if model_only or "optimizer" in exclude:
                    continue
                st = getattr(opt, "state", {}).get(u.name, {})
                for k in ("exp_avg", "exp_avg_sq", "momentum_buffer"):
                    if k in st:
                        fetch(f"optimizer.state.{fqn}.{k}", st[k][slo:slo + n])
                if tr.ema is not None and "ema" not in exclude:
                    fetch(f"ema.ema_params.{fqn}", tr.ema.ema_params[u.name][slo:slo + n])
        if missing:
            raise ConfigError(f"checkpoint {path} lacks model tensors: {missing[:5]}{'...' if len(missing) > 5 else ''}")
        buf_dst = {}
        for name, buf in tr.model.named_buffers():
            key = f"model.{canonical_fqn(name)}@0:{buf.numel()}"
            if key in meta.state_dict_metadata:
                want[key] = torch.empty(buf.numel(), dtype=buf.dtype)
                buf_dst[key] = buf
        obj_keys = ["format"]
        if not model_only:
            t = tr.env.topo
            obj_keys += ["optimizer.step", "lr_scheduler", "train_state", "ema.num_updates", f"dataloader.dp{t.coord('dp')}",
                         f"rng.rank{self.rank}"]
        objs = {}
        for k in obj_keys:
            md = meta.state_dict_metadata.get(f"obj.{k}")
            if md is not None and k.split(".")[0] not in exclude:
                want[f"obj.{k}"] = torch.empty(md.size, dtype=torch.uint8)
                objs[k] = None
        from .boxes import dcp_errors
        with dcp_errors(f"loading {path}"):
            dcp.load(want, checkpoint_id=path, storage_reader=reader, no_dist=True)
        for k in objs:
            objs[k] = _unpack(want.pop(f"obj.{k}"))
        want.update(objs)
        with torch.no_grad():
            for dst, key, off, n in copies:
                dst.copy_(want[key][off:off + n])
            for dst, key, dpos, spos in indexed:
                dst[dpos.to(dst.device)] = want[key][spos].to(dst.device, dst.dtype)
            for key, buf in buf_dst.items():
                buf.copy_(want[key].view_as(buf))
            for rt in [tr.asm.fsdp]:
                for u in rt.units:
                    if u.separate_master:
                        u.shard_lowp.copy_(u.master)
                    if u.world > 1:
                        u.gathered = False
                        if getattr(u, "persistent", False):
                            rt.unshard(u)
        self._restore_objects(want, model_only)

    def _restore_objects(self, want: dict, model_only: bool) -> None:
        tr = self.trainer
        fmt = want.get("format")
        if isinstance(fmt, dict) and fmt.get("version") not in READABLE_VERSIONS:
            raise ConfigError(f"checkpoint format version {fmt.get('version')} is not one of {READABLE_VERSIONS}")
        if model_only:
            return
        if "optimizer.step" in want:
            steps = want["optimizer.step"]
            if not isinstance(steps, (list, tuple)) or len(steps) != len(tr.optimizers.optimizers):
                raise ConfigError(f"checkpoint records {steps!r} optimizer step counters for {len(tr.optimizers.optimizers)} optimizers")
            for o, s in zip(tr.optimizers.optimizers, steps):
                o.step_count = validate_step_counter(s, key="optimizer.step")
        if isinstance(want.get("lr_scheduler"), dict):
            tr.lr_schedulers.load_state_dict(want["lr_scheduler"])
        if isinstance(want.get("train_state"), dict):
            tr.progress.load_state_dict(want["train_state"])
        if tr.ema is not None and isinstance(want.get("ema.num_updates"), int):
            tr.ema.num_updates = want["ema.num_updates"]
        dl = want.get(f"dataloader.dp{tr.env.topo.coord('dp')}")
        if isinstance(dl, dict):
            tr.dataloader.load_state_dict(dl)
            tr.data_iterator = iter(tr.dataloader)
        rng = want.get(f"rng.rank{self.rank}")
        if isinstance(rng, dict):
            torch.set_rng_state(rng["cpu"])
            if "cuda" in rng and tr.env.device.type == "cuda":
                torch.cuda.set_rng_state(rng["cuda"], tr.env.device)

    def close(self) -> None:
        self.wait()
        if self._purge_thread is not None:
            time.sleep(0.05)
            self._purge_q.put(None)
            self._purge_thread.join(timeout=10)
