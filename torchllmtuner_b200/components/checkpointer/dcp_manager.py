"""Distributed checkpoint manager on torch DCP (reference: llmtuner/components/checkpointer/core/base.py:76-972,
backends/distributed_checkpoint.py:102-899, core/format_state.py, core/random_state.py, storage/checkpoint_writer.py).

State categories, in order: format, model, optimizer, lr_scheduler, [ema], train_state, dataloader, rng.

Tensor state lives in flat shards (see parallel/fsdp.py). It is written as 1-D pieces whose keys carry *global*
coordinates of the full parameter, `model.<fqn>@<lo>:<hi>`, `optimizer.state.<fqn>.exp_avg@<lo>:<hi>`, so the layout on
disk is independent of the data-parallel, expert-parallel and (for dim-0 cuts: column-parallel linears, vocab
embedding, experts) tensor-parallel degree of the run that wrote it: a reader asks DCP's metadata which pieces exist and
loads the ones that intersect what it owns. Expert tensors therefore appear as pieces of the FULL `(E, ...)` tensors and a
run resumes at any EP degree. Parameters cut along a later dimension (row-parallel linears, TP-sharded experts) are
keyed in local coordinates with their cut, `...@tp<dim>.<rank>of<size>@<lo>:<hi>`, and resume at the same TP degree.

Publication is atomic: a save writes into `step-N.tmp-<id>/` and renames it to `step-N/` after DCP has written its
`.metadata`; `load` only considers folders that contain `.metadata`. A purge thread keeps the newest K resumable
checkpoints (exports are kept separately). Async modes stage the shards to (pinned) host memory and write from a
background thread over a gloo group.
"""
from __future__ import annotations

import io
import os
import queue
import re
import shutil
import threading
import time
import uuid

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from ...errors import ConfigError
from .manager import CheckpointManager

FORMAT_VERSION = 2
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
    return torch.load(io.BytesIO(t.numpy().tobytes()), weights_only=False)


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
        self.root = os.path.join(config.training.dump_folder, self.cfg.folder)
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
    def _tensor_state(self, model_only: bool = False) -> dict[str, torch.Tensor]:
        tr = self.trainer
        out: dict[str, torch.Tensor] = {}
        for rt, opt in zip([tr.asm.fsdp], tr.optimizers.optimizers):
            moments = getattr(opt, "state", {})
            for fqn, tag, glo, ghi, u, slo in iter_pieces(rt):
                n = ghi - glo
                suffix = f"{tag}@{glo}:{ghi}"
                out[f"model.{fqn}{suffix}"] = u.master[slo:slo + n]
                if model_only:
                    continue
                st = moments.get(u.name)
                if st is not None:
                    for k in ("exp_avg", "exp_avg_sq", "momentum_buffer"):
                        if k in st:
                            out[f"optimizer.state.{fqn}.{k}{suffix}"] = st[k][slo:slo + n]
                if tr.ema is not None:
                    out[f"ema.ema_params.{fqn}{suffix}"] = tr.ema.ema_params[u.name][slo:slo + n]
        for name, buf in tr.model.named_buffers():
            if buf is not None and self._owns_replicated():
                out[f"model.{canonical_fqn(name)}@0:{buf.numel()}"] = buf.detach().reshape(-1)
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
                             "arch": {k: v for k, v in vars(tr.model.config).items() if isinstance(v, (int, float, str, bool, list))}}
            obj["optimizer.step"] = [getattr(o, "step_count", 0) for o in tr.optimizers.optimizers]
            obj["optimizer.param_groups"] = [[{k: v for k, v in g.items() if k != "param_names"} for g in o.param_groups]
                                             for o in tr.optimizers.optimizers]
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

    def save(self, step: int, last_step: bool = False, force: bool = False) -> None:
        if not (force or self._should_save(step, last_step)):
            return
        self.wait()
        model_only = last_step and self.cfg.last_save_model_only and not force and step != 0
        if last_step and self.cfg.last_save_in_hf:
            from .hf import save_hf_checkpoint
            save_hf_checkpoint(self.trainer, os.path.join(self.root, "model-export"), self.cfg.export_dtype)
            return
        save_id = uuid.uuid4().hex[:8]
        if dist.is_initialized():
            ids = [save_id]
            dist.broadcast_object_list(ids, src=0)
            save_id = ids[0]
        final = os.path.join(self.root, "model-export" if model_only and False else f"step-{step}")
        tmp = f"{final}.tmp-{save_id}"
        state = self._tensor_state(model_only=model_only)
        state.update(self._object_state())
        if self.cfg.async_mode == "disabled":
            dcp.save(state, checkpoint_id=tmp)
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
            fut = dcp.async_save(staged, checkpoint_id=tmp, process_group=self._gloo)
            self._async_future = (fut, tmp, final, step)

    def _publish(self, tmp: str, final: str, step: int) -> None:
        """Atomic publication by rank 0 inside an error-coordination boundary: if the rename fails, every rank raises
        and the previously published step stays the latest one."""
        from ...accelerator.collectives import synchronize_local_errors
        if dist.is_initialized():
            dist.barrier()
        with synchronize_local_errors("checkpoint-publish"):
            if self.rank == 0:
                if os.path.isdir(final):
                    shutil.rmtree(final)
                os.replace(tmp, final)
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
            fut, tmp, final, step = self._async_future
            fut.result()
            self._async_future = None
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
                        shutil.rmtree(os.path.join(self.root, f"step-{s}"), ignore_errors=True)
            except OSError:
                pass

    def _adopt_finished_writes(self) -> None:
        """A run that died after a background write finished but before its rename leaves `step-N.tmp-<id>` with a
        `.metadata` file (the coordinator writes it last, after every rank's shards). Such a folder is a complete
        checkpoint: rank 0 publishes it under its final name unless that step was published already."""
        if self.rank != 0 or not os.path.isdir(self.root):
            return
        for name in sorted(os.listdir(self.root)):
            m = _TMP_RE.match(name)
            if not m:
                continue
            src, dst = os.path.join(self.root, name), os.path.join(self.root, f"step-{m.group(1)}")
            if os.path.exists(os.path.join(src, ".metadata")) and not os.path.isdir(dst):
                try:
                    os.replace(src, dst)
                except OSError:
                    pass

    def _existing_steps(self) -> list[int]:
        if not os.path.isdir(self.root):
            return []
        out = []
        for name in os.listdir(self.root):
            m = _STEP_RE.match(name)
            if m and os.path.exists(os.path.join(self.root, name, ".metadata")):
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
            return os.path.join(self.root, f"step-{s}"), False, False
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
        tr = self.trainer
        reader = dcp.FileSystemReader(path)
        meta = reader.read_metadata()
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
        fmt = want.get("format")
        if isinstance(fmt, dict) and fmt.get("version") != FORMAT_VERSION:
            raise ConfigError(f"checkpoint format version {fmt.get('version')} != {FORMAT_VERSION}")
        if model_only:
            return
        if "optimizer.step" in want:
            for o, s in zip(tr.optimizers.optimizers, want["optimizer.step"]):
                o.step_count = int(s)
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
