"""Optimizers over the flat shards of `parallel.fsdp.FlatUnit`s
(reference: llmtuner/components/optimizer/optimizer.py:62-608, adamw_swap.py:71-650).

`ShardedAdamW` runs one fused kernel per unit on (fp32 master, fp32 moments, gradient shard) and rewrites the
low-precision shard that the next all-gather (or the peers' loads) reads. The clip coefficient stays on the device:
the kernel multiplies the gradient by it and skips the update when it is not finite, so no host round trip sits
between backward and the optimizer. Regex parameter groups (first match wins) are honoured per parameter by
cutting the unit into runs of equal hyper-parameters. `state_residency="host"` keeps the moments in pinned host
memory and streams them through the device in bounded slices (AdamWSwap).
"""
from __future__ import annotations

import re

import torch

from ... import ops


class StagedSlices:
    """Streams host-resident optimizer state through the device in bounded slices (reference:
    llmtuner/components/optimizer/adamw_swap.py:71-650). Two device slots rotate; three streams work at once:
        upload    slice i+1: pinned host -> slot (waits until the slot's previous download is done)
        compute   slice i:   the update kernel on the slot (waits for its upload)
        download  slice i-1: slot -> pinned host (waits for its compute)
    so that the PCIe copies in both directions hide behind the kernel, and the device never holds more than two slices
    of moments. Without a CUDA device the slices run one after the other on the host tensors themselves."""

    def __init__(self, device: torch.device, slice_elems: int, arrays: int = 2):
        self.device, self.slice = device, slice_elems
        self.cuda = device.type == "cuda"
        self.stats = {"slices": 0, "uploaded_bytes": 0, "downloaded_bytes": 0, "device_bytes": 0}
        if self.cuda:
            self.slots = [[torch.empty(slice_elems, dtype=torch.float32, device=device) for _ in range(arrays)] for _ in range(2)]
            self.up, self.down = torch.cuda.Stream(device), torch.cuda.Stream(device)
            self.uploaded = [torch.cuda.Event() for _ in range(2)]
            self.computed = [torch.cuda.Event() for _ in range(2)]
            self.drained = [torch.cuda.Event() for _ in range(2)]
            self.stats["device_bytes"] = 2 * arrays * slice_elems * 4
            self._n = 0

    def run(self, host_arrays: list[torch.Tensor], lo: int, hi: int, kernel) -> None:
        """`kernel(a, b, device_views)` updates elements [a, b) given views of the host arrays' slices on the device."""
        if not self.cuda:
            for a in range(lo, hi, self.slice):
                b = min(hi, a + self.slice)
                kernel(a, b, [h[a:b] for h in host_arrays])
                self.stats["slices"] += 1
            return
        main = torch.cuda.current_stream(self.device)
        for a in range(lo, hi, self.slice):
            b = min(hi, a + self.slice)
            s = self._n % 2
            self._n += 1
            views = [slot[:b - a] for slot in self.slots[s]]
            with torch.cuda.stream(self.up):
                self.up.wait_event(self.drained[s])              # the slot's last download (two slices ago) has left it
                for v, h in zip(views, host_arrays):
                    v.copy_(h[a:b], non_blocking=True)
                self.uploaded[s].record(self.up)
            main.wait_event(self.uploaded[s])
            kernel(a, b, views)
            self.computed[s].record(main)
            with torch.cuda.stream(self.down):
                self.down.wait_event(self.computed[s])
                for v, h in zip(views, host_arrays):
                    h[a:b].copy_(v, non_blocking=True)
                self.drained[s].record(self.down)
            self.stats["slices"] += 1
            self.stats["uploaded_bytes"] += (b - a) * 4 * len(host_arrays)
            self.stats["downloaded_bytes"] += (b - a) * 4 * len(host_arrays)

    def finish(self) -> None:
        """The host arrays are complete once the download stream is idle (called at the end of a step)."""
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.down)


class ShardedAdamW:
    def __init__(self, units, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 decoupled: bool = True, param_group_rules=None, host_moments: bool = False, swap_slice_bytes: int = 1 << 28):
        self.units = list(units)
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.decoupled = decoupled
        self.host_moments = host_moments
        self.swap_slice = max(1 << 20, swap_slice_bytes) // 4
        self.rules = [(re.compile(r.pattern), dict(r.optimizer_kwargs)) for r in (param_group_rules or [])]
        self.param_groups = [dict(self.defaults, name=".*", param_names=[])]
        for pat, kw in self.rules:
            g = dict(self.defaults, name=pat.pattern, param_names=[])
            g.update({("lr" if k == "learning_rate" else k): v for k, v in kw.items()})
            self.param_groups.append(g)
        self.step_count = 0
        self.state: dict[str, dict[str, torch.Tensor]] = {}
        self._runs: dict[str, list[tuple[int, int, int]]] = {}
        for u in self.units:
            dev = "cpu" if host_moments else u.master.device
            kw = dict(dtype=torch.float32, device=dev)
            m, v = torch.zeros(u.shard_numel, **kw), torch.zeros(u.shard_numel, **kw)
            if host_moments and torch.cuda.is_available():
                m, v = m.pin_memory(), v.pin_memory()
            self.state[u.name] = {"exp_avg": m, "exp_avg_sq": v}
            self._runs[u.name] = self._build_runs(u)
        self.stager = None
        if host_moments and self.units:
            biggest = max(u.shard_numel for u in self.units)
            self.stager = StagedSlices(self.units[0].master.device, min(self.swap_slice, biggest))

    def _group_index(self, fqn: str) -> int:
        for i, (pat, _) in enumerate(self.rules):
            if pat.search(fqn):
                return i + 1
        return 0

    def _build_runs(self, u):
        """[(shard_lo, shard_hi, group_index)] covering the shard, merged where neighbours share a group."""
        runs: list[list[int]] = []
        pos = 0
        for fqn, _shape, lo, hi, shard_lo in u.shard_slices():
            gi = self._group_index(fqn)
            self.param_groups[gi]["param_names"].append(fqn)
            if shard_lo > pos:
                runs.append([pos, shard_lo, runs[-1][2] if runs else gi])
            n = hi - lo
            if runs and runs[-1][2] == gi and runs[-1][1] == shard_lo:
                runs[-1][1] = shard_lo + n
            else:
                runs.append([shard_lo, shard_lo + n, gi])
            pos = shard_lo + n
        if pos < u.shard_numel:
            if runs:
                runs[-1][1] = u.shard_numel
            else:
                runs.append([0, u.shard_numel, 0])
        return [tuple(r) for r in runs]

    def zero_grad(self, set_to_none: bool = True) -> None:
        for u in self.units:
            u.has_grad = False

    def overlap_order(self):
        """Units in the order the next forward needs them: everything outside the blocks except the head first, the
        blocks in order, the head (needed after the last block) last."""
        first = [u for u in self.units if getattr(u, "block_index", None) is None and u.name != "head"]
        blocks = [u for u in self.units if getattr(u, "block_index", None) is not None]
        last = [u for u in self.units if getattr(u, "block_index", None) is None and u.name == "head"]
        return first + blocks + last

    @torch.no_grad()
    def step(self, clip_coef: torch.Tensor | None = None, overlap: bool = False) -> None:
        """`overlap=True` (single shard rank, device-resident moments, CUDA): the update kernels go to a second stream in
        the order the next forward needs the units and record one event per unit; the forward waits per unit
        (`FSDPRuntime.wait_param_update`), so the memory-bound update of later layers runs under the GEMMs of earlier
        ones. The arithmetic and its order per element are unchanged."""
        self.step_count += 1
        overlap = (overlap and not self.host_moments and all(u.world == 1 for u in self.units)
                   and self.units and self.units[0].master.is_cuda)
        if overlap:
            if getattr(self, "_side", None) is None:
                self._side = torch.cuda.Stream(self.units[0].master.device)
            self._side.wait_stream(torch.cuda.current_stream())          # gradients and the clip coefficient are ready
            with torch.cuda.stream(self._side):
                for u in self.overlap_order():
                    self._step_unit(u, clip_coef)
                    ev = torch.cuda.Event()
                    ev.record(self._side)
                    u.updated_event = ev
            return
        for u in self.units:
            self._step_unit(u, clip_coef)
        if self.stager is not None:
            self.stager.finish()

    def _step_unit(self, u, clip_coef) -> None:
        if not u.has_grad:
            return
        st = self.state[u.name]
        lowp = u.shard_lowp if u.separate_master else None
        for lo, hi, gi in self._runs[u.name]:
            g = self.param_groups[gi]
            kw = dict(lr=g["lr"], beta1=g["betas"][0], beta2=g["betas"][1], eps=g["eps"], weight_decay=g["weight_decay"],
                      step=self.step_count, decoupled=self.decoupled, clip_coef=clip_coef)
            if not self.host_moments:
                ops.adamw_step_(u.master[lo:hi], u.grad_shard[lo:hi], st["exp_avg"][lo:hi], st["exp_avg_sq"][lo:hi],
                                p_lowp=None if lowp is None else lowp[lo:hi], **kw)
            else:
                def update(a, b, mv, _u=u, _lowp=lowp, _kw=kw):
                    ops.adamw_step_(_u.master[a:b], _u.grad_shard[a:b], mv[0], mv[1], p_lowp=None if _lowp is None else _lowp[a:b], **_kw)
                self.stager.run([st["exp_avg"], st["exp_avg_sq"]], lo, hi, update)

    # ------------------------------------------------------------------ checkpoint state keyed by parameter FQN
    def state_dict_shards(self):
        """{unit_name: {"master", "exp_avg", "exp_avg_sq"}} flat shard tensors plus the step counter."""
        return {"step": self.step_count,
                "units": {u.name: {"master": u.master, **self.state[u.name]} for u in self.units}}

    def load_state_dict_shards(self, sd) -> None:
        self.step_count = int(sd["step"])
        for u in self.units:
            src = sd["units"][u.name]
            u.master.copy_(src["master"])
            if u.separate_master:
                u.shard_lowp.copy_(u.master)
            for k in ("exp_avg", "exp_avg_sq"):
                self.state[u.name][k].copy_(src[k])
