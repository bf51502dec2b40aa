"""Optimizer container, gradient clipping and EMA over sharded units
(reference: llmtuner/components/optimizer/optimizer.py:142-608, ema.py:43-410,
llmtuner/accelerator/collectives.py:290-558, llmtuner/trainer/runtime/gradients.py:321-372)."""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ... import ops
from ...errors import ConfigError
from .sharded import ShardedAdamW


class OptimizersContainer:
    """Fan-out over one optimizer per model part. Exposes `step`, `zero_grad`, and flat state for checkpoints."""

    def __init__(self, optimizers):
        self.optimizers = list(optimizers)

    def step(self, clip_coef=None, overlap: bool = False) -> None:
        """`overlap`: let optimizers that can (sharded AdamW on one shard rank) run their update under the next forward."""
        for o in self.optimizers:
            if overlap and isinstance(o, ShardedAdamW):
                o.step(clip_coef, overlap=True)
            else:
                o.step(clip_coef)

    def zero_grad(self) -> None:
        for o in self.optimizers:
            o.zero_grad()

    @property
    def param_groups(self):
        return [g for o in self.optimizers for g in o.param_groups]


def fused_qkv_row_blocks(model):
    """A fused QKV projection is three matrices stacked by rows (query, key, value heads in the ratio H : Hkv : Hkv,
    also after a tensor-parallel cut by heads): Muon orthogonalises them separately."""
    cfg = getattr(model, "config", None)
    if cfg is None or getattr(cfg, "qkv_projection", "separate") != "fused":
        return None
    H, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads

    def blocks(fqn: str, shape):
        if not fqn.endswith("qkv_proj.weight") or shape[0] % (H + 2 * Hkv):
            return None
        unit = shape[0] // (H + 2 * Hkv)
        return [H * unit, Hkv * unit, Hkv * unit]
    return blocks


def build_optimizers(runtimes, opt_cfg, host_state: bool = False) -> OptimizersContainer:
    """`host_state` (set by `fsdp_cpu_offload`) keeps the Adam moments in pinned host memory like AdamWSwap does: on a
    180 GB device the optimizer state is the part worth offloading; parameters and gradients stay resident."""
    outs = []
    for rt in runtimes:
        t = opt_cfg.optimizer_type
        if t in ("Adam", "AdamW", "AdamWSwap"):
            outs.append(ShardedAdamW(rt.units, lr=opt_cfg.learning_rate, betas=opt_cfg.betas, eps=opt_cfg.eps,
                                     weight_decay=opt_cfg.weight_decay, decoupled=t != "Adam",
                                     param_group_rules=opt_cfg.param_groups,
                                     host_moments=(t == "AdamWSwap" or opt_cfg.state_residency == "host" or host_state),
                                     swap_slice_bytes=opt_cfg.swap_max_device_bytes or (1 << 28)))
        elif t == "DistMuon":
            from .muon import DistMuon
            outs.append(DistMuon(rt, lr=opt_cfg.learning_rate, weight_decay=opt_cfg.weight_decay, betas=opt_cfg.betas,
                                 eps=opt_cfg.eps, param_group_rules=opt_cfg.param_groups, row_blocks=fused_qkv_row_blocks(rt.model)))
        else:
            raise ConfigError(f"unknown optimizer_type {t!r}")
    return OptimizersContainer(outs)


class GradientClipper:
    """L2 norm over every unit's gradient shard, combined across the groups that hold disjoint shards, then a clip
    coefficient that lives on the device. Dense shards are summed over `dp_shard_cp` (and `tp` for TP-sharded
    parameters), expert shards over `efsdp` x `ep`."""

    def __init__(self, runtimes, topo, max_norm: float, device):
        self.runtimes, self.topo, self.max_norm = list(runtimes), topo, max_norm
        self.device = torch.device(device)
        f = dict(dtype=torch.float32, device=self.device)
        self.total = torch.zeros(2, **f)       # [dense_sq, expert_sq]
        self.coef = torch.ones(1, **f)
        self.norm = torch.zeros(1, **f)
        self.finite = torch.ones(1, dtype=torch.int32, device=self.device)

    def _reduce(self, x: torch.Tensor, name: str) -> None:
        g = self.topo.get_group(name)
        if g is not None:
            dist.all_reduce(x, group=g)

    @torch.no_grad()
    def __call__(self) -> torch.Tensor:
        dense, expert, tp_rep, whole = [], [], [], []
        tp = self.topo.tp > 1
        for rt in self.runtimes:
            for u in rt.units:
                if not u.has_grad:
                    continue
                if getattr(u, "is_replicated", False):
                    whole.append(u.grad_shard)      # identical on every data rank: counted once, after the group sums
                    continue
                (expert if u.is_expert else dense).append(u.grad_shard)
                if tp:
                    # regions of parameters that every TP rank holds in full: counted once, not tp times
                    rep = {s.fqn for p, s in zip(u.params, u.slots) if getattr(p, "tp_replicated", False)}
                    for fqn, _shape, lo, hi, shard_lo in u.shard_slices():
                        if fqn in rep:
                            tp_rep.append(u.grad_shard[shard_lo:shard_lo + hi - lo])
        zero = lambda: torch.zeros(1, dtype=torch.float32, device=self.device)  # noqa: E731
        sq_d = ops.sq_norm(dense).reshape(1).to(self.device) if dense else zero()
        sq_e = ops.sq_norm(expert).reshape(1).to(self.device) if expert else zero()
        sq_r = ops.sq_norm(tp_rep).reshape(1).to(self.device) if tp_rep else zero()
        if tp:
            sq_d = sq_d - sq_r
            self._reduce(sq_d, "tp")
            if expert:
                self._reduce(sq_e, "tp")
            sq_d = sq_d + sq_r
        if self.topo.size("dp_shard_cp") > 1:
            self._reduce(sq_d, "dp_shard_cp")
        if self.topo.ep > 1:
            self._reduce(sq_e, "efsdp")
            self._reduce(sq_e, "ep")
        elif self.topo.size("dp_shard_cp") > 1:
            self._reduce(sq_e, "dp_shard_cp")
        total = (sq_d + sq_e).reshape(1)
        if whole:
            total = total + ops.sq_norm(whole).reshape(1).to(self.device)
        if self.device.type == "cuda":
            from ...ops.cuda_ext import load
            load().clip_coef(total, self.max_norm, self.coef, self.norm, self.finite)
        else:
            n = torch.sqrt(total)
            self.norm.copy_(n)
            self.coef.copy_(torch.clamp(self.max_norm / (n + 1e-6), max=1.0))
            self.finite.fill_(int(bool(torch.isfinite(n))))
        return self.norm


class EMA:
    """Exponential moving average of the fp32 master shards and, optionally, of selected module buffers
    (reference: llmtuner/components/optimizer/ema.py:43-410).

    The training engine calls `step(current_step)` after the optimizer. An update fires when
    `elapsed = current_step - start_step` is positive and a multiple of `update_every_n_steps`. The firing count
    `n = elapsed / update_every_n_steps + step_bias` is DERIVED from the step, never stored, so a resumed run continues
    with the right decay although only the averages are checkpointed. With `decay=None` the decay of firing n is
    2^(-1 / (half_life_fraction * n)): the half-life is a fixed fraction of the updates done so far.

    `buffer_patterns` (regular expressions searched in wrapper-free buffer names, all aliases considered) add buffers
    such as a MoE block's selection bias to the average; each buffer is tracked once, under its first name, BY IDENTITY:
    replacing a tracked buffer after construction is an error at the next step rather than a silently frozen average."""

    def __init__(self, runtimes, cfg, total_steps: int, model=None):
        import re
        self.cfg = cfg
        self.units = [u for rt in runtimes for u in rt.units]
        self.decay = cfg.decay
        self.ema_params = {u.name: u.master.detach().clone() for u in self.units}
        self.num_updates = 0
        self.buffers: dict[str, torch.Tensor] = {}          # first wrapper-free name -> the live buffer
        self.ema_buffers: dict[str, torch.Tensor] = {}
        self._model = model
        patterns = [re.compile(p) for p in (cfg.buffer_patterns or [])]
        if patterns and model is not None:
            first: dict[int, str] = {}
            for path, buf in model.named_buffers(remove_duplicate=False):
                name = path.replace(".inner.", ".")
                first.setdefault(id(buf), name)
                if any(p.search(name) for p in patterns) and first[id(buf)] not in self.buffers:
                    self.buffers[first[id(buf)]] = buf
            for name, buf in self.buffers.items():
                if not buf.dtype.is_floating_point:
                    raise ConfigError(f"EMA buffer {name} has dtype {buf.dtype}; only floating-point buffers can be averaged")
                self.ema_buffers[name] = buf.detach().clone().float()
        if patterns and not self.buffers:
            import logging
            logging.getLogger("torchllmtuner_b200").warning("EMA buffer_patterns %s matched no buffer: nothing but parameters is "
                                                            "averaged; check the patterns", list(cfg.buffer_patterns))

    def firing(self, step: int) -> int:
        """0 when `step` does not fire, else the firing count n (with `step_bias` added)."""
        if isinstance(step, bool) or not isinstance(step, int) or step < 0:
            raise ValueError("EMA current_step must be a non-negative integer")
        c = self.cfg
        elapsed = step - c.start_step
        if elapsed <= 0 or elapsed % c.update_every_n_steps:
            return 0
        return elapsed // c.update_every_n_steps + c.step_bias

    def decay_at(self, n: int) -> float:
        return self.decay if self.decay is not None else 2.0 ** (-1.0 / (self.cfg.half_life_fraction * n))

    @torch.no_grad()
    def step(self, step: int) -> None:
        n = self.firing(step)
        if n <= 0:
            return
        self.num_updates = n
        d = self.decay_at(n)
        avgs = [self.ema_params[u.name] for u in self.units]
        torch._foreach_lerp_(avgs, [u.master for u in self.units], 1.0 - d)
        if self.buffers:
            live = {id(b) for b in self._model.buffers()} if self._model is not None else None
            for name, buf in self.buffers.items():
                if live is not None and id(buf) not in live:
                    raise RuntimeError(f"EMA tracks the buffer {name} by identity and it is no longer registered in the model: "
                                       "build the EMA after the model is final")
                self.ema_buffers[name].lerp_(buf.detach().float(), 1.0 - d)

    def reset(self) -> None:
        for u in self.units:
            self.ema_params[u.name].copy_(u.master)
        for name, buf in self.buffers.items():
            self.ema_buffers[name].copy_(buf.detach().float())
        self.num_updates = 0

    def state_dict(self):
        return {"ema_params": self.ema_params, "ema_buffers": self.ema_buffers, "num_updates": self.num_updates}

    def load_state_dict(self, sd):
        for k, v in sd["ema_params"].items():
            self.ema_params[k].copy_(v)
        for k, v in (sd.get("ema_buffers") or {}).items():
            if k not in self.ema_buffers:
                raise ConfigError(f"EMA state names the buffer {k}, which this run does not track")
            self.ema_buffers[k].copy_(v)
        self.num_updates = int(sd.get("num_updates", 0))


def check_finite(clipper: GradientClipper, loss_value: float | None = None) -> None:
    """Host-side verdict, read once at the end of the step: the kernels already skipped the update when the
    coefficient was not finite, so raising here is equivalent to raising before the update."""
    from ...errors import LLMTunerError
    if int(clipper.finite.item()) == 0 or (loss_value is not None and not math.isfinite(loss_value)):
        raise LLMTunerError(f"non-finite gradient norm or loss (norm={float(clipper.norm.item())}, loss={loss_value}); "
                            "the optimizer update was skipped on every rank")
