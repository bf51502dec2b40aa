"""Pipeline trainer: the production assembly (model, FSDP runtime, optimizer, data) cut into stages whose activations and
gradients travel over torch.distributed point-to-point sends (NCCL on CUDA), with the loss normalised by the global
valid-token count and gradients left unscaled (reference: experiments/pipeline_parallel/runtime.py:62-291,
microbatch_drivers.py:30-192, pipeline_parallel.py:84-131)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...components.loss import LossFunctions
from ...components.optimizer import GradientClipper, build_lr_scheduler, build_optimizers, check_finite
from ...config import resolve_batch_size_per_rank
from ...datasets import build_dataloader
from ...errors import ConfigError
from ...models.registry import build_registered_model
from ...parallel.fsdp import apply_fsdp
from ...trainer.runtime.environment import build_runtime_environment
from ...utils import get_logger
from .partition import partition_signature, prune_to_stage
from .schedules import build_schedule, stages_per_rank


class PipelineTrainer:
    def __init__(self, config, schedule: str = "1F1B", num_microbatches: int | None = None):
        self.config = config
        self.env = env = build_runtime_environment(config)
        topo = env.topo
        if topo.pp < 2:
            raise ConfigError("the pipeline experiment needs pipeline_parallel_size >= 2")
        if topo.tp > 1 or topo.cp > 1 or topo.ep > 1:
            raise ConfigError("the pipeline experiment composes with data parallelism only")
        self.logger = get_logger("pp")
        self.rank_pp, self.pp = topo.coord("pp"), topo.pp
        self.chunks = stages_per_rank(schedule)                  # looped stages held by one rank
        self.num_stages = self.pp * self.chunks
        self.pp_group = topo.get_group("pp")
        self.pp_ranks = topo.group_ranks("pp")
        # Activations and gradients travel in separate process groups: between two ranks the order of sends then only has
        # to match the order of receives per direction of the pipeline, which every schedule here guarantees.
        self.fwd_pg = self.bwd_pg = None
        for ranks in topo.all_groups("pp"):
            f, b = dist.new_group(ranks), dist.new_group(ranks)
            if env.rank in ranks:
                self.fwd_pg, self.bwd_pg = f, b
        t = config.training
        ac = t.activation_checkpoint_mode if t.activation_checkpoint_mode in ("none", "full") else "none"
        self.parts, self.rts = [], []
        for c in range(self.chunks):
            with torch.device("cpu"):
                model = build_registered_model(config.model, dtype=env.param_dtype)
            model.initialize_parameters(seed=t.seed)
            prune_to_stage(model, c * self.pp + self.rank_pp, self.num_stages)
            model.activation_checkpoint = ac
            rt = apply_fsdp(model, topo, config.parallel.fsdp_config, device=env.device, param_dtype=env.param_dtype, ac_mode=ac)
            for m in model.modules():
                for name, buf in list(m._buffers.items()):
                    if buf is not None:
                        m._buffers[name] = buf.to(env.device)
            self.parts.append(model)
            self.rts.append(rt)
        self.model, self.rt = self.parts[0], self.rts[0]
        sigs = [None] * self.pp
        mine = [p for c, m in enumerate(self.parts) for p in partition_signature(m, c * self.pp + self.rank_pp)["params"]]
        dist.all_gather_object(sigs, mine, group=self.pp_group)
        owned = [p for s in sigs for p in s if "layers" in p]
        if len(owned) != len(set(owned)):
            raise ConfigError("pipeline stages overlap")
        self.optimizers = build_optimizers(self.rts, config.optimizer)
        self.lr = build_lr_scheduler(self.optimizers, config.optimizer.lr_scheduler_config, t.steps)
        self.clipper = GradientClipper(self.rts, topo, t.max_norm, env.device)
        self.loss_fns = LossFunctions(num_chunks=t.chunked_loss_num_chunks)
        self.rows = resolve_batch_size_per_rank(t.global_batch_size, topo.dp, t.gradient_accumulation_steps)
        self.num_mb = num_microbatches or min(self.rows, self.pp)
        if self.rows % self.num_mb:
            raise ConfigError(f"rows per rank {self.rows} must be divisible by num_pp_microbatches {self.num_mb}")
        self.schedule = build_schedule(schedule, self.rank_pp, self.pp, self.num_mb)
        self.loader = build_dataloader(t.dataloader_config, vocab_size=self.model.config.vocab_size, global_batch=t.global_batch_size,
                                       seq_len=t.max_seq_len, seed=t.seed, dp_rank=topo.coord("dp"), dp_degree=topo.dp,
                                       rows_per_rank=self.rows)
        self.step = 0
        self.hidden = self.model.config.hidden_size

    # ------------------------------------------------------------------ p2p
    def _send(self, t: torch.Tensor, forward: bool) -> None:
        """Non-blocking: a stage sends an activation forward while its neighbour sends a gradient back, and two blocking
        sends would wait for each other. The handles are drained at the end of the step."""
        t = t.contiguous()
        peer = self.pp_ranks[(self.rank_pp + (1 if forward else -1)) % self.pp]
        self._pending.append((dist.isend(t, dst=peer, group=self.fwd_pg if forward else self.bwd_pg), t))

    def _recv(self, shape, dtype, forward: bool) -> torch.Tensor:
        """`forward`: an activation from the previous stage's rank; else a gradient from the next stage's rank."""
        buf = torch.empty(shape, dtype=dtype, device=self.env.device)
        peer = self.pp_ranks[(self.rank_pp + (-1 if forward else 1)) % self.pp]
        dist.recv(buf, src=peer, group=self.fwd_pg if forward else self.bwd_pg)
        return buf

    # ------------------------------------------------------------------ one optimizer step
    def train_step(self) -> float:
        dev = self.env.device
        for m in self.parts:
            m.train()
        batch = next(self.loader)
        B, S = batch["input"].shape
        mbs = B // self.num_mb
        gv = torch.tensor([float(batch["num_valid_tokens"])], dtype=torch.float32, device=dev)
        if self.env.topo.dp > 1:
            dist.all_reduce(gv, group=self.env.topo.get_group("dp"))
        saved: dict[tuple[int, int], tuple] = {}
        self._pending = []
        loss_total = torch.zeros((), dtype=torch.float32, device=dev)
        for rt in self.rts:
            rt.before_forward()
        last_b = {c: max(i for i, (k, cc, _) in enumerate(self.schedule) if k == "B" and cc == c) for c in range(self.chunks)}
        for idx, (kind, c, mb) in enumerate(self.schedule):
            m, rt = self.parts[c], self.rts[c]
            sl = slice(mb * mbs, (mb + 1) * mbs)
            if kind == "F":
                sub = {"input": batch["input"][sl], "labels": batch["labels"][sl], "num_valid_tokens": 0}
                inp = m.prepare_inputs(sub, dev, None)
                ctx = m.build_context(inp["positions"], inp["attn_meta"])
                if m.pp_first:
                    x_in = inp["tokens"]
                else:
                    x_in = self._recv((mbs * S, self.hidden), self.env.param_dtype, True).requires_grad_(True)
                if m.pp_last:
                    h = m(x_in, ctx, skip_lm_head=self.loss_fns.chunked)
                    loss_sum = self.loss_fns.from_hidden(h, m.lm_head.weight, inp["targets"]) if self.loss_fns.chunked \
                        else self.loss_fns.from_logits(h, inp["targets"])
                    out = loss_sum / gv.reshape(())
                    loss_total += loss_sum.detach()
                else:
                    out = m(x_in, ctx)
                    self._send(out.detach(), True)
                saved[(c, mb)] = (x_in, out)
            else:
                x_in, out = saved.pop((c, mb))
                rt.is_last_microbatch = idx == last_b[c]
                if m.pp_last:
                    out.backward()
                else:
                    g = self._recv(out.shape, out.dtype, False)
                    out.backward(g)
                if not m.pp_first:
                    self._send(x_in.grad, False)
        for work, _keepalive in self._pending:
            work.wait()
        self._pending = []
        for rt in self.rts:
            rt.finish_backward()
        for rt in self.rts:
            rt.wait_reductions()
        # the clip coefficient needs the norm over all stages
        self.clipper()
        total = (self.clipper.norm ** 2).clone()
        dist.all_reduce(total, group=self.pp_group)
        n = torch.sqrt(total)
        self.clipper.norm.copy_(n)
        self.clipper.coef.copy_(torch.clamp(self.config.training.max_norm / (n + 1e-6), max=1.0))
        self.optimizers.step(self.clipper.coef)
        for rt in self.rts:
            rt.post_optimizer()
        self.lr.step()
        self.step += 1
        # loss lives on the last stage; share it
        stats = torch.stack([loss_total, gv.reshape(())])
        if self.env.topo.dp > 1:
            red = stats[:1].clone()
            dist.all_reduce(red, group=self.env.topo.get_group("dp"))
            stats[0] = red[0]
        dist.broadcast(stats, src=self.pp_ranks[-1], group=self.pp_group)
        loss = float(stats[0] / stats[1].clamp_min(1))
        check_finite(self.clipper, loss)
        return loss

    def close(self) -> None:
        pass
