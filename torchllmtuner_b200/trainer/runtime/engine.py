"""Training engine: one forward/backward per micro-batch and the optimizer step
(reference: llmtuner/trainer/runtime/engine.py:52-494, gradients.py:50-372)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...components.loss import LossFunctions
from .gradients import check_step_condition
from ...models.execution import capabilities_of, validate_prepared_model_inputs, validate_training_output
from ...models.moe import collect_aux_loss, moe_blocks


class TrainingEngine:
    def __init__(self, model, assembly, loss_fns: LossFunctions, optimizers, lr_schedulers, ema, clipper, topo, device):
        self.model, self.asm, self.loss_fns = model, assembly, loss_fns
        self.optimizers, self.lr_schedulers, self.ema, self.clipper = optimizers, lr_schedulers, ema, clipper
        self.topo, self.device = topo, device
        self.rt = assembly.fsdp
        self.caps = capabilities_of(model)
        self.caps.require("hidden" if loss_fns.chunked else "logits")
        self.step_loss = torch.zeros((), dtype=torch.float32, device=device)

    # ------------------------------------------------------------------ step phases
    def begin_step(self) -> None:
        self.step_loss.zero_()
        self.model.train()

    def parallel_dims(self) -> dict | None:
        t = self.topo
        if t.cp == 1 and t.tp == 1:
            return None
        lb = getattr(self.asm.cp_driver, "load_balancer", None)
        return {"cp": t.cp, "cp_rank": t.coord("cp"), "tp": t.tp, "tp_rank": t.coord("tp"), "load_balancer": lb,
                "cp_kv": t.cp_kv, "cp_ulysses": t.cp_ulysses, "cp_kv_rank": t.coord("cp_kv"), "cp_ulysses_rank": t.coord("cp_ulysses")}

    def forward_backward(self, batch: dict, global_valid_tokens: torch.Tensor, is_last_microbatch: bool = True) -> torch.Tensor:
        """Returns the un-normalised loss sum of this micro-batch (device scalar, detached)."""
        m = self.model
        self.rt.is_last_microbatch = is_last_microbatch
        self.rt.aux_grad_scale = 1.0 / global_valid_tokens
        inputs = validate_prepared_model_inputs(m.prepare_inputs(batch, self.device, self.parallel_dims()))
        ctx = m.build_context(inputs["positions"], inputs["attn_meta"], self.asm.cp_driver)
        if self.asm.cp_driver is not None:
            self.asm.cp_driver.begin_microbatch(inputs)
        self.rt.before_forward()
        extra = inputs.get("model_kwargs") or {}          # what a wrapper model needs beside the tokens (image patches, grids)
        if self.loss_fns.chunked:
            h = m(inputs["tokens"], ctx, skip_lm_head=True, **extra)
            validate_training_output(h, inputs["targets"], output_width=self.caps.width("hidden"))
            loss_sum = self.loss_fns.from_hidden(h, m.lm_head.weight, inputs["targets"])
        else:
            logits = m(inputs["tokens"], ctx, **extra)
            validate_training_output(logits, inputs["targets"], output_width=self.caps.width("logits"))
            loss_sum = self.loss_fns.from_logits(logits, inputs["targets"])
        # Load-balance losses are token sums like the CE sum (`MoE.balance_loss_sum`): one division by the global valid-token
        # count normalises both. Blocks that replay their forward inside backward read the same factor from the runtime.
        aux = collect_aux_loss(m)
        loss = (loss_sum if aux is None else loss_sum + aux) / global_valid_tokens
        loss.backward()
        self.rt.finish_backward()
        self.step_loss += loss_sum.detach()
        return loss_sum.detach()

    @torch.no_grad()
    def evaluate(self, batch: dict) -> tuple[torch.Tensor, int]:
        m = self.model
        was = m.training
        m.eval()
        inputs = m.prepare_inputs(batch, self.device, self.parallel_dims())
        ctx = m.build_context(inputs["positions"], inputs["attn_meta"], self.asm.cp_driver)
        self.rt.before_forward()
        h = m(inputs["tokens"], ctx, skip_lm_head=True, **(inputs.get("model_kwargs") or {}))
        loss = self.loss_fns.from_hidden(h, m.lm_head.weight, inputs["targets"]) if self.loss_fns.chunked else \
            self.loss_fns.from_logits(m.lm_head(h), inputs["targets"])
        m.train(was)
        return loss, int((inputs["targets"] != -100).sum())

    def _update_moe_bias(self) -> None:
        blocks = moe_blocks(self.model)
        if not blocks:
            return
        group = self.topo.get_group("loss") if self.topo.ep > 1 else self.topo.get_group("dp_cp")
        counts = torch.stack([b.tokens_per_expert_E for b in blocks])
        if group is not None:
            dist.all_reduce(counts, group=group)
        for b, c in zip(blocks, counts):
            b.tokens_per_expert_E.copy_(c)
            b.update_expert_bias()

    def optimizer_step(self, step: int, overlap: bool = False) -> torch.Tensor:
        """`overlap=True`: the parameter update may still be running on the optimizer's stream when this returns; the next
        forward waits unit by unit, every other reader calls `rt.sync_optimizer()` first."""
        self.rt.wait_reductions()
        norm = self.clipper()
        self._update_moe_bias()
        self.optimizers.step(self.clipper.coef, overlap=overlap)
        self.rt.post_optimizer()
        self.lr_schedulers.step()
        if self.ema is not None:
            self.rt.sync_optimizer()
            self.ema.step(step)
        elif not overlap:
            self.rt.sync_optimizer()
        return norm

    def finish_step(self, step: int, loss_value: float | None = None) -> None:
        from ...parallel.graph_capture import check_sdc
        check_sdc(self.model)
        check_step_condition(self.clipper, loss_value)
