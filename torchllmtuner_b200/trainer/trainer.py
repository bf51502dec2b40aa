"""`Trainer(config).train() / train_step() / validate() / close()` (reference: llmtuner/trainer/trainer.py:81-796)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..accelerator.collectives import set_pg_timeouts
from ..components.metrics import MetricsProcessor
from ..config import LLMTunerConfig, resolve_batch_size_per_rank
from ..datasets import build_dataloader
from ..datasets.contracts import DataloaderExhaustedError
from ..errors import KernelStatusError
from ..ops.cuda_ext import check_status, status_word
from ..utils import GarbageCollection, get_logger, set_log_ranks
from ..utils.metric_loggers import build_metric_logger
from ..utils.nvtx import nvtx_range
from .runtime.batch import fetch_batch, global_valid_tokens
from .runtime.metrics import build_step_metrics
from .runtime.reductions import TrainingReductionMeshes
from .runtime.assembly import (build_loss_functions, build_optimizer_stack, create_training_engine, prepare_parallel_model)
from .runtime.environment import build_runtime_environment
from .runtime.observer import TrainingObserver
from .runtime.results import StepResult, TrainingProgress


class Trainer:
    def __init__(self, config: LLMTunerConfig):
        self.config = config
        self.closed = False
        self._assemble_runtime(config)

    # ------------------------------------------------------------------ assembly
    def _assemble_runtime(self, cfg: LLMTunerConfig) -> None:
        t = cfg.training
        set_log_ranks(t.metrics_config.log_ranks)
        self.logger = get_logger("trainer")
        from ..config.inert_fields import check_unsupported_fields, inert_fields_set
        check_unsupported_fields(cfg)
        for name, why in inert_fields_set(cfg):
            self.logger.warning(f"--{name} is accepted for command-line compatibility and has no effect here: {why}")
        self.env = env = build_runtime_environment(cfg)
        topo = env.topo
        self.model, self.asm = prepare_parallel_model(cfg, env)
        self.loss_fns = build_loss_functions(cfg, env, self.asm)
        self.optimizers, self.lr_schedulers, self.ema, self.clipper = build_optimizer_stack(cfg, env, self.asm)
        self.engine = create_training_engine(cfg, env, self.model, self.asm, self.loss_fns, self.optimizers,
                                             self.lr_schedulers, self.ema, self.clipper)
        self.reductions = TrainingReductionMeshes.from_topology(topo)
        self.dp_degree, self.dp_rank = topo.dp, topo.coord("dp")
        self.rows_per_rank = resolve_batch_size_per_rank(t.global_batch_size, self.dp_degree, t.gradient_accumulation_steps)
        arch = self.model.config
        self.dataloader = build_dataloader(t.dataloader_config, vocab_size=arch.vocab_size, global_batch=t.global_batch_size,
                                           seq_len=t.max_seq_len, seed=t.seed, dp_rank=self.dp_rank, dp_degree=self.dp_degree,
                                           rows_per_rank=self.rows_per_rank, pin_memory=env.device.type == "cuda", model=self.model)
        self.data_iterator = iter(self.dataloader)
        self.progress = TrainingProgress()
        self.num_params = sum(u.numel for u in self.asm.fsdp.units)
        sink = build_metric_logger(t.metrics_config, t.dump_folder, env.rank, cfg.to_dict())
        self.metrics = MetricsProcessor(t.metrics_config, world_size=env.world_size,
                                        flops_per_token=self.model.flops_per_token(t.max_seq_len), num_params=self.num_params,
                                        logger=self.logger, sink=sink, device=env.device if env.device.type == "cuda" else None)
        self.observer = TrainingObserver(t.metrics_config, env.device, env.world_size)
        self.dispatch_timer = None
        if t.metrics_config.measure_moe_dispatch:
            from ..models.moe import MoE
            from .runtime.observer import DispatchTimer
            self.dispatch_timer = DispatchTimer(env.device)
            for m in self.model.modules():
                if isinstance(m, MoE):
                    m.dispatch_timer = m.routed.dispatch_timer = self.dispatch_timer
        from ..utils import nvtx
        nvtx.enable(bool(getattr(t.profiler_config, "enable_profiling", False)))
        from ..components.checkpointer import build_checkpointer
        self.checkpointer = build_checkpointer(cfg, self)
        from ..components.profiler import build_profiler
        self.profiler = build_profiler(cfg, env)
        self.validator = None
        if t.validation_config is not None:
            from .runtime.validation import Validator
            self.validator = Validator(cfg, self)
        self.logger.info(f"assembled {type(self.model).__name__}: {self.num_params / 1e6:.1f}M local params, topology {topo.describe()}, "
                         f"dtype {env.param_dtype}, device {env.device}")

    # ------------------------------------------------------------------ one optimizer step
    def fetch_batch(self):
        """Read one micro-batch; all data-parallel ranks agree on (ready / exhausted / error)."""
        return fetch_batch(self.data_iterator, self.env)

    def train_step(self, batches=None, read_stats: bool = True, overlap_optimizer: bool = False) -> StepResult | None:
        """One optimizer step. `batches` overrides the data loader (a list of trainer batches, which may already
        live on the device); `read_stats=False` skips the single device->host read and returns None.
        `overlap_optimizer=True` (what the training loop passes when `overlap_optimizer_step` is set) lets the parameter
        update run on its own stream under the next step's forward; callers that look at parameters or optimizer state
        between steps leave it off, or call `self.asm.fsdp.sync_optimizer()` first."""
        t = self.config.training
        eng = self.engine
        eng.begin_step()
        if batches is None:
            batches = [self.fetch_batch() for _ in range(t.gradient_accumulation_steps)]
        gv = global_valid_tokens(batches, self.env.device, self.reductions)
        self.checkpointer.maybe_wait_for_staging()
        for i, b in enumerate(batches):
            with nvtx_range(f"forward_backward[{i}]"):
                eng.forward_backward(b, gv, is_last_microbatch=(i == len(batches) - 1))
        step = self.progress.step + 1
        with nvtx_range("optimizer_step"):
            norm = eng.optimizer_step(step, overlap=overlap_optimizer)
        if not read_stats:
            self.progress.step = step
            return None
        # one device->host read per step: [loss_sum, grad_norm, valid tokens]
        # (the kernels' status code rides in the same read)
        status = status_word(self.env.device)
        loss, gnorm, gtok, *code = build_step_metrics(eng.step_loss, norm, gv, self.reductions, status)
        if code and code[0]:
            check_status(f"training step {step}")                       # raises KernelStatusError with site and block
        if status is not None and os.environ.get("LLMT_DEBUG") == "1":
            from ..parallel.symm import damaged_arenas
            if damaged_arenas():
                raise KernelStatusError(f"training step {step}", 5, "a symmetric-memory arena lost its canary words: some kernel wrote past a buffer")
        eng.finish_step(step, loss)
        self.progress.step = step
        self.progress.ntokens_seen += int(gtok)
        return StepResult(step, loss, gnorm, self.lr_schedulers.get_last_lr()[0], int(gtok), 0.0)

    # ------------------------------------------------------------------ loop
    def train(self) -> None:
        t = self.config.training
        self.checkpointer.load(step=t.checkpoint_config.load_step)
        if t.checkpoint_config.load_only:
            return
        try:
            self._run_training()
        finally:
            self.checkpointer.wait()

    def _run_training(self) -> None:
        t = self.config.training
        with GarbageCollection(t.gc_freq) as gc_ctl, self.profiler:
            while self.progress.step < t.steps:
                self.observer.begin_step()
                try:
                    res = self.train_step(overlap_optimizer=t.overlap_optimizer_step)
                except DataloaderExhaustedError:
                    self.logger.info("data exhausted; stopping")
                    break
                tokens_local = t.max_seq_len * self.rows_per_rank * t.gradient_accumulation_steps // (self.env.topo.cp * self.env.topo.tp)
                sec, gtok = self.observer.end_step(tokens_local)
                res.step_seconds = sec
                self._report_completed_step(res, gtok)
                self.profiler.step()
                gc_ctl.run(res.step)
                if res.step == 1:
                    set_pg_timeouts(self.config.parallel.train_timeout_seconds, list(self.env.topo._groups.values()))

    def _report_completed_step(self, res: StepResult, global_tokens: int) -> None:
        moe_times = self.dispatch_timer.collect() if self.dispatch_timer is not None else {}
        if self.metrics.should_log(res.step):
            extra = {**self.observer.steady_state(), **moe_times}
            self.last_metrics = self.metrics.log(res.step, loss=res.loss, grad_norm=res.grad_norm, lr=res.lr,
                                                 global_tokens=global_tokens, step_seconds=res.step_seconds, extra=extra)
        self.checkpointer.save(res.step, last_step=(res.step == self.config.training.steps))
        if self.validator is not None and self.validator.should_validate(res.step):
            self.validator.validate(res.step)

    def validate(self):
        if self.validator is None:
            from .runtime.validation import Validator
            self.validator = Validator(self.config, self)
        return self.validator.validate(self.progress.step)

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        for name in ("checkpointer", "profiler", "metrics", "dataloader"):
            obj = getattr(self, name, None)
            if obj is not None and hasattr(obj, "close"):
                try:
                    obj.close()
                except Exception as e:  # noqa: BLE001
                    self.logger.error(f"closing {name} failed: {e}")
