"""Metric sinks: TensorBoard and Weights & Biases, each optional
(reference: llmtuner/utils/metric_loggers.py:32-164)."""
from __future__ import annotations

import json
import os


def _scalars(metrics: dict) -> dict:
    """Only numbers reach a sink: a step may carry notes (a string, None) beside its measurements."""
    out = {}
    for k, v in metrics.items():
        if isinstance(v, bool) or v is None:
            continue
        try:
            out[k] = float(v)
        except (TypeError, ValueError):
            continue
    return out


class BaseLogger:
    def log(self, metrics: dict, step: int) -> None:  # pragma: no cover - interface
        pass

    def close(self) -> None:
        pass


class JsonlLogger(BaseLogger):
    """Always-available sink: one JSON line per logged step."""

    def __init__(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._f = open(path, "a")

    def log(self, metrics, step):
        self._f.write(json.dumps({"step": step, **_scalars(metrics)}) + "\n")
        self._f.flush()

    def close(self):
        self._f.close()


class TensorBoardLogger(BaseLogger):
    def __init__(self, log_dir: str, tag: str | None = None):
        from torch.utils.tensorboard import SummaryWriter  # raises ImportError when tensorboard is absent
        self.tag = tag
        self.writer = SummaryWriter(log_dir, max_queue=1000)

    def log(self, metrics, step):
        for k, v in _scalars(metrics).items():
            self.writer.add_scalar(k if self.tag is None else f"{self.tag}/{k}", v, step)

    def close(self):
        self.writer.close()


class WandBLogger(BaseLogger):
    def __init__(self, log_dir: str, tag: str | None = None, config: dict | None = None):
        import wandb
        self.wandb, self.tag = wandb, tag
        wandb.init(project=os.environ.get("WANDB_PROJECT", "torchllmtuner_b200"), dir=log_dir, config=config)

    def log(self, metrics, step):
        self.wandb.log({(k if self.tag is None else f"{self.tag}/{k}"): v for k, v in _scalars(metrics).items()}, step=step)

    def close(self):
        self.wandb.finish()


class LoggerContainer(BaseLogger):
    def __init__(self, loggers=()):
        self.loggers = list(loggers)

    def log(self, metrics, step):
        for lg in self.loggers:
            lg.log(metrics, step)

    def close(self):
        for lg in self.loggers:
            lg.close()


def build_metric_logger(metrics_config, dump_folder: str, rank: int, config_dict: dict | None = None) -> LoggerContainer:
    out = LoggerContainer()
    if rank not in metrics_config.log_ranks and not metrics_config.save_for_all_ranks:
        return out
    if metrics_config.enable_tensorboard:
        folder = os.path.join(dump_folder, metrics_config.save_tb_folder)
        if metrics_config.save_for_all_ranks:
            folder = os.path.join(folder, f"rank_{rank}")
        try:
            out.loggers.append(TensorBoardLogger(folder, metrics_config.tag))
        except ImportError:
            out.loggers.append(JsonlLogger(os.path.join(folder, "metrics.jsonl")))
    if metrics_config.enable_wandb:
        try:
            out.loggers.append(WandBLogger(dump_folder, metrics_config.tag, config_dict))
        except ImportError:
            pass
    return out
