"""Throughput / MFU / memory metrics and the console line (reference: llmtuner/components/metrics.py:61-768)."""
from __future__ import annotations

import time
from dataclasses import dataclass

import torch

from ..utils.monitoring import get_measured_peak_flops, get_peak_flops


def token_throughput(tokens: int, seconds: float) -> float:
    return tokens / seconds if seconds > 0 else 0.0


def model_tflops(tps_per_device: float, flops_per_token: float) -> float:
    return tps_per_device * flops_per_token / 1e12


def compute_utilization(tflops: float, peak_flops: float) -> float:
    return 100.0 * tflops * 1e12 / peak_flops if peak_flops > 0 else 0.0


class DeviceMemoryMonitor:
    def __init__(self, device=None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.device = device
        self.total = torch.cuda.get_device_properties(device or 0).total_memory if self.cuda else 0

    def stats(self) -> dict[str, float]:
        if not self.cuda:
            return {}
        s = torch.cuda.memory_stats(self.device)
        gib = 1024.0 ** 3
        peak_res, peak_act = s.get("reserved_bytes.all.peak", 0), s.get("active_bytes.all.peak", 0)
        return {"memory/max_reserved(GiB)": peak_res / gib, "memory/max_reserved(%)": 100.0 * peak_res / max(1, self.total),
                "memory/max_active(GiB)": peak_act / gib, "memory/allocated(GiB)": s.get("allocated_bytes.all.current", 0) / gib,
                "memory/num_alloc_retries": float(s.get("num_alloc_retries", 0)), "memory/num_ooms": float(s.get("num_ooms", 0))}

    def reset_peak(self) -> None:
        if self.cuda:
            torch.cuda.reset_peak_memory_stats(self.device)


@dataclass
class DerivedMetrics:
    global_tps: float
    tps_per_device: float
    tflops_per_device: float
    mfu_percent: float
    mfu_measured_percent: float


class MetricsProcessor:
    """Builds the metric dict of a logged step and the console line:
    step, loss, grad_norm, memory, step_time, lr, tps/device, tflops/device, mfu."""

    def __init__(self, metrics_cfg, *, world_size: int, flops_per_token: float, num_params: int, logger, sink=None, device=None):
        self.cfg, self.world, self.flops_per_token, self.num_params = metrics_cfg, world_size, flops_per_token, num_params
        self.logger, self.sink = logger, sink
        self.peak = get_peak_flops() if torch.cuda.is_available() else 0.0
        self.measured_peak = get_measured_peak_flops()
        self.mem = DeviceMemoryMonitor(device)
        self.t_last = time.perf_counter()

    def should_log(self, step: int) -> bool:
        return step == 1 or step % self.cfg.log_freq == 0

    def derive(self, global_tokens: int, step_seconds: float) -> DerivedMetrics:
        gtps = token_throughput(global_tokens, step_seconds)
        per = gtps / max(1, self.world)
        tf = model_tflops(per, self.flops_per_token)
        return DerivedMetrics(gtps, per, tf, compute_utilization(tf, self.peak), compute_utilization(tf, self.measured_peak))

    def log(self, step: int, *, loss: float, grad_norm: float, lr: float, global_tokens: int, step_seconds: float,
            max_loss: float | None = None, extra: dict | None = None) -> dict:
        d = self.derive(global_tokens, step_seconds)
        m = {"loss_metrics/global_avg_loss": loss, "loss_metrics/global_max_loss": max_loss if max_loss is not None else loss,
             "grad_norm": grad_norm, "lr": lr, "throughput(tps)": d.global_tps, "tps_per_device": d.tps_per_device,
             "tflops": d.tflops_per_device, "mfu(%)": d.mfu_percent, "mfu_measured(%)": d.mfu_measured_percent,
             "time_metrics/end_to_end(s)": step_seconds, **self.mem.stats(), **(extra or {})}
        mem = m.get("memory/max_reserved(GiB)", 0.0)
        self.logger.info(f"step: {step:5d}  loss: {loss:8.4f}  grad_norm: {grad_norm:8.4f}  memory: {mem:6.2f}GiB"
                         f"({m.get('memory/max_reserved(%)', 0.0):.1f}%)  step_time: {step_seconds * 1e3:8.1f}ms  lr: {lr:.3e}"
                         f"  params: {self.num_params / 1e6:.1f}M  tps/device: {d.tps_per_device:,.0f}"
                         f"  tflops/device: {d.tflops_per_device:,.1f}  mfu: {d.mfu_percent:.2f}%")
        if self.sink is not None:
            self.sink.log(m, step)
        self.mem.reset_peak()
        return m

    def close(self) -> None:
        if self.sink is not None:
            self.sink.close()
