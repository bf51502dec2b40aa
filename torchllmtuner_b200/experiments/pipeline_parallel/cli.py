"""`python -m torchllmtuner_b200.experiments.pipeline_parallel.cli --pipeline_parallel_size 2 --pp_schedule 1F1B ...`
accepts the production flags plus `--pp_schedule` and `--num_pp_microbatches`."""
from __future__ import annotations

import sys

from ...config import LLMTunerConfig, build_parser


def main(argv=None) -> int:
    import torch.distributed as dist

    from .runtime import PipelineTrainer
    parser = build_parser()
    parser.add_argument("--pp_schedule", default="1F1B")
    parser.add_argument("--num_pp_microbatches", type=int, default=None)
    ns = vars(parser.parse_args(argv))
    sched, nmb, path = ns.pop("pp_schedule"), ns.pop("num_pp_microbatches"), ns.pop("config", None)
    cfg = LLMTunerConfig.from_file(path) if path else LLMTunerConfig()
    cfg.apply_flat(ns)
    tr = PipelineTrainer(cfg, sched, nmb)
    try:
        for _ in range(cfg.training.steps):
            loss = tr.train_step()
            tr.logger.info(f"step {tr.step} loss {loss:.4f}")
    finally:
        tr.close()
        if dist.is_initialized():
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
