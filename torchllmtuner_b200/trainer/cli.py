"""Command line: flat flags over the thirteen config groups plus `--config file.{yaml,json}`
(reference: llmtuner/trainer/cli.py:57-158). Flags override file values."""
from __future__ import annotations

import sys

from ..config import LLMTunerConfig, build_parser


def parse_config(argv=None) -> LLMTunerConfig:
    ns = vars(build_parser().parse_args(argv))
    path = ns.pop("config", None)
    cfg = LLMTunerConfig.from_file(path) if path else LLMTunerConfig()
    cfg.apply_flat(ns)
    cfg.__post_init__()
    return cfg


def run_training(config: LLMTunerConfig) -> None:
    import torch.distributed as dist

    from .trainer import Trainer
    trainer = Trainer(config)
    try:
        ck = config.training.checkpoint_config
        if ck.create_seed_checkpoint:
            if trainer.env.world_size != 1 or not ck.enable:
                from ..errors import ConfigError
                raise ConfigError("create_seed_checkpoint needs a single process and an enabled checkpoint")
            trainer.checkpointer.save(0, force=True)
        else:
            trainer.train()
    finally:
        trainer.close()
        if dist.is_initialized():
            dist.destroy_process_group()


def main(argv=None) -> int:
    run_training(parse_config(argv))
    return 0


if __name__ == "__main__":
    sys.exit(main())
