"""A self-contained teaching framework: a small Qwen3-MoE in plain PyTorch trained on a `(dp, ep, tp)` mesh with every
collective written out (reference: experiments/mini-llmtuner/README.md:1-80, model.py, layers.py, parallel.py, engine.py,
checkpoint.py). It imports nothing from the production package: one reads it top to bottom to see where each
parallelism cuts the model and which gradient needs which reduction.

    python -m torchllmtuner_b200.experiments.mini.train --device cpu --steps 3 --gradient-accumulation-steps 2
    python -m torchllmtuner_b200.experiments.mini.train --device cpu --steps 2 --checkpoint /tmp/mini
    python -m torchllmtuner_b200.experiments.mini.train --device cpu --steps 3 --resume /tmp/mini
"""
from .config import MiniConfig
from .trainer import MiniTrainer

__all__ = ["MiniConfig", "MiniTrainer"]
