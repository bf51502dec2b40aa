"""L7 datasets: contracts, synthetic sources, text recipes, packing, collators, loader builder."""
from .contracts import BaseDataLoader, Batch, DataloaderExhaustedError, IGNORE_INDEX, TextSequence, to_trainer_batch  # noqa: F401
from .loader_builder import build_dataloader  # noqa: F401
from .synthetic import RandomPackedSource, RandomTokenDataLoader, RandomTokenSource  # noqa: F401
