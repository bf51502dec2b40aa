from .container import EMA, GradientClipper, OptimizersContainer, build_optimizers, check_finite  # noqa: F401
from .lr_scheduler import LRSchedulersContainer, build_lr_scheduler, wsd_factor  # noqa: F401
from .sharded import ShardedAdamW  # noqa: F401
