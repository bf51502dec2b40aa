"""L0 utilities: logging, seeding, FLOP accounting, peak tables, GC control, metric sinks."""
from .logging import get_logger, set_log_ranks  # noqa: F401
from .seeding import seed_everything, set_deterministic_algorithms, preserve_rng_state, derive_distinct_seed  # noqa: F401
from .flops import generic_flops_per_token  # noqa: F401
from .monitoring import get_peak_flops  # noqa: F401
from .garbage_collection import GarbageCollection  # noqa: F401
from .vocabulary import vocab_shard_bounds  # noqa: F401
