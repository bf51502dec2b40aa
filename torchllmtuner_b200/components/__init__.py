"""L6 components: losses, optimizers, checkpointing, metrics, profiler, tokenizers."""
