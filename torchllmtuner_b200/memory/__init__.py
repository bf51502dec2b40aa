"""Memory policies: activation checkpointing, activation offload, meta-device materialisation."""
