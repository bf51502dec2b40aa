"""L2 kernel layer: hot ops with a hand-written sm_100a implementation for CUDA tensors and a plain PyTorch
statement for CPU tensors (reference facade: llmtuner/kernel/registry.py:1-103, llmtuner/kernel/ops/*.py)."""
from . import reference  # noqa: F401
from .attn_meta import AttnMeta  # noqa: F401
from .functional import (DEVICE_ATTENTION_HEAD_DIMS, IGNORE_INDEX, adamw_step_, add_rms_norm, attention, attention_with_lse, cross_entropy_sum,  # noqa: F401
                         gemm, linear, linears, linear_cross_entropy_sum, qk_norm_rope, rms_norm, rope_tables, sq_norm, swiglu)
from .registry import dispatch_kernel, get_kernel, register_kernel  # noqa: F401
