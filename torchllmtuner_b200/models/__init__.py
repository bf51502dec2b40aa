"""L4 models: registry, structural contracts, Qwen3 dense/MoE and the shared MoE stack."""
from .contracts import BoundDecoder, DecoderStructure, GatedMLPStructure, MoEBlockContract  # noqa: F401
from .qwen3 import QWEN3_8B, QWEN3_30B_A3B, ForwardContext, Qwen3Config, Qwen3ForCausalLM, build_qwen3  # noqa: F401
from .registry import (ModelSpec, build_registered_model, get_model_spec, register_model, registered_models,  # noqa: F401
                       resolve_state_format)
