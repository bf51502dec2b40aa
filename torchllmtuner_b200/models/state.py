"""Model state formats: native parameter names/layouts <-> Hugging Face names/layouts
(reference: llmtuner/models/state.py:19-133, llmtuner/models/qwen/qwen3/state.py:1-169).

A format maps one native tensor (by canonical FQN) to one or more HF tensors and back. Qwen3: dense names are
identical; the router is `mlp.gate.weight`; packed experts `w1_EFD/w3_EFD/w2_EDF` become per-expert
`mlp.experts.<e>.{gate,up,down}_proj.weight`."""
from __future__ import annotations

import re
from dataclasses import dataclass


@dataclass
class HFPiece:
    hf_name: str
    native_flat_lo: int       # range of the flattened native tensor covered by this HF tensor
    native_flat_hi: int


class ModelStateFormat:
    name = "native"

    def to_hf(self, fqn: str, shape) -> list[HFPiece]:
        n = 1
        for s in shape:
            n *= s
        return [HFPiece(fqn, 0, n)]

    def hf_config(self, arch) -> dict:
        return dict(vars(arch))


class Qwen3StateFormat(ModelStateFormat):
    name = "qwen3"
    _EXP = re.compile(r"^(model\.layers\.\d+\.mlp)\.routed\.experts\.(w1_EFD|w3_EFD|w2_EDF)$")
    _ROUTER = re.compile(r"^(model\.layers\.\d+\.mlp)\.router\.gate\.weight$")
    _PROJ = {"w1_EFD": "gate_proj", "w3_EFD": "up_proj", "w2_EDF": "down_proj"}

    def to_hf(self, fqn, shape):
        m = self._EXP.match(fqn)
        if m:
            E = shape[0]
            per = shape[1] * shape[2]
            return [HFPiece(f"{m.group(1)}.experts.{e}.{self._PROJ[m.group(2)]}.weight", e * per, (e + 1) * per) for e in range(E)]
        m = self._ROUTER.match(fqn)
        if m:
            return [HFPiece(f"{m.group(1)}.gate.weight", 0, shape[0] * shape[1])]
        return super().to_hf(fqn, shape)

    def hf_config(self, arch) -> dict:
        moe = arch.num_experts > 0
        cfg = {"architectures": ["Qwen3MoeForCausalLM" if moe else "Qwen3ForCausalLM"], "model_type": "qwen3_moe" if moe else "qwen3",
               "vocab_size": arch.vocab_size, "hidden_size": arch.hidden_size, "intermediate_size": arch.intermediate_size,
               "num_hidden_layers": arch.num_hidden_layers, "num_attention_heads": arch.num_attention_heads,
               "num_key_value_heads": arch.num_key_value_heads, "head_dim": arch.head_dim, "rms_norm_eps": arch.rms_norm_eps,
               "rope_theta": arch.rope_theta, "tie_word_embeddings": arch.tie_word_embeddings, "hidden_act": "silu",
               "max_position_embeddings": arch.max_position_embeddings, "torch_dtype": "bfloat16"}
        if moe:
            cfg.update(num_experts=arch.num_experts, num_experts_per_tok=arch.num_experts_per_tok,
                       moe_intermediate_size=arch.moe_intermediate_size, norm_topk_prob=arch.norm_topk_prob,
                       decoder_sparse_step=arch.decoder_sparse_step, mlp_only_layers=list(arch.mlp_only_layers))
        return cfg


_FORMATS = {"native": ModelStateFormat(), "qwen3": Qwen3StateFormat()}


def get_state_format(name: str) -> ModelStateFormat:
    return _FORMATS.get(name, _FORMATS["native"])


def register_state_format(fmt: ModelStateFormat) -> None:
    _FORMATS[fmt.name] = fmt
