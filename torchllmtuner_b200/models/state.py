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


@dataclass
class RefPiece:
    """`n` consecutive elements of the flattened native tensor, starting at `native_lo`, are elements
    `ref_lo .. ref_lo + n` of the flattened tensor `name` (whole shape `shape`) of the reference's own model classes."""
    name: str
    shape: tuple
    ref_lo: int
    native_lo: int
    n: int


class ModelStateFormat:
    name = "native"

    def to_reference(self, fqn: str, shape) -> list[RefPiece]:
        """Names and layouts of the reference's native modules (its distributed checkpoints are keyed by them). The
        default covers tensors that `to_hf` maps one to one."""
        pieces = self.to_hf(fqn, shape)
        if len(pieces) != 1:
            raise NotImplementedError(f"{self.name}: no reference layout for {fqn}")
        return [RefPiece(pieces[0].hf_name, tuple(shape), 0, pieces[0].native_flat_lo, pieces[0].native_flat_hi - pieces[0].native_flat_lo)]

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

    def to_reference(self, fqn, shape):
        # packed experts of the reference (llmtuner/models/qwen/qwen3/model.py:312): gate_up_proj (E, 2F, D) holds the gate
        # rows then the up rows of each expert, down_proj (E, D, F)
        m = self._EXP.match(fqn)
        if m:
            E, a, b = shape
            which = m.group(2)
            if which == "w2_EDF":
                return [RefPiece(f"{m.group(1)}.experts.down_proj", (E, a, b), 0, 0, E * a * b)]
            half = a * b
            off = 0 if which == "w1_EFD" else half
            return [RefPiece(f"{m.group(1)}.experts.gate_up_proj", (E, 2 * a, b), e * 2 * half + off, e * half, half) for e in range(E)]
        return super().to_reference(fqn, shape)

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
