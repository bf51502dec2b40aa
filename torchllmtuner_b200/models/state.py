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


def refuse_unsupported_hf_settings(hf: dict, accepted: dict) -> None:
    """A config.json may switch on something this framework's model of the family does not have (a bias on the attention
    projections, a sliding window, a scaled rotary embedding). Building the model anyway would load the weights it knows
    and silently compute something else, so such a folder is refused, naming the setting."""
    from ..errors import UnsupportedCombinationError
    for key, ok in accepted.items():
        if key in hf and hf[key] is not None and hf[key] not in ok:
            raise UnsupportedCombinationError(f"config.json sets {key}={hf[key]!r}; this framework's model supports {key} in {list(ok)}")
    rope = hf.get("rope_parameters") or hf.get("rope_scaling") or {}
    kind = rope.get("rope_type", rope.get("type", "default")) if isinstance(rope, dict) else "default"
    if kind not in ("default", None):
        raise UnsupportedCombinationError(f"config.json asks for a {kind!r} rotary embedding; only the default one is built")


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

    def hf_pieces(self, fqn: str, shape) -> list[RefPiece]:
        """The general form of `to_hf`, used by the safetensors import / export: several native tensors may fill one HF
        tensor (packed gate/up experts). The default restates `to_hf`: one HF tensor per piece, and when a native tensor
        splits into several (per-expert files) each takes the native shape without its leading dimension."""
        pieces = self.to_hf(fqn, shape)
        pshape = tuple(shape[1:]) if len(pieces) > 1 else tuple(shape)
        return [RefPiece(p.hf_name, pshape, 0, p.native_flat_lo, p.native_flat_hi - p.native_flat_lo) for p in pieces]

    def hf_config(self, arch) -> dict:
        return dict(vars(arch))

    def hf_config_of(self, model) -> dict:
        """config.json for `model`; formats whose file describes more than the decoder's architecture override this."""
        return self.hf_config(model.config)

    # `model_name_or_path=<folder>`: which registered model a config.json's `model_type` builds, and the architecture
    # fields it carries (the inverse of `hf_config`; fields a builder does not know are ignored by it)
    hf_model_types: dict = {}

    def arch_from_hf(self, hf: dict) -> dict:
        out = {k: v for k, v in hf.items() if not isinstance(v, dict)}
        rope = hf.get("rope_parameters")               # transformers 5 nests what used to be the top-level `rope_theta`
        if isinstance(rope, dict) and "rope_theta" in rope:
            out.setdefault("rope_theta", rope["rope_theta"])
        return out

    def hf_aliases(self, name: str) -> list[str]:
        """Other names under which published files may store the tensor `name` (tried in order when `name` is absent)."""
        return []

    def hf_piece_variants(self, fqn: str, shape) -> list[list[RefPiece]]:
        """Layouts in which published files may hold the native tensor `fqn`; the first is what the export writes. The
        importer takes the first one whose tensors are all there."""
        return [self.hf_pieces(fqn, shape)]


class Qwen3StateFormat(ModelStateFormat):
    name = "qwen3"
    hf_model_types = {"qwen3": "qwen3_moe", "qwen3_moe": "qwen3_moe"}

    def arch_from_hf(self, hf: dict) -> dict:
        out = ModelStateFormat.arch_from_hf(self, hf)
        # a dense config.json has neither key; published files say `num_experts`, transformers 5 writes `num_local_experts`
        out["num_experts"] = hf.get("num_experts", hf.get("num_local_experts", 0)) or 0
        refuse_unsupported_hf_settings(hf, {"attention_bias": (False,), "use_sliding_window": (False,), "hidden_act": ("silu",),
                                            "attention_dropout": (0, 0.0)})
        return out
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


class DeepseekV4StateFormat(Qwen3StateFormat):
    """Native names follow the reference's module tree except inside the MoE block: the router projection is
    `mlp.gate.weight`, the hash table `mlp.gate.tid2eid`, the indexer's head weights sit under `indexer.scorer`
    (reference: llmtuner/models/deepseek/deepseek_v4/modeling.py:219-247, indexer.py:18-60). Experts: one tensor per
    expert and projection in HF files, packed `gate_up_proj` / `down_proj` in the reference's own checkpoints."""
    name = "deepseek_v4"
    hf_model_types = {"deepseek_v4": "deepseek_v4"}

    def arch_from_hf(self, hf: dict) -> dict:
        out = ModelStateFormat.arch_from_hf(self, hf)
        out["num_experts"] = hf.get("n_routed_experts", hf.get("num_experts", 0))
        if "moe_intermediate_size" not in hf and "intermediate_size" in hf:      # published files call the expert width this
            out["moe_intermediate_size"] = hf["intermediate_size"]
        rope = hf.get("rope_parameters") or {}
        if "main" in rope:
            out["rope_theta"] = rope["main"].get("rope_theta", out.get("rope_theta"))
        if "compress" in rope:
            out["compress_rope_theta"] = rope["compress"].get("rope_theta", out.get("compress_rope_theta"))
        return {k: v for k, v in out.items() if v is not None}

    _RENAMES = ((re.compile(r"^(model\.layers\.\d+\.mlp)\.router\.gate\.weight$"), r"\1.gate.weight"),
                (re.compile(r"^(model\.layers\.\d+\.self_attn\.compressor\.indexer)\.weights_proj\.weight$"), r"\1.scorer.weights_proj.weight"))
    BUFFER_RENAMES = {"mlp.router.tid2eid": "mlp.gate.tid2eid", "mlp.expert_bias_E": "mlp.gate.e_score_correction_bias"}

    def _rename(self, fqn: str) -> str:
        for rx, to in self._RENAMES:
            if rx.match(fqn):
                return rx.sub(to, fqn)
        return fqn

    def to_hf(self, fqn, shape):
        if self._EXP.match(fqn):
            return super().to_hf(fqn, shape)
        n = 1
        for x in shape:
            n *= x
        return [HFPiece(self._rename(fqn), 0, n)]

    def to_reference(self, fqn, shape):
        if self._EXP.match(fqn):
            return super().to_reference(fqn, shape)
        n = 1
        for x in shape:
            n *= x
        return [RefPiece(self._rename(fqn), tuple(shape), 0, 0, n)]

    def hf_config(self, arch) -> dict:
        keep = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "head_dim", "q_lora_rank", "o_lora_rank",
                "o_groups", "qk_rope_head_dim", "swiglu_limit", "rms_norm_eps", "sliding_window", "layer_types", "mlp_layer_types",
                "compress_rates", "index_head_dim", "index_n_heads", "index_topk", "hc_mult", "hc_eps", "hc_sinkhorn_iters",
                "num_experts_per_tok", "scoring_func", "routed_scaling_factor", "tie_word_embeddings", "max_position_embeddings")
        cfg = {k: getattr(arch, k) for k in keep}
        cfg.update(architectures=["DeepseekV4ForCausalLM"], model_type="deepseek_v4", n_routed_experts=arch.num_experts,
                   intermediate_size=arch.moe_intermediate_size, n_shared_experts=1, hidden_act="silu", torch_dtype="bfloat16",
                   rope_parameters={"main": {"rope_type": "default", "rope_theta": arch.rope_theta,
                                             "partial_rotary_factor": arch.qk_rope_head_dim / arch.head_dim},
                                    "compress": {"rope_type": "default", "rope_theta": arch.compress_rope_theta,
                                                 "partial_rotary_factor": arch.qk_rope_head_dim / arch.head_dim}})
        return cfg


class Qwen35StateFormat(ModelStateFormat):
    """Qwen3.5: the delta-net mixer is `linear_attn` in published files, the router `mlp.gate`, the shared expert
    `mlp.shared_expert`, experts packed as `mlp.experts.gate_up_proj` (E, 2F, D: gate rows then up rows of each expert) and
    `mlp.experts.down_proj` (reference: llmtuner/models/qwen/qwen3_5_moe/model.py:217-275, gated_delta.py:34-72)."""
    name = "qwen3_5"
    hf_model_types = {"qwen3_5_text": "qwen3_5", "qwen3_5_moe_text": "qwen3_5_moe", "qwen3_5": "qwen3_5", "qwen3_5_moe": "qwen3_5_moe"}

    def arch_from_hf(self, hf: dict) -> dict:
        hf = hf.get("text_config") or hf                      # the vision-language config nests the decoder's
        out = ModelStateFormat.arch_from_hf(self, hf)
        rope = hf.get("rope_parameters") or hf.get("rope_scaling") or {}
        for k in ("rope_theta", "partial_rotary_factor", "mrope_section"):
            if k in rope:
                out[k] = rope[k]
        out["num_experts"] = hf.get("num_experts", hf.get("num_local_experts", 0)) or 0
        out.pop("model_type", None)                           # the registered builder names it
        return out

    def hf_aliases(self, name: str) -> list[str]:
        # transformers writes the text decoder under the vision-language model's tree, also for text-only checkpoints
        return ["model.language_model." + name[len("model."):]] if name.startswith("model.") else []

    _LINEAR = re.compile(r"^(model\.layers\.\d+)\.self_attn\.((?:in_proj_(?:qkv|z|b|a)|conv1d|norm|out_proj)\.weight|dt_bias|A_log)$")
    _EXP = re.compile(r"^(model\.layers\.\d+\.mlp)\.routed\.experts\.(w1_EFD|w3_EFD|w2_EDF)$")
    _ROUTER = re.compile(r"^(model\.layers\.\d+\.mlp)\.router\.gate\.weight$")
    _SHARED = re.compile(r"^(model\.layers\.\d+\.mlp)\.shared_experts\.(.+)$")

    def hf_pieces(self, fqn, shape):
        n = 1
        for x in shape:
            n *= x
        m = self._EXP.match(fqn)
        if m:
            E, a, b = shape
            if m.group(2) == "w2_EDF":
                return [RefPiece(f"{m.group(1)}.experts.down_proj", (E, a, b), 0, 0, n)]
            half = a * b
            off = 0 if m.group(2) == "w1_EFD" else half
            return [RefPiece(f"{m.group(1)}.experts.gate_up_proj", (E, 2 * a, b), e * 2 * half + off, e * half, half) for e in range(E)]
        for rx, fmt in ((self._LINEAR, "{0}.linear_attn.{1}"), (self._ROUTER, "{0}.gate.weight"), (self._SHARED, "{0}.shared_expert.{1}")):
            m = rx.match(fqn)
            if m:
                return [RefPiece(fmt.format(*m.groups()), tuple(shape), 0, 0, n)]
        return [RefPiece(fqn, tuple(shape), 0, 0, n)]

    to_reference = hf_pieces

    _PROJ = {"w1_EFD": "gate_proj", "w3_EFD": "up_proj", "w2_EDF": "down_proj"}

    def hf_piece_variants(self, fqn, shape):
        """Packed experts are what the module tree holds; files written by `save_pretrained` carry one tensor per expert
        and projection (`experts.<e>.gate_proj.weight`), as Qwen3-MoE files do."""
        each = self._per_expert(fqn, shape)
        return [self.hf_pieces(fqn, shape)] + ([each] if each else [])

    def _per_expert(self, fqn, shape):
        m = self._EXP.match(fqn)
        if not m:
            return None
        E, a, b = shape
        return [RefPiece(f"{m.group(1)}.experts.{e}.{self._PROJ[m.group(2)]}.weight", (a, b), 0, e * a * b, a * b) for e in range(E)]

    def to_hf(self, fqn, shape):
        if self._EXP.match(fqn) and not fqn.endswith("w2_EDF"):
            raise NotImplementedError("packed gate/up experts: use hf_pieces")
        return [HFPiece(p.name, p.native_lo, p.native_lo + p.n) for p in self.hf_pieces(fqn, shape)]

    def hf_config(self, arch) -> dict:
        moe = arch.num_experts > 0
        keep = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                "rms_norm_eps", "layer_types", "full_attention_interval", "linear_num_value_heads", "linear_num_key_heads",
                "linear_key_head_dim", "linear_value_head_dim", "linear_conv_kernel_dim", "attn_output_gate", "tie_word_embeddings",
                "max_position_embeddings")
        cfg = {k: getattr(arch, k) for k in keep}
        cfg.update(architectures=["Qwen3_5MoeForCausalLM" if moe else "Qwen3_5ForCausalLM"], model_type="qwen3_5_moe_text" if moe else "qwen3_5_text",
                   hidden_act="silu", torch_dtype="bfloat16",
                   rope_parameters={"rope_type": "default", "rope_theta": arch.rope_theta, "partial_rotary_factor": arch.partial_rotary_factor,
                                    "mrope_section": list(arch.mrope_section), "mrope_interleaved": True})
        if moe:
            cfg.update(num_experts=arch.num_experts, num_experts_per_tok=arch.num_experts_per_tok, moe_intermediate_size=arch.moe_intermediate_size,
                       shared_expert_intermediate_size=arch.shared_expert_intermediate_size, norm_topk_prob=arch.norm_topk_prob)
        return cfg


class Qwen35VLStateFormat(Qwen35StateFormat):
    """The vision-language model: the text decoder's tensors (`text.` here) sit under `model.language_model.` in
    published files, the tower's (`visual.`) under `model.visual.`; `lm_head.weight` stays at the top. With the
    `models/qwen_vit.py` tower the names and shapes below `visual.` are the published ones."""
    name = "qwen3_5_vl"
    hf_model_types: dict = {}        # a vision-language folder builds the text decoder unless the run names a `_vl` model

    @staticmethod
    def _place(piece: RefPiece) -> RefPiece:
        name = piece.name
        if name.startswith("model."):
            name = "model.language_model." + name[len("model."):]
        return RefPiece(name, piece.shape, piece.ref_lo, piece.native_lo, piece.n)

    def hf_piece_variants(self, fqn, shape):
        if fqn.startswith("text."):
            inner = fqn[len("text."):]
            variants = [Qwen35StateFormat.hf_pieces(self, inner, shape)]
            each = self._per_expert(inner, shape)
            return [[self._place(p) for p in v] for v in variants + ([each] if each else [])]
        n = 1
        for x in shape:
            n *= x
        if fqn.startswith("visual."):
            return [[RefPiece("model." + fqn, tuple(shape), 0, 0, n)]]
        return [[RefPiece(fqn, tuple(shape), 0, 0, n)]]

    def hf_pieces(self, fqn, shape):
        return self.hf_piece_variants(fqn, shape)[0]

    to_reference = hf_pieces

    def hf_aliases(self, name: str) -> list[str]:
        return []

    def hf_config(self, arch) -> dict:
        text = Qwen35StateFormat.hf_config(self, arch)
        return {"architectures": ["Qwen3_5MoeForConditionalGeneration" if arch.num_experts > 0 else "Qwen3_5ForConditionalGeneration"],
                "model_type": "qwen3_5_moe" if arch.num_experts > 0 else "qwen3_5", "text_config": text,
                "tie_word_embeddings": arch.tie_word_embeddings, "torch_dtype": "bfloat16"}

    def hf_config_of(self, model) -> dict:
        """Adds what only the whole model knows: the placeholder token and, for the published tower, its geometry."""
        cfg = self.hf_config(model.config)
        cfg["image_token_id"] = int(model.image_token_id)
        v = getattr(getattr(model, "visual", None), "config", None)
        if v is not None and hasattr(v, "num_position_embeddings"):
            cfg["vision_config"] = {k: getattr(v, k) for k in ("depth", "hidden_size", "intermediate_size", "num_heads", "in_channels", "patch_size",
                                                              "spatial_merge_size", "temporal_patch_size", "out_hidden_size",
                                                              "num_position_embeddings")}
            cfg["vision_config"].update(model_type=cfg["model_type"], hidden_act="gelu_pytorch_tanh")
        return cfg


class KimiStateFormat(ModelStateFormat):
    """Kimi checkpoints name the sparse block `block_sparse_moe` and keep one module per expert with projections `w1`
    (gate), `w3` (up), `w2` (down); the reference's own module tree is the same, so its distributed checkpoints use these
    names too (reference: llmtuner/models/kimi/kimi_k3/model.py:102-110, mlp.py:47-61, checkpoint.py:27-342)."""
    name = "kimi"
    hf_model_types = {"kimi_linear": "kimi_linear", "kimi_k3": "kimi_k3"}

    def arch_from_hf(self, hf: dict) -> dict:
        hf = hf.get("text_config") or hf
        out = ModelStateFormat.arch_from_hf(self, hf)
        if "num_experts_per_token" in hf:
            out["num_experts_per_tok"] = hf["num_experts_per_token"]
        lin = hf.get("linear_attn_config") or {}
        for theirs, ours in (("kda_layers", "kda_layers"), ("num_heads", "linear_heads"), ("head_dim", "linear_head_dim"),
                             ("short_conv_kernel_size", "short_conv_kernel_size"), ("use_full_rank_gate", "use_full_rank_gate"),
                             ("gate_lower_bound", "gate_lower_bound")):
            if theirs in lin:
                out[ours] = lin[theirs]
        out.pop("model_type", None)
        return out

    _EXP = re.compile(r"^(model\.layers\.\d+)\.mlp\.routed\.experts\.(w1_EFD|w3_EFD|w2_EDF)$")
    _SPARSE = re.compile(r"^(model\.layers\.\d+)\.mlp\.(router\.gate\.weight|shared_experts\..+|routed_expert_(?:down_proj|up_proj|norm)\.weight)$")
    _PROJ = {"w1_EFD": "w1", "w3_EFD": "w3", "w2_EDF": "w2"}
    BUFFER_RENAMES = {"mlp.expert_bias_E": "block_sparse_moe.gate.e_score_correction_bias"}

    def to_hf(self, fqn, shape):
        m = self._EXP.match(fqn)
        if m:
            per = shape[1] * shape[2]
            return [HFPiece(f"{m.group(1)}.block_sparse_moe.experts.{e}.{self._PROJ[m.group(2)]}.weight", e * per, (e + 1) * per)
                    for e in range(shape[0])]
        m = self._SPARSE.match(fqn)
        n = 1
        for x in shape:
            n *= x
        if m:
            tail = "gate.weight" if m.group(2) == "router.gate.weight" else m.group(2)
            return [HFPiece(f"{m.group(1)}.block_sparse_moe.{tail}", 0, n)]
        return [HFPiece(fqn, 0, n)]

    def to_reference(self, fqn, shape):
        m = self._EXP.match(fqn)
        if m:
            per = shape[1] * shape[2]
            return [RefPiece(p.hf_name, tuple(shape[1:]), 0, p.native_flat_lo, per) for p in self.to_hf(fqn, shape)]
        p = self.to_hf(fqn, shape)[0]
        return [RefPiece(p.hf_name, tuple(shape), 0, 0, p.native_flat_hi)]

    def hf_config(self, arch) -> dict:
        keep = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                "rms_norm_eps", "q_lora_rank", "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "mla_use_output_gate",
                "first_k_dense_replace", "moe_layer_freq", "num_experts", "num_shared_experts", "num_expert_group", "topk_group",
                "moe_renormalize", "routed_scaling_factor", "moe_router_activation_func", "moe_intermediate_size",
                "routed_expert_hidden_size", "latent_moe_use_norm", "hidden_act", "activation_situ_beta", "activation_situ_linear_beta",
                "attn_res_block_size", "tie_word_embeddings")
        cfg = {k: getattr(arch, k) for k in keep}
        n = arch.num_hidden_layers
        cfg.update(architectures=["KimiLinearForCausalLM"], model_type="kimi_linear", num_experts_per_token=arch.num_experts_per_tok,
                   mla_use_nope=True, torch_dtype="bfloat16",
                   linear_attn_config={"kda_layers": list(arch.kda_layers), "full_attn_layers": [i + 1 for i in range(n) if (i + 1) not in arch.kda_layers],
                                       "num_heads": arch.linear_heads, "head_dim": arch.linear_head_dim,
                                       "short_conv_kernel_size": arch.short_conv_kernel_size, "use_full_rank_gate": arch.use_full_rank_gate,
                                       "gate_lower_bound": arch.gate_lower_bound})
        return cfg


_FORMATS = {"native": ModelStateFormat(), "qwen3": Qwen3StateFormat(), "deepseek_v4": DeepseekV4StateFormat(), "kimi": KimiStateFormat(),
            "qwen3_5": Qwen35StateFormat(), "qwen3_5_vl": Qwen35VLStateFormat()}


def registered_for_hf_model_type(model_type: str):
    """(registry key, state format) that builds a config.json of this `model_type`, or (None, None)."""
    for fmt in _FORMATS.values():
        key = fmt.hf_model_types.get(model_type)
        if key is not None:
            return key, fmt
    return None, None


def get_state_format(name: str) -> ModelStateFormat:
    return _FORMATS.get(name, _FORMATS["native"])


def register_state_format(fmt: ModelStateFormat) -> None:
    _FORMATS[fmt.name] = fmt
