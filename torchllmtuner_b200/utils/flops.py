"""Model FLOPs per token (reference: llmtuner/utils/flops.py:25-171).

flops/token = 3 * [sum_layers(attn_params + ffn_params) + 2*V*D] + sum_layers 6*Hq*(d_qk+d_v)*S
with attn_params = 2*(D*Hq*d + 2*D*Hkv*d + Hq*d*D); dense ffn = 3*2*D*F;
MoE ffn = 2*(D*E + k*3*D*Fe + 3*D*F_shared). No causal discount, no recompute credit.
"""
from __future__ import annotations


def generic_flops_per_token(*, hidden_size: int, num_layers: int, num_heads: int, num_kv_heads: int, head_dim: int,
                            intermediate_size: int, vocab_size: int, seq_len: int, num_experts: int = 0,
                            top_k: int = 0, moe_intermediate_size: int = 0, shared_intermediate_size: int = 0,
                            moe_layer_mask=None) -> float:
    D, d = hidden_size, head_dim
    attn = 2 * (D * num_heads * d + 2 * D * num_kv_heads * d + num_heads * d * D)
    dense_ffn = 3 * 2 * D * intermediate_size
    moe_ffn = 2 * (D * num_experts + top_k * 3 * D * moe_intermediate_size + 3 * D * shared_intermediate_size)
    total = 0.0
    for i in range(num_layers):
        is_moe = bool(num_experts) and (moe_layer_mask is None or moe_layer_mask[i])
        total += attn + (moe_ffn if is_moe else dense_ffn)
    matmul = 3 * (total + 2 * vocab_size * D)
    attention = num_layers * 6 * num_heads * (d + d) * seq_len
    return float(matmul + attention)
