"""tcgen05 flash attention (forward, dQ, dK/dV) vs per-document fp32 softmax attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=3e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * (b.abs().max().item() + 1e-6), f"err {err}, ref scale {b.abs().max().item()}"


CASES = [
    # (cu_seqlens, Hq, Hkv, d, causal)
    ([0, 128], 2, 1, 128, True),
    ([0, 256], 4, 2, 64, True),
    ([0, 384, 512, 1000], 4, 2, 128, True),
    ([0, 77, 300, 301, 900], 8, 2, 128, True),
    ([0, 200, 520], 2, 2, 64, False),
    ([0, 1024, 2048], 8, 2, 128, True),
]


@pytest.mark.parametrize("cu,Hq,Hkv,d,causal", CASES)
def test_attention_fwd_bwd(cu, Hq, Hkv, d, causal):
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import reference as ref
    from torchllmtuner_b200.ops.cuda_ext import check_status
    torch.manual_seed(0)
    T = cu[-1]
    qkv = torch.randn(T, (Hq + 2 * Hkv) * d, device="cuda").bfloat16().requires_grad_()
    q = qkv[:, :Hq * d].view(T, Hq, d)
    k = qkv[:, Hq * d:(Hq + Hkv) * d].view(T, Hkv, d)
    v = qkv[:, (Hq + Hkv) * d:].view(T, Hkv, d)
    meta = ops.AttnMeta.build(cu, causal=causal, device="cuda")
    o = ops.attention(q, k, v, meta)
    torch.cuda.synchronize()
    check_status("attn_fwd")
    go = torch.randn_like(o)
    (g1,) = torch.autograd.grad(o, [qkv], go)
    torch.cuda.synchronize()
    check_status("attn_bwd")
    qf = qkv.detach().float().requires_grad_()
    q2 = qf[:, :Hq * d].view(T, Hq, d)
    k2 = qf[:, Hq * d:(Hq + Hkv) * d].view(T, Hkv, d)
    v2 = qf[:, (Hq + Hkv) * d:].view(T, Hkv, d)
    o2, lse2 = ref.attention(q2, k2, v2, torch.tensor(cu, dtype=torch.int32), causal)
    (g2,) = torch.autograd.grad(o2, [qf], go.float())
    _close(o, o2)
    _close(g1[:, :Hq * d], g2[:, :Hq * d])
    _close(g1[:, Hq * d:(Hq + Hkv) * d], g2[:, Hq * d:(Hq + Hkv) * d])
    _close(g1[:, (Hq + Hkv) * d:], g2[:, (Hq + Hkv) * d:])
    o3, lse3 = ops.attention_with_lse(q.detach(), k.detach(), v.detach(), meta)
    _close(lse3, lse2.to(lse3.device), 1e-2)


def test_attention_cross_lengths():
    """Keys longer than queries (context-parallel style shard): explicit q offsets."""
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import reference as ref
    torch.manual_seed(1)
    Hq, Hkv, d = 4, 2, 128
    cu_q, cu_k, offs = [0, 128, 384], [0, 512, 1024], [384, 100]
    q = torch.randn(cu_q[-1], Hq, d, device="cuda").bfloat16()
    k = torch.randn(cu_k[-1], Hkv, d, device="cuda").bfloat16()
    v = torch.randn(cu_k[-1], Hkv, d, device="cuda").bfloat16()
    meta = ops.AttnMeta.build(cu_q, cu_k, offs, causal=True, device="cuda")
    o, lse = ops.attention_with_lse(q, k, v, meta)
    o2, lse2 = ref.attention(q.float(), k.float(), v.float(), torch.tensor(cu_q), True, None, torch.tensor(cu_k), offs)
    _close(o, o2)
    _close(lse, lse2, 1e-2)
