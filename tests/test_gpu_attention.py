"""tcgen05 flash attention (forward, dQ, dK/dV) vs per-document fp32 softmax attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


from tolerances import ATTENTION, ATTENTION_GRAD, assert_close


def _close(a, b, name="o"):
    assert_close(a, b, name=name, **(ATTENTION_GRAD if name.startswith("d") else ATTENTION))


def _close_lse(a, b):
    assert_close(a, b, rtol=1e-3, atol_rms=1e-3, name="lse")


CASES = [
    # (cu_seqlens, Hq, Hkv, d, causal)
    ([0, 128], 2, 1, 128, True),
    ([0, 256], 4, 2, 64, True),
    ([0, 384, 512, 1000], 4, 2, 128, True),
    ([0, 77, 300, 301, 900], 8, 2, 128, True),
    ([0, 200, 520], 2, 2, 64, False),
    ([0, 1024, 2048], 8, 2, 128, True),
]


@pytest.fixture(autouse=True)
def _default_backward():
    from torchllmtuner_b200.ops import functional as F
    yield
    F.set_attention_backward(None)


@pytest.mark.parametrize("mode", ["fused", "split"])
@pytest.mark.parametrize("cu,Hq,Hkv,d,causal", CASES)
def test_attention_fwd_bwd(cu, Hq, Hkv, d, causal, mode):
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import functional as F
    from torchllmtuner_b200.ops import reference as ref
    from torchllmtuner_b200.ops.cuda_ext import check_status
    F.set_attention_backward(mode)
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
    _close(o, o2, "o")
    _close(g1[:, :Hq * d], g2[:, :Hq * d], "dq")
    _close(g1[:, Hq * d:(Hq + Hkv) * d], g2[:, Hq * d:(Hq + Hkv) * d], "dk")
    _close(g1[:, (Hq + Hkv) * d:], g2[:, (Hq + Hkv) * d:], "dv")
    o3, lse3 = ops.attention_with_lse(q.detach(), k.detach(), v.detach(), meta)
    _close_lse(lse3, lse2.to(lse3.device))


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
    _close_lse(lse, lse2.to(lse.device))


def _packed_lengths(total, lo=512, hi=32768, seed=0):
    """Document lengths drawn log-uniform in [lo, hi] until `total` tokens are filled (the last one is cut)."""
    import math
    import random
    rng = random.Random(seed)
    cu = [0]
    while cu[-1] < total:
        n = int(round(math.exp(rng.uniform(math.log(lo), math.log(hi)))))
        cu.append(min(total, cu[-1] + n))
    return cu


@pytest.mark.parametrize("mode", ["fused", "split"])
def test_attention_bench_shape_packed(mode):
    """The benchmark shape: 8192 packed tokens, 32 query / 8 key-value heads of 128, documents log-uniform 512..32768."""
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import functional as F
    from torchllmtuner_b200.ops import reference as ref
    from torchllmtuner_b200.ops.cuda_ext import check_status
    F.set_attention_backward(mode)
    torch.manual_seed(3)
    Hq, Hkv, d = 32, 8, 128
    cu = _packed_lengths(8192, lo=512, hi=4096, seed=1)     # several documents inside the 8192-token row
    T = cu[-1]
    q = (torch.randn(T, Hq, d, device="cuda")).bfloat16().requires_grad_()
    k = (torch.randn(T, Hkv, d, device="cuda")).bfloat16().requires_grad_()
    v = (torch.randn(T, Hkv, d, device="cuda")).bfloat16().requires_grad_()
    meta = ops.AttnMeta.build(cu, causal=True, device="cuda")
    o = ops.attention(q, k, v, meta)
    go = torch.randn_like(o)
    dq, dk, dv = torch.autograd.grad(o, [q, k, v], go)
    torch.cuda.synchronize()
    check_status("attention bench shape")
    # fp32 statement one document at a time (the full 8192 x 8192 x 32 score tensor would not be a small reference)
    for a, b in zip(cu[:-1], cu[1:]):
        qf, kf, vf = (t.detach()[a:b].float().requires_grad_() for t in (q, k, v))
        o2, _ = ref.attention(qf, kf, vf, torch.tensor([0, b - a], dtype=torch.int32), True)
        g2 = torch.autograd.grad(o2, [qf, kf, vf], go[a:b].float())
        _close(o[a:b], o2, f"o[{a}:{b}]")
        for name, mine, theirs in zip(("dq", "dk", "dv"), (dq, dk, dv), g2):
            _close(mine[a:b], theirs, f"{name}[{a}:{b}]")


def test_attention_backward_modes_agree_on_dk_dv():
    """Both backward forms compute dK and dV from the same rounded P and dS, so those two agree bit for bit."""
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import functional as F
    torch.manual_seed(5)
    q = torch.randn(1000, 8, 128, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(1000, 2, 128, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(1000, 2, 128, device="cuda").bfloat16().requires_grad_()
    meta = ops.AttnMeta.build([0, 300, 1000], causal=True, device="cuda")
    o = ops.attention(q, k, v, meta)
    go = torch.randn_like(o)
    res = {}
    for mode in ("fused", "split"):
        F.set_attention_backward(mode)
        res[mode] = torch.autograd.grad(o, [q, k, v], go, retain_graph=True)
    assert torch.equal(res["fused"][2], res["split"][2])
    _close(res["fused"][0], res["split"][0].float(), "dq fused vs split")
    _close(res["fused"][1], res["split"][1].float(), "dk fused vs split")


@pytest.mark.parametrize("cu,Hq,Hkv,causal", [([0, 128], 2, 1, True), ([0, 77, 300, 301, 900], 8, 2, True),
                                                ([0, 200, 520], 2, 2, False), ([0, 1024, 2048], 8, 2, True)])
def test_attention_head_size_256(cu, Hq, Hkv, causal):
    """Head size 256: forward kernel (a 16-slice K loop for S, one N=256 product for P V, 384 TMEM columns), backward
    rebuilt per chunk of query rows from the saved log-sum-exp."""
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import reference as ref
    from torchllmtuner_b200.ops.cuda_ext import check_status
    d = 256
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
    qf = qkv.detach().float().requires_grad_()
    q2 = qf[:, :Hq * d].view(T, Hq, d)
    k2 = qf[:, Hq * d:(Hq + Hkv) * d].view(T, Hkv, d)
    v2 = qf[:, (Hq + Hkv) * d:].view(T, Hkv, d)
    o2, lse2 = ref.attention(q2, k2, v2, torch.tensor(cu, dtype=torch.int32), causal)
    (g2,) = torch.autograd.grad(o2, [qf], go.float())
    _close(o, o2, "o")
    _close(g1[:, :Hq * d], g2[:, :Hq * d], "dq")
    _close(g1[:, Hq * d:(Hq + Hkv) * d], g2[:, Hq * d:(Hq + Hkv) * d], "dk")
    _close(g1[:, (Hq + Hkv) * d:], g2[:, (Hq + Hkv) * d:], "dv")
    _, lse3 = ops.attention_with_lse(q.detach(), k.detach(), v.detach(), meta)
    _close_lse(lse3, lse2.to(lse3.device))


@pytest.mark.parametrize("causal,diag", [(True, 100), (True, -3), (False, 0)])
def test_attention_rows_kernels_match_the_tensor_expressions(causal, diag):
    """The one-pass P and dS kernels of the row-chunked backward against the same algebra in fp32 tensor expressions,
    with an odd column count, rows that see no key (lse = -inf) and a diagonal that starts before column 0."""
    from torchllmtuner_b200.ops import reference as ref
    from torchllmtuner_b200.ops.cuda_ext import load
    ext = load()
    torch.manual_seed(0)
    B, g, n, C = 3, 2, 37, 301
    s = torch.randn(B, g * n, C, device="cuda") * 3
    lse = torch.logsumexp(s * 0.25, -1) + 0.5
    if causal and diag < 0:
        lse[:, :3] = float("-inf")
        lse[:, n:n + 3] = float("-inf")
    p = ext.attn_rows_probs(s.clone(), lse.contiguous(), n, diag, 0.25, causal)
    want = ref._rows_probs(s.clone(), lse, n, diag, 0.25, causal, torch.float32)
    assert p.dtype == torch.bfloat16 and torch.isfinite(p.float()).all()
    assert_close(p.float(), want, rtol=2 ** -7, atol_rms=1e-3, name="p")
    dp = torch.randn(B, g * n, C, device="cuda") * 4
    dl = torch.randn(B, g * n, device="cuda")
    ds = ext.attn_rows_ds(dp.clone(), p, dl)
    assert_close(ds.float(), (dp - dl.unsqueeze(-1)) * p.float(), rtol=2 ** -7, atol_rms=1e-3, name="ds")


@pytest.mark.parametrize("d,dv,causal", [(72, 72, False), (192, 128, True), (40, 64, True)])
def test_attention_pads_widths_without_a_kernel_variant(d, dv, causal):
    """Head widths between the kernel variants (a vision tower's 72, latent attention's 192 keys / 128 values) run zero-padded
    to the next variant; outputs and gradients equal the fp32 statement at the true widths."""
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.ops import reference as ref
    torch.manual_seed(0)
    cu, Hq, Hkv = [0, 150, 400], 4, 2
    T = cu[-1]
    q = torch.randn(T, Hq, d, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(T, Hkv, d, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(T, Hkv, dv, device="cuda").bfloat16().requires_grad_()
    meta = ops.AttnMeta.build(cu, causal=causal, device="cuda")
    scale = d ** -0.5
    o = ops.attention(q, k, v, meta, scale)
    assert o.shape == (T, Hq, dv)
    go = torch.randn_like(o)
    g1 = torch.autograd.grad(o, [q, k, v], go)
    q2, k2, v2 = (t.detach().float().requires_grad_() for t in (q, k, v))
    o2, _ = ref.attention_pieces(q2, k2, v2, meta.pieces, causal, scale)
    g2 = torch.autograd.grad(o2, [q2, k2, v2], go.float())
    _close(o, o2, "o")
    for a, b, n in zip(g1, g2, ("dq", "dk", "dv")):
        assert a.shape == b.shape
        _close(a, b, n)
