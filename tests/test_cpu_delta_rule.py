"""Chunk-parallel gated delta rule against its token-by-token statement: values, gradients, documents, strong decay."""
import pytest
import torch
import torch.nn.functional as F

from torchllmtuner_b200.models.families import DeltaRuleMixer, HybridConfig, chunked_delta_rule, delta_rule_scan
from torchllmtuner_b200.models.qwen3 import ForwardContext
from torchllmtuner_b200.ops.attn_meta import AttnMeta


def _inputs(T, H, dk, dv, channels, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = F.normalize(torch.randn(T, H, dk, generator=g), dim=-1).requires_grad_()
    k = F.normalize(torch.randn(T, H, dk, generator=g), dim=-1).requires_grad_()
    v = torch.randn(T, H, dv, generator=g).requires_grad_()
    beta = torch.rand(T, H, generator=g).requires_grad_()
    ld = (-F.softplus(torch.randn(T, H, channels, generator=g) * 3)).requires_grad_()
    return [q, k, v, beta, ld]


@pytest.mark.parametrize("channels,T,chunk", [(1, 37, 8), (8, 37, 8), (1, 64, 16), (8, 50, 16), (8, 16, 16), (1, 5, 64),
                                              (1, 150, 8), (8, 200, 16), (8, 128, 8), (1, 72, 8)])      # the last four: more chunks than the loop form takes
def test_chunked_form_matches_the_scan(channels, T, chunk):
    x = _inputs(T, 3, 8, 6, channels)
    a, b = delta_rule_scan(*x), chunked_delta_rule(*x, chunk)
    assert torch.allclose(a, b, atol=5e-6)
    w = torch.randn_like(a)
    for ga, gb in zip(torch.autograd.grad((a * w).sum(), x), torch.autograd.grad((b * w).sum(), x)):
        assert torch.allclose(ga, gb, atol=5e-5)


def test_strong_decay_stays_finite_and_forgets():
    T = 40
    q, k, v, beta, _ = (t.detach() for t in _inputs(T, 2, 4, 4, 4))
    o = chunked_delta_rule(q, k, v, beta, torch.full((T, 2, 4), -200.0), 16)
    assert torch.isfinite(o).all()
    # with the state wiped at every step, o_t = beta_t (k_t . q_t) v_t
    want = beta.unsqueeze(-1) * (k * q).sum(-1, keepdim=True) * v
    assert torch.allclose(o, want, atol=1e-6)


@pytest.mark.parametrize("channel", [False, True])
def test_mixer_resets_its_state_at_document_starts(channel):
    cfg = HybridConfig(vocab_size=32, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16, delta_heads=2, delta_head_dim=8, delta_channel_decay=channel,
                       delta_chunk_size=8)
    torch.manual_seed(0)
    m = DeltaRuleMixer(cfg)
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.3) if p.dim() > 1 else torch.nn.init.ones_(p)
    x = torch.randn(30, 32)

    def run(rows, cu):
        meta = AttnMeta.build(torch.tensor(cu))
        return m(rows, ForwardContext(None, None, meta))
    both = run(x, [0, 13, 30])
    assert torch.allclose(both[:13], run(x[:13], [0, 13]), atol=1e-5)
    assert torch.allclose(both[13:], run(x[13:], [0, 17]), atol=1e-5)
    assert not torch.allclose(both[13:], run(x, [0, 30])[13:], atol=1e-3)


def _kcp_worker(rank, world, store_path, out_path):
    import torch.distributed as dist
    from torchllmtuner_b200.parallel.context_parallel import ContextParallelDriver
    dist.init_process_group("gloo", store=dist.FileStore(store_path, world), rank=rank, world_size=world)
    try:
        class Topo:
            cp_ulysses, cp_kv, cp = 1, 1, world
            def get_group(self, name): return None
            def coord(self, name): return rank

        class Cfg:
            context_parallel_load_balancer = None
        B, S, H, dk, dv = 2, 24, 2, 4, 4
        # documents: one crosses the rank boundary, one starts inside a span, one starts exactly at a boundary
        cu = {2: [0, 5, 24, 36, 48], 3: [0, 5, 24, 32, 48]}[world]
        res = {}
        for channels in (1, dk):
            x = _inputs(B * S, H, dk, dv, channels, seed=3)
            t = S // world
            rows = torch.cat([torch.arange(b * S + rank * t, b * S + (rank + 1) * t) for b in range(B)])
            local = [a.detach()[rows].clone().requires_grad_() for a in x]
            drv = ContextParallelDriver(Topo(), Cfg())
            drv._mb = {"B": B, "S": S, "gcu": cu}
            o = drv.delta_rule(*local, chunk=4)
            w = torch.randn(B * S, H, dv, generator=torch.Generator().manual_seed(9))
            (o * w[rows]).sum().backward()
            res[channels] = (rows, o.detach(), [a.grad for a in local])
        torch.save(res, f"{out_path}.{rank}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_delta_rule_hands_the_state_across_ranks(tmp_path, world):
    import torch.multiprocessing as mp
    out = str(tmp_path / "o")
    mp.spawn(_kcp_worker, args=(world, str(tmp_path / "store"), out), nprocs=world, join=True)
    B, S, H, dk, dv = 2, 24, 2, 4, 4
    cu = {2: [0, 5, 24, 36, 48], 3: [0, 5, 24, 32, 48]}[world]
    parts = [torch.load(f"{out}.{r}", weights_only=False) for r in range(world)]
    for channels in (1, dk):
        x = _inputs(B * S, H, dk, dv, channels, seed=3)
        want = torch.cat([delta_rule_scan(*(a[lo:hi] for a in x)) for lo, hi in zip(cu[:-1], cu[1:])])
        w = torch.randn(B * S, H, dv, generator=torch.Generator().manual_seed(9))
        grads = torch.autograd.grad((want * w).sum(), x)
        for rows, o, g in (p[channels] for p in parts):
            assert torch.allclose(o, want[rows], atol=1e-5)
            for got, full in zip(g, grads):
                assert torch.allclose(got, full[rows], atol=1e-4)


@pytest.mark.parametrize("N", [1, 2, 9, 10, 16, 23])
def test_affine_scan_matches_the_step_by_step_recurrence(N):
    from torchllmtuner_b200.models.families import affine_scan
    torch.manual_seed(N)
    A = (torch.randn(N, 2, 5, 5, dtype=torch.float64) * 0.4).requires_grad_()
    B = torch.randn(N, 2, 5, 3, dtype=torch.float64, requires_grad=True)
    S0 = torch.randn(2, 5, 3, dtype=torch.float64, requires_grad=True)

    def plain(A, B, S):
        out = []
        for n in range(N):
            out.append(S)
            S = A[n] @ S + B[n]
        return torch.stack(out), S
    got, want = affine_scan(A, B, S0), plain(A, B, S0)
    assert torch.allclose(got[0], want[0], atol=1e-12) and torch.allclose(got[1], want[1], atol=1e-12)
    w0, w1 = torch.randn_like(want[0]), torch.randn_like(want[1])
    for ga, gb in zip(torch.autograd.grad((got[0] * w0).sum() + (got[1] * w1).sum(), [A, B, S0]),
                      torch.autograd.grad((want[0] * w0).sum() + (want[1] * w1).sum(), [A, B, S0])):
        assert torch.allclose(ga, gb, atol=1e-11)


def test_long_sequences_carry_and_return_state_like_short_ones():
    """The scan form (many chunks) and the loop form (few chunks) agree when a sequence is processed in two halves with
    the state handed over, for both decay forms."""
    for channels in (1, 8):
        q, k, v, beta, ld = (t.detach() for t in _inputs(160, 2, 8, 6, channels, seed=3))
        whole, s_whole = chunked_delta_rule(q, k, v, beta, ld, 8, None, True)                       # 20 chunks: scan form
        a, s_a = chunked_delta_rule(q[:40], k[:40], v[:40], beta[:40], ld[:40], 8, None, True)       # 5 chunks: loop form
        b, s_b = chunked_delta_rule(q[40:], k[40:], v[40:], beta[40:], ld[40:], 8, s_a, True)        # 15 chunks: scan form from a state
        assert torch.allclose(torch.cat((a, b)), whole, atol=2e-5) and torch.allclose(s_b, s_whole, atol=2e-5)
        assert torch.allclose(whole, delta_rule_scan(q, k, v, beta, ld), atol=2e-5)


def test_scan_blocks_carry_the_state(monkeypatch):
    """With a tiny block budget the scan runs as several blocks of chunks; values and gradients do not change."""
    from torchllmtuner_b200.models import families as fam
    x = _inputs(200, 2, 8, 6, 8, seed=5)
    want = chunked_delta_rule(*x, 8)
    gw = torch.autograd.grad(want.square().sum(), x)
    monkeypatch.setattr(fam, "SCAN_BLOCK_BYTES", 1)            # -> blocks of SEQUENTIAL_CHUNKS + 1 = 9 chunks, 25 chunks in all
    got = chunked_delta_rule(*x, 8)
    assert torch.allclose(got, want, atol=1e-6)
    for a, b in zip(torch.autograd.grad(got.square().sum(), x), gw):
        assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("channels", [1, 8])
def test_against_the_flash_linear_attention_reference_recurrences(channels):
    """An independent statement of both recurrences: the plain-PyTorch references of the `fla` package (the library the
    reference framework calls for these mixers). One decay per head is its gated delta rule, one per key channel its KDA.
    The long sequence takes the scan form, the short one the loop form; an initial state and the final state agree too."""
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        naive_kda = pytest.importorskip("fla.ops.kda.naive").naive_recurrent_kda
        naive_gdn = pytest.importorskip("fla.ops.gated_delta_rule.naive").naive_recurrent_gated_delta_rule
    for T, chunk in ((150, 8), (40, 16)):
        q, k, v, beta, ld = (t.detach() for t in _inputs(T, 3, 8, 6, channels, seed=T))
        s0 = torch.randn(3, 8, 6) * 0.3
        got, s_got = chunked_delta_rule(q, k, v, beta, ld, chunk, s0, True)
        if channels == 1:
            want, s_want = naive_gdn(q[None], k[None], v[None], beta[None], ld[None, ..., 0], scale=1.0, initial_state=s0[None],
                                     output_final_state=True)
        else:
            want, s_want = naive_kda(q[None], k[None], v[None], ld[None], beta[None], scale=1.0, initial_state=s0[None],
                                     output_final_state=True)
        assert torch.allclose(got, want[0].float(), atol=2e-5), (got - want[0]).abs().max()
        assert torch.allclose(s_got, s_want[0].float(), atol=2e-5)
