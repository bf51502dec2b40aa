"""MoE kernels (router top-k, permute, combine, grouped experts) vs the plain PyTorch statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=3e-2):
    a, b = a.float(), b.float()
    assert (a - b).abs().max().item() <= tol * (b.abs().max().item() + 1e-6), ((a - b).abs().max().item(), b.abs().max().item())


@pytest.mark.parametrize("T,E,k,fn,renorm,use_bias", [(300, 128, 8, "softmax", True, True), (64, 8, 2, "sigmoid", True, False),
                                                      (1000, 256, 6, "softmax", False, False), (17, 64, 4, "sigmoid", False, True)])
def test_router_topk_matches_reference(T, E, k, fn, renorm, use_bias):
    from torchllmtuner_b200.models.moe.routing import _RouterTopK
    from torchllmtuner_b200.ops import reference as ref
    torch.manual_seed(0)
    logits = torch.randn(T, E, device="cuda", requires_grad=True)
    bias = 0.1 * torch.randn(E, device="cuda") if use_bias else None
    w, idx, counts = _RouterTopK.apply(logits, bias, k, fn, renorm, 1.5)
    l2 = logits.detach().clone().requires_grad_()
    w2, idx2, counts2 = ref.router_topk(l2, bias, k, fn, renorm, 1.5)
    assert torch.equal(idx, idx2) and torch.equal(counts, counts2)
    assert (w - w2).abs().max().item() < 1e-5
    g = torch.randn_like(w)
    (d1,) = torch.autograd.grad(w, [logits], g)
    (d2,) = torch.autograd.grad(w2, [l2], g)
    assert (d1 - d2).abs().max().item() < 1e-5 * max(1.0, d2.abs().max().item())


def test_moe_block_cuda_matches_cpu_reference():
    from torchllmtuner_b200.models.moe import MoE
    torch.manual_seed(0)
    D, E, k, F_ = 256, 8, 2, 128
    cpu = MoE(D, E, k, F_, dtype=torch.float32)
    for p in cpu.parameters():
        torch.nn.init.normal_(p, std=0.05)
    gpu = MoE(D, E, k, F_, dtype=torch.bfloat16, device="cuda")
    gpu.load_state_dict({n: v.to("cuda") for n, v in cpu.state_dict().items()})
    x = torch.randn(500, D)
    xc = x.clone().requires_grad_()
    xg = x.to("cuda", torch.bfloat16).requires_grad_()
    # use the bf16-rounded weights/inputs on both sides
    with torch.no_grad():
        for pc, pg in zip(cpu.parameters(), gpu.parameters()):
            pc.copy_(pg.float().cpu())
    yc = cpu(xg.detach().float().cpu().requires_grad_() if False else xc.detach().bfloat16().float().requires_grad_())
    yg = gpu(xg)
    _close(yg, yc.to("cuda"), 5e-2)
    go = torch.randn_like(yg)
    gg = torch.autograd.grad(yg, [xg] + list(gpu.parameters()), go, allow_unused=True)
    xc2 = xc.detach().bfloat16().float().requires_grad_()
    yc2 = cpu(xc2)
    gc = torch.autograd.grad(yc2, [xc2] + list(cpu.parameters()), go.float().cpu(), allow_unused=True)
    for a, b in zip(gg, gc):
        if a is not None and b is not None:
            _close(a, b.to("cuda"), 6e-2)


@pytest.mark.parametrize("n,E,R", [(1000, 8, 2), (32768, 128, 8), (4097, 64, 4), (5, 16, 2)])
def test_ep_plan_matches_stable_sort(n, E, R):
    """Destination rows of the peer-memory dispatcher: stable position inside each expert's run plus the run's start."""
    from torchllmtuner_b200.ops.cuda_ext import load
    ext = load()
    g = torch.Generator(device="cuda").manual_seed(n + E)
    flat = torch.randint(0, E, (n,), generator=g, device="cuda")
    send_off = torch.randint(0, 1000, (E,), generator=g, device="cuda").to(torch.int32)
    drank, drow = ext.ep_plan(flat, E, R, send_off)
    counts = torch.bincount(flat, minlength=E)
    start = counts.cumsum(0) - counts
    order = torch.argsort(flat, stable=True)
    rank = torch.empty_like(order)
    rank[order] = torch.arange(n, device="cuda")
    pos = rank - start[flat]
    assert torch.equal(drow.long(), send_off.long()[flat] + pos)
    assert torch.equal(drank.long(), flat // (E // R))
