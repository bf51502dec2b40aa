"""tcgen05 GEMM vs a plain fp32 PyTorch product, all operand layouts, edge shapes, grouped forms."""
import pytest
import torch

pytestmark = pytest.mark.gpu


from tolerances import GEMM_BF16, GEMM_F32, assert_close


def _close(out, ref, name="gemm"):
    assert_close(out, ref, name=name, **(GEMM_F32 if out.dtype == torch.float32 else GEMM_BF16))


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 320), (200, 136, 72), (1024, 4096, 1024), (64, 64, 64), (136, 520, 200),
          (2048, 128, 512)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("layout", ["tn", "nn", "tt"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_layouts(M, N, K, layout, out_dtype):
    from torchllmtuner_b200.ops import gemm
    from torchllmtuner_b200.ops.cuda_ext import check_status
    torch.manual_seed(0)
    dev = "cuda"
    A = torch.randn(M, K, device=dev).bfloat16()
    B = torch.randn(N, K, device=dev).bfloat16()
    ref = A.float() @ B.float().t()
    if layout == "tn":
        out = gemm(A, B, out_dtype=out_dtype)
    elif layout == "nn":   # B stored [K, N]
        out = gemm(A, B.t().contiguous(), b_mn=True, out_dtype=out_dtype)
    else:                  # A stored [K, M], B stored [K, N]
        out = gemm(A.t().contiguous(), B.t().contiguous(), a_mn=True, b_mn=True, out_dtype=out_dtype)
    torch.cuda.synchronize()
    check_status("gemm")
    _close(out, ref)


@pytest.mark.parametrize("M,N,K,layout", [(1024, 151936, 4096, "tn"), (8192, 4096, 12288, "tn"), (4096, 12288, 8192, "tt"), (8192, 4096, 4096, "nn")])
def test_gemm_benchmark_shapes(M, N, K, layout):
    """Shapes of the Qwen3-8B step: vocabulary head (N = 151,936), down projection (K = 12,288), its weight gradient
    (reduction over 8192 tokens) and an input gradient."""
    from torchllmtuner_b200.ops import gemm
    from torchllmtuner_b200.ops.cuda_ext import check_status
    torch.manual_seed(0)
    A = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    B = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    if layout == "tn":
        out = gemm(A, B)
    elif layout == "nn":
        out = gemm(A, B.t().contiguous(), b_mn=True)
    else:
        out = gemm(A.t().contiguous(), B.t().contiguous(), a_mn=True, b_mn=True)
    torch.cuda.synchronize()
    check_status("gemm")
    for r0 in range(0, M, 1024):       # reference in row blocks to bound the fp32 temporaries
        _close(out[r0:r0 + 1024], A[r0:r0 + 1024].float() @ B.float().t(), f"rows {r0}")


def test_gemm_accumulate_and_strided_out():
    from torchllmtuner_b200.ops import gemm
    from torchllmtuner_b200.ops.cuda_ext import check_status
    torch.manual_seed(1)
    M, N, K = 256, 384, 512
    A = torch.randn(K, M, device="cuda").bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    ref = acc + A.float().t() @ B.float()
    gemm(A, B, a_mn=True, b_mn=True, out=acc, accumulate=True)
    check_status("gemm")
    _close(acc, ref)
    big = torch.zeros(M, 2 * N, device="cuda", dtype=torch.bfloat16)
    gemm(A, B, a_mn=True, b_mn=True, out=big[:, N:])
    check_status("gemm")
    _close(big[:, N:], A.float().t() @ B.float())
    assert big[:, :N].abs().max().item() == 0


def test_gemm_determinism():
    from torchllmtuner_b200.ops import gemm
    A = torch.randn(512, 1024, device="cuda").bfloat16()
    B = torch.randn(768, 1024, device="cuda").bfloat16()
    assert torch.equal(gemm(A, B), gemm(A, B))


def _segments(counts):
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + -(-c // 128) * 128)
    return offs


@pytest.mark.parametrize("counts", [[128, 256, 0, 130, 5], [700, 1, 0, 0, 300, 128]])
def test_grouped_gemm_and_wgrad(counts):
    from torchllmtuner_b200.ops.cuda_ext import check_status, load
    ext = load()
    torch.manual_seed(2)
    G, K, N = len(counts), 256, 384
    offs = _segments(counts)
    rows = offs[-1]
    x = torch.zeros(rows, K, device="cuda", dtype=torch.bfloat16)
    for g, c in enumerate(counts):
        x[offs[g]:offs[g] + c] = torch.randn(c, K, device="cuda").bfloat16()
    w = torch.randn(G, N, K, device="cuda").bfloat16() * 0.1
    seg = torch.tensor(offs, dtype=torch.int32, device="cuda")
    y = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    ext.grouped_gemm(x, w, y, seg, False)
    check_status("grouped_gemm")
    for g, c in enumerate(counts):
        if c:
            _close(y[offs[g]:offs[g] + c], x[offs[g]:offs[g] + c].float() @ w[g].float().t())
    # dgrad form: y2 = dy @ w  (w stored [G, N, K] read as [G, K'=N, N'=K])
    dy = torch.zeros(rows, N, device="cuda", dtype=torch.bfloat16)
    for g, c in enumerate(counts):
        dy[offs[g]:offs[g] + c] = torch.randn(c, N, device="cuda").bfloat16()
    dx = torch.empty(rows, K, device="cuda", dtype=torch.bfloat16)
    ext.grouped_gemm(dy, w, dx, seg, True)
    check_status("grouped_dgrad")
    for g, c in enumerate(counts):
        if c:
            _close(dx[offs[g]:offs[g] + c], dy[offs[g]:offs[g] + c].float() @ w[g].float())
    dw = torch.empty(G, N, K, device="cuda", dtype=torch.float32)
    ext.grouped_wgrad(dy, x, dw, seg, False)
    check_status("grouped_wgrad")
    for g, c in enumerate(counts):
        ref = dy[offs[g]:offs[g] + c].float().t() @ x[offs[g]:offs[g] + c].float()
        if c:
            _close(dw[g], ref)
        else:
            assert dw[g].abs().max().item() == 0


def test_bounded_wait_expires_into_status_word():
    """A flag that nothing sets: the wait gives up after its poll limit, the kernel returns, the host reads the
    status and the context stays usable."""
    from torchllmtuner_b200.ops.cuda_ext import KernelStatusError, check_status, load
    ext = load()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    ext.wait_flags(flags.data_ptr(), 4, 1, 9100, 1 << 14)
    with pytest.raises(KernelStatusError) as e:
        check_status("bounded wait test")
    assert "9100" in str(e.value) or "910" in str(e.value)
    # the status word was cleared by the read and the device still works
    a = torch.randn(256, 128, device="cuda").bfloat16()
    b = torch.randn(256, 128, device="cuda").bfloat16()
    out = torch.empty(256, 256, device="cuda", dtype=torch.bfloat16)
    ext.gemm(a, b, out, False, False, False, 0)
    check_status("after recovery")
    assert torch.allclose(out.float(), a.float() @ b.float().t(), atol=0.5, rtol=5e-2)


def test_projections_of_the_same_rows_sum_their_input_gradient_in_the_epilogue():
    """`ops.linears(x, W0, W1, W2)`: the same outputs as three `ops.linear` calls; dx is accumulated by the second and third
    GEMM's epilogue instead of by elementwise additions, so it may differ from the separate form by one bf16 rounding."""
    from torchllmtuner_b200 import ops
    torch.manual_seed(0)
    x = (torch.randn(1024, 512, device="cuda") * 0.5).bfloat16().requires_grad_()
    ws = [(torch.randn(n, 512, device="cuda") * 0.05).bfloat16().requires_grad_() for n in (512, 128, 256)]
    gs = [torch.randn(1024, n, device="cuda").bfloat16() for n in (512, 128, 256)]
    ys = ops.linears(x, *ws)
    torch.autograd.backward(ys, gs)
    got = [x.grad.clone()] + [w.grad.clone() for w in ws]
    x.grad = None
    for w in ws:
        w.grad = None
    ys2 = [ops.linear(x, w) for w in ws]
    for a, b in zip(ys, ys2):
        assert torch.equal(a, b)
    torch.autograd.backward(ys2, gs)
    ref_dx = sum(g.float() @ w.float() for g, w in zip(gs, ws))
    assert (got[0].float() - ref_dx).abs().max() <= 0.02 * ref_dx.abs().max()
    assert (got[0].float() - x.grad.float()).abs().max() <= 0.02 * ref_dx.abs().max()
    for a, w in zip(got[1:], ws):
        assert torch.equal(a, w.grad)
