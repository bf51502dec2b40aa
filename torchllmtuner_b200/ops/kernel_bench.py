"""Micro-benchmarks of the sm_100a kernels with roofline fractions.

    python -m torchllmtuner_b200.ops.kernel_bench --op gemm --m 8192 --n 8192 --k 4096 [--layout tn|nn|tt] [--iters 10]
    python -m torchllmtuner_b200.ops.kernel_bench --op attention --seq 8192 --heads 32 --kv-heads 8 --head-dim 128
    python -m torchllmtuner_b200.ops.kernel_bench --op rmsnorm --rows 8192 --cols 4096

Timing: CUDA events on the launching stream, `--warmup` untimed iterations, an L2 flush (256 MiB memset) between timed
iterations, median reported. Peaks: `--peak-tflops` / `--peak-gbs` (defaults: the measured cuBLAS bf16 burst figure and
copy bandwidth of this machine when MEASURED_PEAKS.json sits at the repository root, else 1590 TFLOP/s and 6650 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def timeit(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main() -> None:
    from .. import ops
    from .cuda_ext import check_status
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm", "attention", "attention_bwd", "rmsnorm", "swiglu", "ce", "adamw", "qk_norm_rope", "grouped_gemm", "router", "delta_rule"])
    ap.add_argument("--m", type=int, default=8192); ap.add_argument("--n", type=int, default=8192); ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="tn", choices=["tn", "nn", "tt"])
    ap.add_argument("--seq", type=int, default=8192); ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8); ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=8192); ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--chunk", type=int, default=64); ap.add_argument("--channel-decay", action="store_true"); ap.add_argument("--loop", action="store_true")
    ap.add_argument("--iters", type=int, default=10); ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--peak-tflops", type=float, default=None); ap.add_argument("--peak-gbs", type=float, default=None)
    a = ap.parse_args()
    ptf, pgb, src = _peaks()
    ptf, pgb = a.peak_tflops or ptf, a.peak_gbs or pgb
    dev = "cuda"
    out = {"op": a.op, "peaks": src}
    if a.op == "gemm":
        A = torch.randn(a.m, a.k, device=dev).bfloat16(); B = torch.randn(a.n, a.k, device=dev).bfloat16()
        if a.layout == "tn":
            fn = lambda: ops.gemm(A, B)  # noqa: E731
        elif a.layout == "nn":
            Bt = B.t().contiguous(); fn = lambda: ops.gemm(A, Bt, b_mn=True)  # noqa: E731
        else:
            At, Bt = A.t().contiguous(), B.t().contiguous(); fn = lambda: ops.gemm(At, Bt, a_mn=True, b_mn=True)  # noqa: E731
        ms = timeit(fn, a.iters, a.warmup)
        tf = 2.0 * a.m * a.n * a.k / ms / 1e9
        out.update(shape=[a.m, a.n, a.k], layout=a.layout, ms=ms, tflops=tf, frac_of_peak=tf / ptf)
    elif a.op in ("attention", "attention_bwd"):
        S, H, Hk, d = a.seq, a.heads, a.kv_heads, a.head_dim
        q = torch.randn(S, H, d, device=dev).bfloat16().requires_grad_(); k = torch.randn(S, Hk, d, device=dev).bfloat16().requires_grad_()
        v = torch.randn(S, Hk, d, device=dev).bfloat16().requires_grad_()
        meta = ops.AttnMeta.uniform(1, S, device=dev)
        fl = 4.0 * S * S * H * d / 2
        if a.op == "attention":
            ms = timeit(lambda: ops.attention(q, k, v, meta), a.iters, a.warmup)
        else:
            o = ops.attention(q, k, v, meta); go = torch.randn_like(o); fl *= 2.5
            ms = timeit(lambda: torch.autograd.grad(o, [q, k, v], go, retain_graph=True), a.iters, a.warmup)
        tf = fl / ms / 1e9
        out.update(seq=S, heads=[H, Hk], head_dim=d, ms=ms, tflops_causal=tf, frac_of_peak=tf / ptf)
    elif a.op == "delta_rule":
        # gated delta rule, forward + backward in fp32: --heads, --head-dim, --chunk; --channel-decay for a decay per key channel;
        # --loop forces the chunk-after-chunk form the scan form replaces
        import torch.nn.functional as F
        from ..models import families as fam
        S, H, d = a.seq, a.heads, a.head_dim
        g = torch.Generator(device=dev).manual_seed(0)
        x = [F.normalize(torch.randn(S, H, d, generator=g, device=dev), dim=-1).requires_grad_() for _ in range(2)]
        x += [torch.randn(S, H, d, generator=g, device=dev).requires_grad_(), torch.rand(S, H, generator=g, device=dev).requires_grad_(),
              (-F.softplus(torch.randn(S, H, d if a.channel_decay else 1, generator=g, device=dev))).requires_grad_()]
        if a.loop:
            fam.SEQUENTIAL_CHUNKS = 1 << 30

        def step():
            torch.autograd.grad(fam.chunked_delta_rule(*x, a.chunk).square().sum(), x)
        ms = timeit(step, a.iters, a.warmup)
        out.update(seq=S, heads=H, head_dim=d, chunk=a.chunk, channel_decay=a.channel_decay, form="loop" if a.loop else "scan", ms_fwd_bwd=ms)
    elif a.op == "rmsnorm":
        x = torch.randn(a.rows, a.cols, device=dev).bfloat16(); w = torch.ones(a.cols, device=dev).bfloat16()
        ms = timeit(lambda: ops.rms_norm(x, w, 1e-6), a.iters, a.warmup)
        gb = 2.0 * x.numel() * 2 / ms / 1e6
        out.update(shape=[a.rows, a.cols], ms=ms, gbs=gb, frac_of_peak=gb / pgb)
    elif a.op == "swiglu":
        g = torch.randn(a.rows, a.cols, device=dev).bfloat16(); u = torch.randn(a.rows, a.cols, device=dev).bfloat16()
        ms = timeit(lambda: ops.swiglu(g, u), a.iters, a.warmup)
        gb = 3.0 * g.numel() * 2 / ms / 1e6
        out.update(shape=[a.rows, a.cols], ms=ms, gbs=gb, frac_of_peak=gb / pgb)
    elif a.op == "ce":
        lg = torch.randn(a.rows, a.cols, device=dev).bfloat16(); y = torch.randint(0, a.cols, (a.rows,), device=dev)
        ms = timeit(lambda: ops.cross_entropy_sum(lg, y), a.iters, a.warmup)
        out.update(shape=[a.rows, a.cols], ms=ms)
    elif a.op == "adamw":
        n = a.rows * a.cols
        p32 = torch.randn(n, device=dev); p16 = p32.bfloat16(); g = torch.randn(n, device=dev).bfloat16()
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        ms = timeit(lambda: ops.adamw_step_(p32, g, m, v, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1,
                                            p_lowp=p16), a.iters, a.warmup)
        gb = n * (4 * 3 * 2 + 2 + 2) / ms / 1e6          # p32, m, v read + written; bf16 grad read; bf16 param written
        out.update(numel=n, ms=ms, gbs=gb, frac_of_peak=gb / pgb)
    elif a.op == "qk_norm_rope":
        S, H, Hk, d = a.seq, a.heads, a.kv_heads, a.head_dim
        q = torch.randn(S, H, d, device=dev).bfloat16(); k = torch.randn(S, Hk, d, device=dev).bfloat16()
        w = torch.ones(d, device=dev).bfloat16()
        ang = torch.arange(S, device=dev, dtype=torch.float32)[:, None] * (1.0 / (1e6 ** (torch.arange(0, d, 2, device=dev) / d)))[None]
        cos, sin = ang.cos(), ang.sin()
        ms = timeit(lambda: ops.qk_norm_rope(q, k, w, w, cos, sin, 1e-6), a.iters, a.warmup)
        gb = 2.0 * (q.numel() + k.numel()) * 2 / ms / 1e6
        out.update(seq=S, heads=[H, Hk], ms=ms, gbs=gb, frac_of_peak=gb / pgb)
    elif a.op == "grouped_gemm":
        from ..models.moe.experts import grouped_linear
        E, rows_per = a.heads, a.rows // a.heads // 128 * 128
        x = torch.randn(E * rows_per, a.k, device=dev).bfloat16(); w = (torch.randn(E, a.n, a.k, device=dev) * 0.02).bfloat16()
        seg = (torch.arange(E + 1, device=dev) * rows_per).to(torch.int32)
        ms = timeit(lambda: grouped_linear(x, w, seg), a.iters, a.warmup)
        tf = 2.0 * E * rows_per * a.n * a.k / ms / 1e9
        out.update(experts=E, rows_per_expert=rows_per, n=a.n, k=a.k, ms=ms, tflops=tf, frac_of_peak=tf / ptf)
    elif a.op == "router":
        from .cuda_ext import load
        logits = torch.randn(a.rows, a.cols, device=dev)
        ext = load()
        ms = timeit(lambda: ext.router_topk(logits, None, 8, 0, True, 1.0), a.iters, a.warmup)
        out.update(shape=[a.rows, a.cols], k=8, ms=ms, gbs=logits.numel() * 4 / ms / 1e6)
    check_status(a.op)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
