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
    ap.add_argument("--op", required=True, choices=["gemm", "attention", "attention_bwd", "rmsnorm", "swiglu", "ce"])
    ap.add_argument("--m", type=int, default=8192); ap.add_argument("--n", type=int, default=8192); ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="tn", choices=["tn", "nn", "tt"])
    ap.add_argument("--seq", type=int, default=8192); ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8); ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=8192); ap.add_argument("--cols", type=int, default=4096)
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
    check_status(a.op)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
