"""Micro-benchmark of the fused compute + collective kernels against the unfused sequence (NCCL collective, then the
same tcgen05 GEMM), one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node R --master-addr 127.0.0.1 --master-port 29541 \
        -m torchllmtuner_b200.parallel.fused_bench --op ag_gemm --rows 8192 --in-cols 4096 --out-cols 3072
    ... --op gemm_rs --rows 8192 --in-cols 1536 --out-cols 4096

`rows` is the gathered row count T (each rank holds T/R), `out-cols` (N) and `in-cols` (K) are the local GEMM extents. Time: CUDA events on the
launching stream, median over `--iters`, maximum over ranks. Roofline: the slower of FLOPs / measured GEMM peak and
NVLink bytes / 770 GB/s per direction (bytes a rank must receive: (R-1)/R of the gathered or of the partial chunk set).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _median_max(fn, iters, warmup, dev):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["ag_gemm", "gemm_rs"])
    ap.add_argument("--rows", type=int, default=8192); ap.add_argument("--in-cols", type=int, default=4096); ap.add_argument("--out-cols", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=20); ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..ops.cuda_ext import check_status
    from ..ops.functional import gemm
    from ..ops.kernel_bench import _peaks
    from .symm_tp import FusedTPComm
    T, K, N = a.rows, a.in_cols, a.out_cols
    comm = FusedTPComm(dist.group.WORLD, dev, T, max(K, N))
    g = torch.Generator(device=dev).manual_seed(rank)
    if a.op == "ag_gemm":
        xs = torch.randn(T // world, K, generator=g, device=dev).bfloat16()
        w = (torch.randn(N, K, generator=g, device=dev) * 0.02).bfloat16()
        full = torch.empty(T, K, dtype=torch.bfloat16, device=dev)
        y = torch.empty(T, N, dtype=torch.bfloat16, device=dev)

        def unfused():
            dist.all_gather_into_tensor(full, xs)
            gemm(full, w, out=y)

        def fused():
            comm.ag_gemm(xs, w)
        link_bytes = (world - 1) * (T // world) * K * 2
    else:
        x = torch.randn(T, K, generator=g, device=dev).bfloat16()
        w = (torch.randn(N, K, generator=g, device=dev) * 0.02).bfloat16()
        part = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
        out = torch.empty(T // world, N, dtype=torch.bfloat16, device=dev)

        def unfused():
            gemm(x, w, out=part)
            dist.reduce_scatter_tensor(out, part)

        def fused():
            comm.gemm_rs(x, w)
        link_bytes = (world - 1) * (T // world) * N * 2

    def gemm_only():
        if a.op == "ag_gemm":
            gemm(full, w, out=y)
        else:
            gemm(x, w, out=part)
    t_gemm = _median_max(gemm_only, a.iters, a.warmup, dev)
    t_unfused = _median_max(unfused, a.iters, a.warmup, dev)
    t_fused = _median_max(fused, a.iters, a.warmup, dev)
    check_status("fused bench")
    ptf, _, src = _peaks()
    flops = 2.0 * T * N * K
    t_roof = max(flops / (ptf * 1e12), link_bytes / 770e9) * 1e3
    if rank == 0:
        print(json.dumps({"op": a.op, "ranks": world, "rows": T, "k": K, "n": N, "ms_gemm_alone": t_gemm, "ms_unfused": t_unfused,
                          "ms_fused": t_fused, "speedup_vs_unfused": t_unfused / t_fused, "ms_roofline": t_roof,
                          "frac_of_roofline": t_roof / t_fused, "peaks": src, "link_bytes_per_rank": link_bytes,
                          "tflops_fused": flops / t_fused / 1e9}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
