"""Workers for the peer-memory expert-parallel dispatcher tests (one process per GPU)."""
import json
import os
import sys

import torch


def _worker(rank: int, world: int, port: int, out_path: str, iters: int, overflow: bool = False, skew: bool = False):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from torchllmtuner_b200.models.moe.experts import GroupedExperts
    from torchllmtuner_b200.ops.cuda_ext import check_status
    from torchllmtuner_b200.parallel.expert_parallel import AllToAllTokenDispatcher
    from torchllmtuner_b200.parallel.symm_ep import PeerTokenDispatcher
    E, k, T, D, F = 8 * world, 4, 384, 256, 128
    nccl = AllToAllTokenDispatcher(E, dist.group.WORLD, world, rank)
    peer = PeerTokenDispatcher(E, dist.group.WORLD, world, rank, fallback=nccl, capacity_factor=1.0 if overflow else (None if skew else 3.0))
    torch.manual_seed(7)
    experts = GroupedExperts(E // world, D, F, dtype=torch.bfloat16, device=dev)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    with torch.no_grad():
        for p in experts.parameters():
            p.copy_((torch.randn(p.shape, generator=g, device=dev) * 0.05).to(p.dtype))
    worst = {"out": 0.0, "dx": 0.0, "dw": 0.0, "dparam": 0.0}

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))

    for it in range(iters):
        x0 = (torch.randn(T, D, generator=g, device=dev) * 0.5).bfloat16()
        scores = torch.rand(T, E, generator=g, device=dev)
        if it == 1:
            scores[:, : E // 2] += 0.2           # unbalanced routing that still fits the receive buffers
        if overflow or skew:
            scores[:, : E // world] += 10.0      # every copy goes to rank 0 (overflows unless the buffers are worst-case sized)
        w0, idx = scores.topk(k, dim=-1)
        w0 = (w0 / w0.sum(-1, keepdim=True)).float()
        dout = (torch.randn(T, D, generator=g, device=dev) * 0.1).bfloat16()
        res = []
        for disp in (nccl, peer):
            x, w = x0.clone().requires_grad_(), w0.clone().requires_grad_()
            for p in experts.parameters():
                p.grad = None
            rows, seg, st = disp.dispatch(x, idx)
            y = experts(rows, seg)
            out = disp.combine(y, w, st)
            out.backward(dout)
            res.append((out.detach(), x.grad, w.grad, [p.grad.clone() for p in experts.parameters()]))
        (o0, dx0, dw0, dp0), (o1, dx1, dw1, dp1) = res
        worst["out"] = max(worst["out"], rel(o1, o0))
        worst["dx"] = max(worst["dx"], rel(dx1, dx0))
        worst["dw"] = max(worst["dw"], rel(dw1, dw0))
        worst["dparam"] = max(worst["dparam"], max(rel(a, b) for a, b in zip(dp1, dp0)))
        if it % 2 == rank % 2:
            torch.cuda._sleep(20_000_000)
    torch.cuda.synchronize()
    if overflow:
        from torchllmtuner_b200.errors import KernelStatusError
        try:
            check_status("fused ep overflow test")
            seen = 0.0
        except KernelStatusError as e:
            seen = 1.0 if "capacity overflow" in str(e) else 0.0
        # the context is still usable: a small GEMM runs and the status word is clean again
        from torchllmtuner_b200.ops.functional import gemm
        a = torch.randn(128, 64, device=dev).bfloat16()
        gemm(a, a)
        check_status("after overflow")
        t = torch.tensor([seen], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            with open(out_path, "w") as f:
                json.dump({"overflow_seen": float(t)}, f)
        dist.barrier()
        dist.destroy_process_group()
        return
    check_status("fused ep test")
    ex = next(iter(__import__("torchllmtuner_b200.parallel.symm_ep", fromlist=["_EXCHANGES"])._EXCHANGES.values()))
    assert ex.check_canaries(), "a kernel wrote past a buffer of the symmetric arena"
    t = torch.tensor([worst[k_] for k_ in sorted(worst)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({**dict(zip(sorted(worst), t.tolist())), "stats": peer.exchange.stats if peer.exchange else
                       next(iter(__import__("torchllmtuner_b200.parallel.symm_ep", fromlist=["_EXCHANGES"])._EXCHANGES.values())).stats}, f)
    dist.barrier()
    dist.destroy_process_group()


def run_fused_ep(world: int, iters: int = 4, overflow: bool = False, skew: bool = False) -> dict:
    import tempfile

    import torch.multiprocessing as mp
    out = tempfile.mktemp(suffix=".json")
    port = 22000 + (os.getpid() * 17 + world) % 20000
    mp.spawn(_worker, args=(world, port, out, iters, overflow, skew), nprocs=world, join=True)
    with open(out) as f:
        res = json.load(f)
    os.unlink(out)
    return res
