"""Workers for the fused tensor-parallel GEMM tests (one process per GPU, NCCL only for the reference collectives)."""
import json
import os
import sys

import torch


def _worker(rank: int, world: int, port: int, out_path: str, iters: int):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from torchllmtuner_b200.ops.cuda_ext import check_status
    from torchllmtuner_b200.parallel.symm_tp import FusedTPComm, GatherLinears, LinearReduceScatter
    T, D, N1, N2, Kl = 256 * world, 512, 384, 136, 320
    comm = FusedTPComm(dist.group.WORLD, dev, T, D)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    res = {"ag": 0.0, "rs": 0.0, "ag_bwd": 0.0, "rs_bwd": 0.0}

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))

    for it in range(iters):
        xs = (torch.randn(T // world, D, generator=g, device=dev) * 0.5).bfloat16().requires_grad_()
        w1 = (torch.randn(N1, D, generator=g, device=dev) * 0.05).bfloat16().requires_grad_()
        w2 = (torch.randn(N2, D, generator=g, device=dev) * 0.05).bfloat16().requires_grad_()
        # reference: NCCL gather + fp32 matmuls
        full = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(full, xs.detach())
        y1, y2 = GatherLinears.apply(comm, xs, w1, w2)
        r1, r2 = full.float() @ w1.float().t(), full.float() @ w2.float().t()
        res["ag"] = max(res["ag"], rel(y1, r1), rel(y2, r2))
        d1 = (torch.randn(T, N1, generator=g, device=dev) * 0.1).bfloat16()
        d2 = (torch.randn(T, N2, generator=g, device=dev) * 0.1).bfloat16()
        torch.autograd.backward([y1, y2], [d1, d2])
        dfull = d1.float() @ w1.float() + d2.float() @ w2.float()
        dref = torch.empty(T // world, D, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(dref, dfull)
        res["ag_bwd"] = max(res["ag_bwd"], rel(xs.grad, dref), rel(w1.grad, d1.float().t() @ full.float()))
        # row-parallel form
        a = (torch.randn(T, Kl, generator=g, device=dev) * 0.5).bfloat16().requires_grad_()
        w = (torch.randn(D, Kl, generator=g, device=dev) * 0.05).bfloat16().requires_grad_()
        out = LinearReduceScatter.apply(comm, a, w)
        pref = a.float() @ w.float().t()
        oref = torch.empty(T // world, D, dtype=torch.float32, device=dev)
        dist.reduce_scatter_tensor(oref, pref)
        res["rs"] = max(res["rs"], rel(out, oref))
        dy = (torch.randn(T // world, D, generator=g, device=dev) * 0.1).bfloat16()
        out.backward(dy)
        dyf = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(dyf, dy)
        res["rs_bwd"] = max(res["rs_bwd"], rel(a.grad, dyf.float() @ w.float()), rel(w.grad, dyf.float().t() @ a.float()))
        if it % 2 == rank % 2:          # skew the ranks so that flags, not luck, order the accesses
            torch.cuda._sleep(20_000_000)
    torch.cuda.synchronize()
    check_status("fused tp test")
    assert comm.check_canaries(), "a kernel wrote past a buffer of the symmetric arena"
    t = torch.tensor([res[k] for k in sorted(res)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({**dict(zip(sorted(res), t.tolist())), "stats": comm.stats}, f)
    dist.barrier()
    dist.destroy_process_group()


def run_fused_tp(world: int, iters: int = 5) -> dict:
    import tempfile

    import torch.multiprocessing as mp
    out = tempfile.mktemp(suffix=".json")
    port = 21000 + (os.getpid() * 13 + world) % 20000
    mp.spawn(_worker, args=(world, port, out, iters), nprocs=world, join=True)
    with open(out) as f:
        res = json.load(f)
    os.unlink(out)
    return res


def _absent_peer_worker(rank: int, world: int, port: int, out_path: str):
    """Rank 1 never publishes its chunk (it skips the launch on the host). Rank 0's bounded flag wait expires, the kernel
    returns, the status word becomes an exception, and the error-coordination boundary raises on both ranks."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from torchllmtuner_b200.accelerator.collectives import CoordinatedError, synchronize_local_errors
    from torchllmtuner_b200.errors import KernelStatusError
    from torchllmtuner_b200.ops.cuda_ext import check_status
    from torchllmtuner_b200.parallel.symm_tp import AG, FusedTPComm
    comm = FusedTPComm(dist.group.WORLD, dev, 256 * world, 256)
    verdict = "none"
    try:
        with synchronize_local_errors("all-gather of step 7"):
            if rank == 0:
                # what ag_gemm does before its GEMM, with a short poll limit: wait for every rank's `ready` epoch
                comm.ext.signal_peers([b + comm.off_flag[(AG, 0)] for b in comm.peer_base], comm.rank, 1)
                comm.ext.wait_flags(comm.base + comm.off_flag[(AG, 0)], world, 1, 7400, 1 << 15)
                check_status("all-gather wait")
    except KernelStatusError as e:
        verdict = "own:" + str(e)
    except CoordinatedError as e:
        verdict = "peer:" + str(e)
    torch.cuda.synchronize()
    ok = comm.check_canaries()
    gathered = [None] * world
    dist.all_gather_object(gathered, (verdict, ok))
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.barrier()
    dist.destroy_process_group()


def run_absent_peer(world: int = 2):
    import tempfile

    import torch.multiprocessing as mp
    out = tempfile.mktemp(suffix=".json")
    port = 24000 + (os.getpid() * 23 + world) % 20000
    mp.spawn(_absent_peer_worker, args=(world, port, out), nprocs=world, join=True)
    with open(out) as f:
        res = json.load(f)
    os.unlink(out)
    return res


def _vocab_worker(rank: int, world: int, port: int, out_path: str, iters: int):
    """Vocabulary-parallel head loss and embedding on the fused path against the full-vocabulary fp32 statement."""
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    import torch.nn.functional as F
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from torchllmtuner_b200.models.common import Embedding, Linear
    from torchllmtuner_b200.ops.cuda_ext import check_status
    from torchllmtuner_b200.parallel import symm_tp
    from torchllmtuner_b200.parallel.tensor_parallel import VocabParallelEmbedding
    from torchllmtuner_b200.parallel.vocab_parallel import VocabParallelHead, vocab_parallel_head_loss
    cr, D, V = 256, 256, 8 * 251 * world - (world - 1)   # chunk = 2008 (a multiple of 8), the last shard has padding rows
    T = cr * world
    g = torch.Generator(device=dev).manual_seed(7)    # the same table / head / tokens on every rank
    full_head = Linear(D, V, torch.bfloat16, dev)
    table = Embedding(V, D, dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        full_head.weight.copy_((torch.randn(V, D, generator=g, device=dev) * 0.2).bfloat16())
        table.weight.copy_(torch.randn(V, D, generator=g, device=dev).bfloat16())
    head = VocabParallelHead(full_head, rank, world, dist.group.WORLD)
    vpe = VocabParallelEmbedding(table, rank, world, dist.group.WORLD)
    res = {"loss": 0.0, "dh": 0.0, "dw": 0.0, "emb": 0.0, "demb": 0.0}

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))

    for it in range(iters):
        h = (torch.randn(T, D, generator=g, device=dev) * 0.5).bfloat16()
        targets = torch.randint(0, V, (T,), generator=g, device=dev)
        targets[::11] = -100
        hs = h[rank * cr:(rank + 1) * cr].clone().requires_grad_()
        head.weight.grad = None
        loss = vocab_parallel_head_loss(hs, head, targets[rank * cr:(rank + 1) * cr])
        (loss * 0.01).backward()
        tot = loss.detach().clone()
        dist.all_reduce(tot)
        hf = h.float().requires_grad_()
        wf = full_head.weight.detach().float().requires_grad_()
        ref = F.cross_entropy(hf @ wf.t(), targets, ignore_index=-100, reduction="sum")
        (ref * 0.01).backward()
        res["loss"] = max(res["loss"], abs(float(tot) - float(ref.detach())) / abs(float(ref.detach())))
        res["dh"] = max(res["dh"], rel(hs.grad, hf.grad[rank * cr:(rank + 1) * cr]))
        real = head.end - head.start
        res["dw"] = max(res["dw"], rel(head.weight.grad[:real], wf.grad[head.start:head.end]))
        assert float(head.weight.grad[real:].abs().max()) == 0.0 if real < head.chunk else True
        ids = torch.randint(0, V, (T,), generator=g, device=dev)
        go = torch.randn(T, D, generator=g, device=dev).bfloat16()
        vpe.weight.grad = None
        out = vpe(ids[rank * cr:(rank + 1) * cr])
        res["emb"] = max(res["emb"], float((out.detach().float() - table.weight[ids[rank * cr:(rank + 1) * cr]].float()).abs().max()))
        out.backward(go[rank * cr:(rank + 1) * cr])
        want = torch.zeros(V, D, device=dev).index_add_(0, ids, go.float())
        res["demb"] = max(res["demb"], rel(vpe.weight.grad[: vpe.end - vpe.start], want[vpe.start:vpe.end]))
        if it % 2 == rank % 2:
            torch.cuda._sleep(20_000_000)
    torch.cuda.synchronize()
    check_status("vocab-parallel test")
    stats = next(iter(symm_tp._COMMS.values())).stats if symm_tp._COMMS else {}
    t = torch.tensor([res[k] for k in sorted(res)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({**dict(zip(sorted(res), t.tolist())), "stats": stats}, f)
    dist.barrier()
    dist.destroy_process_group()


def run_vocab_parallel(world: int, iters: int = 3) -> dict:
    import tempfile

    import torch.multiprocessing as mp
    out = tempfile.mktemp(suffix=".json")
    port = 21500 + (os.getpid() * 13 + world) % 20000
    mp.spawn(_vocab_worker, args=(world, port, out, iters), nprocs=world, join=True)
    with open(out) as f:
        res = json.load(f)
    os.unlink(out)
    return res
