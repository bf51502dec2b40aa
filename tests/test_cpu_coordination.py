"""Failure detection without a device fault: every failure is made on the host and observed by gloo ranks
(model: the reference's coordination tests, tests/unit_tests/cpu/accelerator/test_collectives.py)."""
import os
import sys
import tempfile

import pytest
import torch


def _spawn(fn, world, *args):
    import torch.multiprocessing as mp
    out = tempfile.mkdtemp()
    port = 23000 + (os.getpid() * 19 + hash(fn.__name__)) % 15000
    mp.spawn(_entry, args=(world, port, fn.__name__, out, args), nprocs=world, join=True)
    res = []
    for r in range(world):
        with open(os.path.join(out, f"{r}.txt")) as f:
            res.append(f.read())
    return res


def _entry(rank, world, port, fn_name, out, args):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      LLMTUNER_DEVICE="cpu")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import datetime

    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    torch.set_num_threads(1)
    try:
        verdict = globals()[fn_name](rank, world, *args)
    except BaseException as e:  # noqa: BLE001
        verdict = f"UNCAUGHT {type(e).__name__}: {e}"
    with open(os.path.join(out, f"{rank}.txt"), "w") as f:
        f.write(verdict)
    if verdict.startswith("left") or verdict.startswith("timeout"):
        os._exit(0)                      # a rank left on purpose: no farewell collectives
    dist.barrier()
    dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------- cases (run in children)
def _case_one_rank_raises(rank, world):
    from torchllmtuner_b200.accelerator.collectives import CoordinatedError, synchronize_local_errors
    try:
        with synchronize_local_errors("load-shard"):
            if rank == 1:
                raise ValueError("disk error on rank 1")
    except ValueError:
        return "own"
    except CoordinatedError as e:
        return "peer:" + str(e)
    return "none"


def _case_all_ok(rank, world):
    from torchllmtuner_b200.accelerator.collectives import synchronize_local_errors
    with synchronize_local_errors("phase"):
        pass
    return "ok"


def _case_nan_update_is_skipped_everywhere(rank, world):
    """A non-finite gradient on one rank: the global norm is non-finite on every rank, no rank updates, all raise."""
    from dist_cases import base_flat
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.errors import LLMTunerError
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(data_parallel_shard_size=world, dump_folder=tempfile.mkdtemp()))
    tr = Trainer(cfg)
    tr.train_step()
    before = [u.master.clone() for u in tr.asm.fsdp.units]
    if rank == 0:       # poison one gradient contribution on one rank through the loss scale
        for p in tr.model.parameters():
            p.register_hook(lambda g: g * float("nan"))
            break
    try:
        tr.train_step()
        verdict = "no-raise"
    except LLMTunerError:
        same = all(torch.equal(a, u.master) for a, u in zip(before, tr.asm.fsdp.units))
        verdict = "raised,unchanged" if same else "raised,CHANGED"
    tr.close()
    return verdict


def _case_checkpoint_publication_failure(rank, world, folder):
    """The rank that publishes fails; every rank learns of it and the previous checkpoint stays the latest."""
    from dist_cases import base_flat
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(data_parallel_shard_size=world, dump_folder=folder, enable=True, interval=1000, last_save_model_only=False))
    tr = Trainer(cfg)
    tr.train_step()
    tr.checkpointer.save(tr.progress.step, force=True)
    tr.checkpointer.wait()
    first = tr.checkpointer.latest_step()
    tr.train_step()
    import torchllmtuner_b200.components.checkpointer.dcp_manager as dm
    real = os.replace

    def failing_replace(a, b):
        if rank == 0 and "step-" in str(b):
            raise OSError("injected publication failure")
        return real(a, b)
    dm.os.replace = failing_replace
    try:
        tr.checkpointer.save(tr.progress.step, force=True)
        tr.checkpointer.wait()
        verdict = "no-raise"
    except Exception as e:  # noqa: BLE001
        verdict = type(e).__name__
    finally:
        dm.os.replace = real
    latest = tr.checkpointer.latest_step()
    tr.close()
    return f"{verdict},{first},{latest}"


def _case_rank_leaves_between_steps(rank, world):
    """Rank 1 leaves after a completed step with nothing in flight; rank 0's next collective ends with an error inside
    the shortened process-group timeout instead of hanging."""
    import datetime
    import time

    import torch.distributed as dist
    from torchllmtuner_b200.accelerator.collectives import set_pg_timeouts
    t = torch.ones(1)
    dist.all_reduce(t)                                   # "step 1": both ranks take part
    set_pg_timeouts(3, [])
    if rank == 1:
        return "left"
    t0 = time.time()
    try:
        work = dist.all_reduce(t, async_op=True)
        work.wait(datetime.timedelta(seconds=3))
        return "no-error"
    except Exception as e:  # noqa: BLE001
        return f"timeout after {time.time() - t0:.1f}s: {type(e).__name__}"


def _case_vocab_parallel_loss_and_embedding(rank, world):
    """Vocab-sharded logits: loss, gradient and entropy equal the full-vocabulary statement; the vocab-parallel embedding
    returns this rank's token shard of the full lookup."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from torchllmtuner_b200.components.loss import LossParallelCrossEntropy, vocab_parallel_entropy
    from torchllmtuner_b200.models.common import Embedding
    from torchllmtuner_b200.parallel.tensor_parallel import VocabParallelEmbedding
    from torchllmtuner_b200.utils.vocabulary import vocab_shard_bounds
    torch.manual_seed(5)
    T, V, D = 24, 37, 8                                     # V does not divide evenly
    logits = torch.randn(T, V, dtype=torch.float64)
    targets = torch.randint(0, V, (T,))
    targets[3] = -100
    lo, hi = vocab_shard_bounds(V, world, rank)
    shard = logits[:, lo:hi].clone().requires_grad_()
    loss = LossParallelCrossEntropy.apply(shard, targets, dist.group.WORLD, lo)
    loss.backward()
    full = logits.clone().requires_grad_()
    ref = F.cross_entropy(full, targets, ignore_index=-100, reduction="sum")
    ref.backward()
    e1 = abs(float(loss) - float(ref))
    e2 = float((shard.grad - full.grad[:, lo:hi]).abs().max())
    ent = vocab_parallel_entropy(logits[:, lo:hi], dist.group.WORLD)
    p = torch.softmax(logits, -1)
    e3 = float((ent - (-(p * torch.log(p)).sum(-1))).abs().max())
    # embedding: same table on every rank, each keeps rows [lo, hi); tokens arrive sequence-sharded
    table = Embedding(V, D, dtype=torch.float32)
    with torch.no_grad():
        table.weight.copy_(torch.arange(V * D, dtype=torch.float32).view(V, D) / 100.0)
    vpe = VocabParallelEmbedding(table, rank, world, dist.group.WORLD)
    ids = torch.randint(0, V, (T,))
    mine = ids[rank * (T // world):(rank + 1) * (T // world)]
    out = vpe(mine)
    e4 = float((out - table.weight[mine]).abs().max())
    return f"{e1:.2e},{e2:.2e},{e3:.2e},{e4:.2e}"


def _case_vocab_parallel_head(rank, world):
    """Sequence-sharded hidden states against a vocabulary-sharded head: the summed loss over the ranks, the hidden-state
    gradient shard, the head gradient shard and the embedding gradient equal the full-vocabulary statement."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from torchllmtuner_b200.models.common import Embedding, Linear
    from torchllmtuner_b200.parallel.tensor_parallel import VocabParallelEmbedding
    from torchllmtuner_b200.parallel.vocab_parallel import VocabParallelHead, vocab_parallel_head_loss
    torch.manual_seed(11)
    T, V, D = 16 * world, 37, 8                             # V does not divide evenly: the last shard is padded
    cr = T // world
    full_head = Linear(D, V, torch.float64, None)
    with torch.no_grad():
        full_head.weight.copy_(torch.randn(V, D, dtype=torch.float64) * 0.3)
    h = torch.randn(T, D, dtype=torch.float64)
    targets = torch.randint(0, V, (T,))
    targets[5] = -100
    head = VocabParallelHead(full_head, rank, world, dist.group.WORLD)
    hs = h[rank * cr:(rank + 1) * cr].clone().requires_grad_()
    loss = vocab_parallel_head_loss(hs, head, targets[rank * cr:(rank + 1) * cr])
    (loss * 0.25).backward()                                # the same upstream factor on every rank, as in training
    tot = loss.detach().clone()
    dist.all_reduce(tot)
    hf = h.clone().requires_grad_()
    wf = full_head.weight.detach().clone().requires_grad_()
    ref = F.cross_entropy(hf @ wf.t(), targets, ignore_index=-100, reduction="sum")
    (ref * 0.25).backward()
    e1 = abs(float(tot) - float(ref.detach()))
    e2 = float((hs.grad - hf.grad[rank * cr:(rank + 1) * cr]).abs().max())
    real = head.end - head.start
    e3 = float((head.weight.grad[:real] - wf.grad[head.start:head.end]).abs().max()) if real else 0.0
    e3 = max(e3, float(head.weight.grad[real:].abs().max()) if real < head.chunk else 0.0)      # padding rows stay zero
    lg = head.full_logits(hs.detach())
    e4 = float((lg - (h[rank * cr:(rank + 1) * cr] @ full_head.weight.t())).abs().max())
    # embedding gradient: owned rows receive the output gradient of every token with that id, from every rank's shard
    table = Embedding(V, D, dtype=torch.float64)
    with torch.no_grad():
        table.weight.copy_(torch.randn(V, D, dtype=torch.float64))
    vpe = VocabParallelEmbedding(table, rank, world, dist.group.WORLD)
    ids = torch.randint(0, V, (T,))
    go = torch.randn(T, D, dtype=torch.float64)
    out = vpe(ids[rank * cr:(rank + 1) * cr])
    out.backward(go[rank * cr:(rank + 1) * cr])
    want = torch.zeros(V, D, dtype=torch.float64).index_add_(0, ids, go)
    e5 = float((vpe.weight.grad[: vpe.end - vpe.start] - want[vpe.start:vpe.end]).abs().max()) if vpe.end > vpe.start else 0.0
    return f"{e1:.2e},{e2:.2e},{e3:.2e},{e4:.2e},{e5:.2e}"


def _case_unequal_loader_exhaustion(rank, world):
    """Rank 1's data stream ends one batch early; rank 0's raises. Both ranks must leave `fetch_batch` the same way,
    before any step collective."""
    from types import SimpleNamespace as NS

    from torchllmtuner_b200.datasets.contracts import DataloaderExhaustedError
    from torchllmtuner_b200.trainer.runtime.batch import fetch_batch
    env = NS(world_size=world, device=torch.device("cpu"))
    out = []
    it = iter([{"x": 1}, {"x": 2}] if rank == 0 else [{"x": 1}])
    for _ in range(2):
        try:
            out.append("ready" if fetch_batch(it, env) is not None else "none")
        except DataloaderExhaustedError:
            out.append("exhausted")

    def broken():
        if rank == 0:
            raise OSError("disk error")
        yield {"x": 3}
    try:
        fetch_batch(broken(), env)
        out.append("ready")
    except OSError:
        out.append("own-error")
    except RuntimeError as e:
        out.append("peer-error" if "peer rank failed" in str(e) else "other")
    return ",".join(out)


# ---------------------------------------------------------------------------------------------- tests
def test_unequal_loader_exhaustion_and_read_errors_are_agreed_on():
    res = _spawn(_case_unequal_loader_exhaustion, 2)
    assert res[0] == "ready,exhausted,own-error" and res[1] == "ready,exhausted,peer-error", res


def test_vocab_parallel_cross_entropy_entropy_and_embedding_match_the_full_vocabulary():
    for r in _spawn(_case_vocab_parallel_loss_and_embedding, 2):
        assert r.count(",") == 3, r
        assert all(float(x) < 1e-5 for x in r.split(",")), r


@pytest.mark.parametrize("world", [2, 3])
def test_vocab_parallel_head_loss_and_gradients_match_the_full_head(world):
    for r in _spawn(_case_vocab_parallel_head, world):
        assert r.count(",") == 4, r
        assert all(float(x) < 2e-5 for x in r.split(",")), r      # the statement computes in fp32


def test_rank_leaving_between_steps_ends_the_next_collective_with_an_error():
    res = _spawn(_case_rank_leaves_between_steps, 2)
    assert res[1] == "left" and res[0].startswith("timeout after"), res
    assert float(res[0].split()[2][:-2]) < 15.0, res


def test_one_rank_raising_becomes_every_rank_raising():
    res = _spawn(_case_one_rank_raises, 2)
    assert res[1] == "own" and res[0].startswith("peer:") and "load-shard" in res[0], res


def test_no_error_passes_through():
    assert _spawn(_case_all_ok, 2) == ["ok", "ok"]


def test_non_finite_gradient_skips_update_on_every_rank():
    res = _spawn(_case_nan_update_is_skipped_everywhere, 2)
    assert res == ["raised,unchanged", "raised,unchanged"], res


def test_checkpoint_publication_failure_keeps_previous_checkpoint():
    folder = tempfile.mkdtemp()
    res = _spawn(_case_checkpoint_publication_failure, 2, folder)
    for r in res:
        assert r.count(",") == 2, res
        verdict, first, latest = r.split(",")
        assert verdict != "no-raise" and first == latest, res


# ---------------------------------------------------------------------------------------------- a rank dies during a save
def _rank_exit_worker(rank, world, port, folder, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                      LLMTUNER_DEVICE="cpu")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import datetime

    import torch.distributed as dist
    from dist_cases import base_flat
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.accelerator.collectives import set_pg_timeouts
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    torch.set_num_threads(1)
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(data_parallel_shard_size=world, dump_folder=folder, enable=True, interval=1000, last_save_model_only=False))
    tr = Trainer(cfg)
    for _ in range(2):
        tr.dataloader.cursor = 0
        tr.train_step()
    tr.checkpointer.save(2, force=True)
    tr.checkpointer.wait()
    tr.dataloader.cursor = 0
    tr.train_step()
    set_pg_timeouts(4, [])
    import torchllmtuner_b200.components.checkpointer.dcp_manager as dm
    if rank == 1:
        real_save = dm.dcp.save

        def dying_save(*a, **k):
            os._exit(17)                      # the rank vanishes inside the step-3 save, before anything is published
        dm.dcp.save = dying_save
    verdict = "saved"
    try:
        tr.checkpointer.save(3, force=True)
        tr.checkpointer.wait()
    except BaseException as e:  # noqa: BLE001
        verdict = "error:" + type(e).__name__
    with open(os.path.join(out, f"{rank}.txt"), "w") as f:
        f.write(f"{verdict},{tr.checkpointer.latest_step()}")
    os._exit(0)


def test_rank_dying_inside_a_save_leaves_the_previous_checkpoint_and_it_resumes_exactly(tmp_path):
    import torch.multiprocessing as mp
    from dist_cases import base_flat, run_ranks
    folder, out = str(tmp_path / "run"), str(tmp_path / "out")
    os.makedirs(out)
    port = 25000 + os.getpid() % 15000
    ctx = mp.spawn(_rank_exit_worker, args=(2, port, folder, out), nprocs=2, join=False)
    for p in ctx.processes:
        p.join(120)
    assert ctx.processes[1].exitcode == 17
    verdict, latest = open(os.path.join(out, "0.txt")).read().split(",")
    assert verdict.startswith("error:") and latest == "2", (verdict, latest)
    assert not os.path.exists(os.path.join(folder, "checkpoint", "step-3", ".metadata"))
    # a fresh job resumes from step 2 and reproduces the uninterrupted run
    ref = run_ranks(2, base_flat(data_parallel_shard_size=2), steps=4)
    got = run_ranks(2, base_flat(data_parallel_shard_size=2, dump_folder=folder, enable=True, _load=True,
                                 exclude_from_loading=["dataloader", "rng"]), steps=2)
    assert max(abs(a - b) for a, b in zip(ref["loss"][2:], got["loss"])) < 1e-6, (ref, got)


# ---------------------------------------------------------------------------------------------- HF export / import under TP
def _case_hf_round_trip_under_tp(rank, world, folder):
    """Two tensor-parallel ranks export full Hugging Face tensors (row-parallel weights are scattered back into place),
    then import them again into freshly, differently initialised shards."""
    import torch.distributed as dist
    from dist_cases import base_flat
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.components.checkpointer.hf import load_hf_checkpoint, save_hf_checkpoint
    flat = base_flat(tensor_parallel_size=2, data_parallel_shard_size=1, dump_folder=folder)
    cfg = LLMTunerConfig()
    cfg.apply_flat(flat)
    tr = Trainer(cfg)
    tr.train_step()
    save_hf_checkpoint(tr, os.path.join(folder, "hf"), "float32")
    want = {u.name: u.master.clone() for u in tr.asm.fsdp.units}
    tr.close()
    cfg2 = LLMTunerConfig()
    cfg2.apply_flat(dict(flat, seed=7))
    tr2 = Trainer(cfg2)
    before = max(float((u.master - want[u.name]).abs().max()) for u in tr2.asm.fsdp.units)
    load_hf_checkpoint(tr2, os.path.join(folder, "hf"))
    after = max(float((u.master - want[u.name]).abs().max()) for u in tr2.asm.fsdp.units)
    tr2.close()
    dist.barrier()
    return f"{before:.3e},{after:.3e}"


def test_hf_export_and_import_under_tensor_parallelism(tmp_path):
    folder = str(tmp_path / "run")
    for r in _spawn(_case_hf_round_trip_under_tp, 2, folder):
        assert r.count(",") == 1, r
        before, after = (float(x) for x in r.split(","))
        assert before > 1e-3 and after == 0.0, r
    # the exported folder holds full tensors: a single rank reads it too
    import torch
    from dist_cases import base_flat
    from safetensors import safe_open
    from torchllmtuner_b200 import LLMTunerConfig, Trainer
    from torchllmtuner_b200.components.checkpointer.hf import load_hf_checkpoint
    cfg = LLMTunerConfig()
    cfg.apply_flat(base_flat(dump_folder=folder, seed=11))
    os.environ["LLMTUNER_DEVICE"] = "cpu"
    tr = Trainer(cfg)
    try:
        load_hf_checkpoint(tr, os.path.join(folder, "hf"))
        import glob
        f = safe_open(glob.glob(os.path.join(folder, "hf", "*.safetensors"))[0], "pt")
        name = "model.layers.0.self_attn.o_proj.weight"
        assert name in f.keys()
        assert torch.equal(dict(tr.model.named_parameters())[name].detach().float(), f.get_tensor(name).float())
    finally:
        tr.close()
