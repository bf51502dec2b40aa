"""Small pieces with sharp edges, each on its own: the variable-size exchange behind DistMuon (gloo arm), sliced streaming
of host-resident state, step-counter validation, box planners refusing checkpoints that do not fit, and the order in which
an overlapped optimizer update visits the sharding units."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _exchange_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from torchllmtuner_b200.components.optimizer.muon import exchange
    # rank r sends (r + 1) * (d + 1) elements to rank d, each holding 100 * r + d
    send = [torch.full(((rank + 1) * (d + 1),), 100.0 * rank + d, dtype=torch.bfloat16) for d in range(world)]
    recv_sizes = [(s + 1) * (rank + 1) for s in range(world)]
    got = exchange(send, recv_sizes, dist.group.WORLD)
    ok = all(g.numel() == n and g.dtype == torch.bfloat16 and bool((g.float() == 100.0 * s + rank).all())
             for s, (g, n) in enumerate(zip(got, recv_sizes)))
    empty = exchange([torch.zeros(0, dtype=torch.bfloat16) for _ in range(world)], [0] * world, dist.group.WORLD)
    ok = ok and all(e.numel() == 0 for e in empty)
    if rank == 0:
        open(out, "w").write("ok" if ok else "bad")
    dist.barrier()
    dist.destroy_process_group()


def test_variable_size_exchange_without_native_all_to_all(tmp_path):
    import socket
    out = str(tmp_path / "res")
    with socket.socket() as sk:                       # a port nobody holds right now
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    mp.spawn(_exchange_worker, args=(3, port, out), nprocs=3, join=True)
    assert open(out).read() == "ok"


def test_staged_slices_cover_a_range_exactly_once_on_the_host():
    from torchllmtuner_b200.components.optimizer.sharded import StagedSlices
    st = StagedSlices(torch.device("cpu"), slice_elems=7)
    m, v = torch.zeros(40), torch.zeros(40)
    seen = []

    def kernel(a, b, views):
        seen.append((a, b))
        views[0][:] += 1.0          # in place on the host arrays' own slices
        views[1][:] += 2.0
    st.run([m, v], 3, 33, kernel)
    st.finish()
    assert seen == [(3, 10), (10, 17), (17, 24), (24, 31), (31, 33)]
    assert m[3:33].eq(1).all() and m[:3].eq(0).all() and m[33:].eq(0).all() and v[3:33].eq(2).all()
    assert st.stats["slices"] == 5


def test_step_counter_validation():
    from torchllmtuner_b200.components.checkpointer.dcp_manager import validate_step_counter
    from torchllmtuner_b200.errors import ConfigError
    assert validate_step_counter(7, key="k") == 7 and validate_step_counter(torch.tensor(3.0), key="k") == 3
    for bad in (-1, 2.5, float("nan"), float("inf"), True, "3", torch.tensor([1, 2])):
        with pytest.raises(ConfigError):
            validate_step_counter(bad, key="k")


def test_box_planners_refuse_a_checkpoint_that_does_not_fit(tmp_path):
    """Boxes written from two 'ranks' form one whole tensor; a reader gets exactly its box, and is refused when the stored
    tensor has another shape or does not cover the box."""
    import torch.distributed.checkpoint as dcp
    from torchllmtuner_b200.components.checkpointer.boxes import BoxLoadPlanner, BoxSavePlanner, boxes_of_slice
    from torchllmtuner_b200.errors import ConfigError
    full = torch.arange(6 * 4, dtype=torch.float32).view(6, 4)
    flat = full.reshape(-1)
    table, state = {}, {}
    for lo, hi in ((0, 10), (10, 24)):                               # two flat shards that cut a row in the middle
        for b in boxes_of_slice("w", lo, hi, (6, 4), (6, 4), (0, 0)):
            key = f"w#box{len(table)}"
            table[key] = b
            state[key] = flat[lo + b.start: lo + b.start + b.numel].view(b.sizes)
    path = str(tmp_path / "ck")
    dcp.save(state, checkpoint_id=path, planner=BoxSavePlanner(table), no_dist=True)
    whole = {"w": torch.zeros(6, 4)}
    dcp.load(whole, checkpoint_id=path, no_dist=True)                # any reader sees one ordinary tensor
    assert torch.equal(whole["w"], full)
    # a reader that owns flat [5, 19) under another cut
    rtable, want, dst = {}, {}, torch.zeros(14)
    for b in boxes_of_slice("w", 5, 19, (6, 4), (6, 4), (0, 0)):
        key = f"w#box{len(rtable)}"
        rtable[key] = b
        want[key] = dst[b.start:b.start + b.numel].view(b.sizes)
    dcp.load(want, checkpoint_id=path, planner=BoxLoadPlanner(rtable), no_dist=True)
    assert torch.equal(dst, flat[5:19])
    # another global shape
    other = boxes_of_slice("w", 0, 8, (2, 4), (8, 4), (0, 0))
    with pytest.raises(BaseException) as refused:       # DCP wraps planner errors in a BaseException subclass
        dcp.load({"w#box0": torch.zeros(other[0].sizes)}, checkpoint_id=path, planner=BoxLoadPlanner({"w#box0": other[0]}), no_dist=True)
    assert "expects (8, 4)" in repr(refused.value) or "expects (8, 4)" in str(getattr(refused.value, "failures", ""))
    # a missing tensor is reported, not invented
    p = BoxLoadPlanner({"v#box0": boxes_of_slice("v", 0, 4, (4,), (4,), (0,))[0]})
    dcp.load({"v#box0": torch.zeros(4)}, checkpoint_id=path, planner=p, no_dist=True)
    assert p.missing == {"v"}
    with pytest.raises(ConfigError):
        boxes_of_slice("w", 0, 8, (2, 4), (1, 4), (0, 1))           # a box that cannot lie inside the global tensor


def test_overlapped_update_visits_units_in_the_order_the_forward_needs_them():
    from types import SimpleNamespace as U
    from torchllmtuner_b200.components.optimizer.sharded import ShardedAdamW
    units = [U(name="embedding", block_index=None), U(name="block0", block_index=0), U(name="block0.experts", block_index=0),
             U(name="block1", block_index=1), U(name="head", block_index=None), U(name="rest", block_index=None)]
    opt = ShardedAdamW.__new__(ShardedAdamW)
    opt.units = units
    assert [u.name for u in opt.overlap_order()] == ["embedding", "rest", "block0", "block0.experts", "block1", "head"]


def test_a_planner_error_reaches_the_caller_as_this_frameworks_error(tmp_path):
    """torch wraps what a planner raises in an exception that derives from BaseException; the checkpointer's boundary
    unwraps it so that `except Exception` cleanup paths and the caller's `except ConfigError` both work."""
    import torch.distributed.checkpoint as dcp
    from torchllmtuner_b200.components.checkpointer.boxes import (BoxLoadPlanner, BoxSavePlanner, CheckpointIOError,
                                                                  boxes_of_slice, dcp_errors)
    from torchllmtuner_b200.errors import ConfigError
    b = boxes_of_slice("w", 0, 8, (2, 4), (2, 4), (0, 0))[0]
    path = str(tmp_path / "ck")
    with dcp_errors("saving"):
        dcp.save({"w#box0": torch.ones(2, 4)}, checkpoint_id=path, planner=BoxSavePlanner({"w#box0": b}), no_dist=True)
    wrong = boxes_of_slice("w", 0, 8, (2, 4), (4, 4), (0, 0))[0]
    with pytest.raises(ConfigError, match="expects"):
        with dcp_errors("loading"):
            dcp.load({"w#box0": torch.zeros(2, 4)}, checkpoint_id=path, planner=BoxLoadPlanner({"w#box0": wrong}), no_dist=True)
    with pytest.raises(CheckpointIOError, match="ranks"):
        with dcp_errors("loading"):
            dcp.load({"w": torch.zeros(3, 4)}, checkpoint_id=path, no_dist=True)      # torch's own size check


@pytest.mark.parametrize("causal", [True, False])
def test_attention_backward_from_lse_matches_autograd(causal):
    """The chunked backward that serves head sizes with a forward kernel only: same gradients as autograd through the
    plain statement, for grouped heads, several documents, a chunk size that cuts documents, and offset diagonals."""
    import torch
    from torchllmtuner_b200.ops import reference as ref
    torch.manual_seed(0)
    Hq, Hkv, d = 4, 2, 16
    pieces = [(0, 37, 0, 37, 0), (37, 20, 37, 50, 30), (57, 9, 87, 9, 0)]       # the middle piece: 20 queries at the end of 50 keys
    q = torch.randn(66, Hq, d, dtype=torch.float64, requires_grad=True)
    k = torch.randn(96, Hkv, d, dtype=torch.float64, requires_grad=True)
    v = torch.randn(96, Hkv, d, dtype=torch.float64, requires_grad=True)

    def plain(q, k, v):                      # float64 statement (attention_pieces computes in fp32)
        outs = []
        for (q0, n, k0, m, off) in pieces:
            s = torch.einsum("qhd,khd->hqk", q[q0:q0 + n], k[k0:k0 + m].repeat_interleave(Hq // Hkv, 1)) * 0.3
            if causal:
                s = s.masked_fill(torch.arange(m)[None, :] > torch.arange(n)[:, None] + off, float("-inf"))
            outs.append((torch.einsum("hqk,khd->qhd", s.softmax(-1), v[k0:k0 + m].repeat_interleave(Hq // Hkv, 1)), s.logsumexp(-1)))
        return torch.cat([o for o, _ in outs]), torch.cat([l for _, l in outs], 1)
    o, lse = plain(q, k, v)
    go = torch.randn_like(o)
    want = torch.autograd.grad(o, [q, k, v], go)
    for chunk in (7, 512):
        got = ref.attention_backward_rows(q.detach(), k.detach(), v.detach(), o.detach(), go, lse.detach(), pieces, causal, 0.3, q_chunk=chunk)
        for a, b, n in zip(got, want, "qkv"):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-5), (n, chunk, (a - b).abs().max())    # softmax algebra is fp32


def test_attention_accepts_values_narrower_than_keys():
    """Latent attention has 192-wide keys and 128-wide values; the op's contract is q/k [.., d], v [.., dv] -> [.., dv]."""
    import torch
    from torchllmtuner_b200 import ops
    from torchllmtuner_b200.errors import ConfigError
    torch.manual_seed(0)
    q, k, v = torch.randn(10, 4, 8), torch.randn(10, 2, 8), torch.randn(10, 2, 6)
    meta = ops.AttnMeta.build(torch.tensor([0, 4, 10]))
    o = ops.attention(q, k, v, meta, 0.3)
    assert o.shape == (10, 4, 6)
    s = torch.einsum("qhd,khd->hqk", q[:4], k[:4].repeat_interleave(2, 1)) * 0.3
    s = s.masked_fill(torch.arange(4)[None, :] > torch.arange(4)[:, None], float("-inf"))
    want = torch.einsum("hqk,khd->qhd", s.softmax(-1), v[:4].repeat_interleave(2, 1))
    assert torch.allclose(o[:4], want, atol=1e-5)
    assert ops.functional.device_head_dim(72) == 128 and ops.functional.device_head_dim(192) == 256 and ops.functional.device_head_dim(300) is None
    with pytest.raises(ConfigError):
        ops.attention(q, k, torch.randn(9, 2, 6), meta, 0.3)          # rows must agree
