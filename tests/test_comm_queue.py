"""Slicing of peer-memory collectives into side jobs (host logic only; pointers are fake integers)."""
from torchllmtuner_b200.parallel.symm import COPY, REDUCE, CommQueue, Job


def test_copy_job_is_cut_in_order_and_completely():
    q = CommQueue(ext=None, bytes_per_gflop=1000.0, min_flops=0.0)
    done = []
    job = Job(COPY, [10_000], 50_000, 4096 + 16, 16, 1, 1, tag="u")
    job.on_done.append(lambda: done.append(1))
    q.push(job)
    covered, pos = 0, 0
    while q:
        s, cbs = q.take(1e9)          # 1 GFLOP -> 1000 bytes -> 992 after rounding to 16
        assert s["src"][0] == 10_000 + pos and s["dst"] == 50_000 + pos and s["n"] % 16 == 0
        pos += s["n"]
        covered += s["n"]
        for cb in cbs:
            cb()
    assert covered == 4096 + 16 and done == [1]


def test_reduce_job_advances_every_source_and_fp32_destination():
    q = CommQueue(ext=None, bytes_per_gflop=64.0, min_flops=0.0)
    q.push(Job(REDUCE, [1000, 2000], 9000, 64, 8, 2, 4, accumulate=True, wait_flags=7, n_wait=2, wait_value=3))
    s1, _ = q.take(1e9)               # 64 bytes / (2 sources * 2 bytes) = 16 elements
    assert s1["n"] == 16 and s1["src"] == [1000, 2000] and s1["dst"] == 9000 and s1["accumulate"] and s1["wait_value"] == 3
    s2, _ = q.take(1e9)
    assert s2["src"] == [1000 + 32, 2000 + 32] and s2["dst"] == 9000 + 64


def test_small_gemms_carry_nothing_and_flush_finishes_jobs():
    q = CommQueue(ext=None, bytes_per_gflop=1e6, min_flops=2e9)
    q.push(Job(COPY, [0], 0, 160, 16, 1, 1, tag="a"))
    q.push(Job(COPY, [0], 0, 160, 16, 1, 1, tag="b"))
    assert q.take(1e6) == (None, ())
    q.flush("a")
    assert len(q.jobs) == 1 and q.jobs[0].tag == "b"
    q.flush(None)
    assert not q


def test_canary_words_detect_a_write_past_the_last_buffer():
    import torch
    from torchllmtuner_b200.parallel.symm import canary_intact, write_canary
    arena = torch.zeros(4096 + 256, dtype=torch.uint8)
    write_canary(arena)
    assert canary_intact(arena)
    arena[:4096].fill_(7)                      # legal writes leave it intact
    assert canary_intact(arena)
    arena[4096 + 17] = 1                       # one byte past the buffers
    assert not canary_intact(arena)
