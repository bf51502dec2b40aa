"""Data pipeline: synthetic determinism and resume, text/SFT processing, packing, collating, cursor identity."""
import json
import os

import pytest
import torch

from torchllmtuner_b200.components.tokenizer import WhitespaceTokenizer
from torchllmtuner_b200.config import DataloaderConfig
from torchllmtuner_b200.datasets import RandomTokenDataLoader, RandomTokenSource, build_dataloader
from torchllmtuner_b200.datasets.contracts import IGNORE_INDEX, TextSequence
from torchllmtuner_b200.datasets.packing import concat_then_split, first_fit
from torchllmtuner_b200.datasets.processors import ChatProcessor


def test_synthetic_same_seed_step_same_batch_and_dp_slices():
    src = RandomTokenSource(1000, 8, 16, seed=3)
    a, b = src.global_batch_at(5), src.global_batch_at(5)
    assert torch.equal(a.input_ids, b.input_ids) and not torch.equal(a.input_ids, src.global_batch_at(6).input_ids)
    l0, l1 = RandomTokenDataLoader(src, 0, 2, 4), RandomTokenDataLoader(src, 1, 2, 4)
    b0, b1 = next(l0), next(l1)
    assert torch.equal(torch.cat([b0["input"], b1["input"]]), src.global_batch_at(0).input_ids)
    assert torch.equal(b0["labels"][:, :-1], b0["input"][:, 1:]) and (b0["labels"][:, -1] == IGNORE_INDEX).all()
    sd = l0.state_dict()
    nxt = next(l0)
    l2 = RandomTokenDataLoader(src, 0, 2, 4)
    l2.load_state_dict(sd)
    assert torch.equal(next(l2)["input"], nxt["input"])
    with pytest.raises(Exception):
        RandomTokenDataLoader(src, 0, 4, 2).load_state_dict(sd)


def _seq(n, base=0):
    toks = list(range(base, base + n))
    labels = toks[1:] + [IGNORE_INDEX]
    return TextSequence(toks, labels, list(range(n)), [0] * n)


def test_concat_then_split_positions_cuts_and_border_labels():
    rows = list(concat_then_split([_seq(5), _seq(7, 100), _seq(3, 200)], seq_len=8, pad_id=0))
    assert [len(r.tokens) for r in rows] == [8, 8]
    assert rows[0].cuts == [0, 5, 8] and rows[0].positions == [0, 1, 2, 3, 4, 0, 1, 2]
    assert rows[0].labels[4] == IGNORE_INDEX                 # nothing predicted across a document border
    assert rows[0].labels[7] == 103 and rows[1].tokens[0] == 103   # a document cut by the row end still predicts its next token
    assert rows[1].labels[3] == IGNORE_INDEX                 # ... and its true end is a border
    assert rows[1].cuts[-1] == 8 and rows[1].tokens[-1] == 0 and rows[1].labels[-1] == IGNORE_INDEX
    capped = list(concat_then_split([_seq(2), _seq(2, 10), _seq(2, 20)], seq_len=8, max_num_documents=2))
    assert len(capped) == 2 and capped[0].cuts[:3] == [0, 2, 4]


def test_first_fit_never_splits_documents():
    rows = list(first_fit([_seq(6), _seq(5, 100), _seq(2, 200), _seq(3, 300)], seq_len=8, num_bins=2))
    for r in rows:
        assert len(r.tokens) == 8
    docs = sorted(c2 - c1 for r in rows for c1, c2 in zip(r.cuts[:-1], r.cuts[1:]))
    assert {6, 5, 2, 3} <= set(docs)


def test_sft_masks_the_prompt(tmp_path):
    tok = WhitespaceTokenizer.from_texts(["what is two plus two", "four", "user assistant"])
    seq = ChatProcessor(tok)({"prompt": "what is two plus two", "response": "four"})
    sup = [t for t, l in zip(seq.tokens[1:], seq.labels[:-1]) if l != IGNORE_INDEX]
    assert tok.stoi["four"] in sup and tok.stoi["what"] not in sup


def test_text_loader_end_to_end_and_resume(tmp_path):
    texts = [" ".join(f"w{(i * 7 + j) % 50}" for j in range(5 + i % 9)) for i in range(40)]
    data = tmp_path / "corpus.jsonl"
    data.write_text("\n".join(json.dumps({"text": t}) for t in texts))
    tok = WhitespaceTokenizer.from_texts(texts)
    vocab = tmp_path / "vocab.json"
    tok.save(str(vocab))
    cfg = DataloaderConfig(dataset="local_jsonl", dataset_path=str(data), tokenizer_path=str(vocab), tokenizer_backend="whitespace",
                           num_prefetch_batches=0)
    mk = lambda: build_dataloader(cfg, vocab_size=1000, global_batch=4, seq_len=32, seed=1, dp_rank=0, dp_degree=2, rows_per_rank=2)  # noqa: E731
    a = mk()
    b1, b2 = next(a), next(a)
    assert b1["input"].shape == (2, 32) and b1["cu_seqlens"][0] == 0 and b1["cu_seqlens"][-1] == 64
    assert (b1["positions"][0, :3] == torch.tensor([0, 1, 2])).all()
    sd = a.state_dict()
    b3 = next(a)
    c = mk()
    c.load_state_dict(sd)
    assert torch.equal(next(c)["input"], b3["input"])
    cfg2 = DataloaderConfig(dataset="local_jsonl", dataset_path=str(data), tokenizer_path=str(vocab), tokenizer_backend="whitespace",
                            packing="first_fit", num_prefetch_batches=2)
    d = build_dataloader(cfg2, vocab_size=1000, global_batch=4, seq_len=32, seed=1, dp_rank=0, dp_degree=2, rows_per_rank=2)
    assert next(d)["input"].shape == (2, 32)
    with pytest.raises(Exception):
        d.load_state_dict(sd)          # different packing -> different corpus identity


def test_multimodal_helpers():
    from torchllmtuner_b200.datasets.multimodal import (build_mrope_positions, calculate_vision_tokens, insert_vision_placeholders,
                                                        process_image, smart_resize)
    h, w = smart_resize(500, 333, factor=28)
    assert h % 28 == 0 and w % 28 == 0
    patches, grid = process_image(torch.rand(3, 120, 90), patch=14, merge=2)
    assert patches.shape == (grid[1] * grid[2], 3 * 14 * 14)
    n = calculate_vision_tokens(grid)
    ids = insert_vision_placeholders([5, 99, 6], 99, [grid])
    assert ids.count(99) == n
    pos = build_mrope_positions(ids, 99, [grid])
    assert pos.shape == (3, len(ids)) and pos[0, 1] == pos[0, n] and pos[:, -1].max() == pos[:, -1].min()


def test_streaming_source_resumes_at_the_same_row_with_shuffle_buffer():
    from torchllmtuner_b200.datasets.sources import StreamingSource
    make = lambda: ({"id": i} for i in range(100))  # noqa: E731
    a = StreamingSource(make, shuffle_buffer_size=16, seed=3)
    first = [next(a)["id"] for _ in range(30)]
    state = a.state_dict()
    rest = [next(a)["id"] for _ in range(20)]
    b = StreamingSource(make, shuffle_buffer_size=16, seed=3)
    b.load_state_dict(state)
    assert [next(b)["id"] for _ in range(20)] == rest
    assert sorted(first + rest + [r["id"] for r in a]) == list(range(100))       # a permutation, nothing lost


def test_hf_disk_source_round_trip(tmp_path):
    datasets = pytest.importorskip("datasets")
    from torchllmtuner_b200.datasets.sources import HuggingFaceDiskSource
    ds = datasets.Dataset.from_dict({"text": [f"row {i}" for i in range(7)]})
    ds.save_to_disk(str(tmp_path / "d"))
    src = HuggingFaceDiskSource(str(tmp_path / "d"))
    assert len(src) == 7 and src[3]["text"] == "row 3"


def test_huggingface_tokenizer_special_tokens_and_chat_template(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    import json

    from tokenizers import models, pre_tokenizers
    from torchllmtuner_b200.components.tokenizer.huggingface import HuggingFaceTokenizer
    vocab = {"<s>": 0, "</s>": 1, "<unk>": 2, "hello": 3, "world": 4, "user": 5, "assistant": 6, ":": 7}
    tok = tokenizers.Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    d = tmp_path / "tok"
    d.mkdir()
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({
        "bos_token": "<s>", "eos_token": {"content": "</s>"},
        "chat_template": "{% for m in messages %}{{ m['role'] }} : {{ m['content'] }} {{ eos_token }}{% endfor %}"}))
    t = HuggingFaceTokenizer(str(d))
    assert (t.bos_id, t.eos_id, t.pad_id, t.vocab_size) == (0, 1, 1, 8)
    assert t.encode("hello world", add_bos=True, add_eos=True) == [0, 3, 4, 1]
    assert t.decode([3, 4]) == "hello world"
    text = t.apply_chat_template([{"role": "user", "content": "hello"}, {"role": "assistant", "content": "world"}])
    assert text.replace("</s>", " </s> ").split() == ["user", ":", "hello", "</s>", "assistant", ":", "world", "</s>"]
    assert t.identity().startswith("hf:") and t.identity() == HuggingFaceTokenizer(str(d)).identity()
    # what published templates rely on: raise_exception, loop controls, tojson that keeps unicode
    t.chat_template = ("{% for m in messages %}{% if m['role'] == 'tool' %}{{ raise_exception('tool turns need a call') }}{% endif %}"
                       "{% if m['role'] == 'system' %}{% continue %}{% endif %}{{ m['content'] | tojson }}{% endfor %}")
    assert t.apply_chat_template([{"role": "system", "content": "x"}, {"role": "user", "content": "h\u00e9"}]) == '"h\u00e9"'
    with pytest.raises(Exception, match="tool turns need a call"):
        t.apply_chat_template([{"role": "tool", "content": "x"}])


def test_dataset_composition_concat_mix_and_epoch_order():
    from torchllmtuner_b200.datasets.composition import DatasetConcat, DatasetIterationPolicy, DatasetMix, SingleDataset, epoch_order
    a = SingleDataset([{"v": i} for i in range(5)], lambda r: r["v"])
    b = SingleDataset([{"v": 100 + i} for i in range(3)], lambda r: r["v"])
    cat = DatasetConcat([a, b])
    assert len(cat) == 8 and [cat.get(i) for i in range(8)] == [0, 1, 2, 3, 4, 100, 101, 102]
    mix = DatasetMix([a, b], [0.9, 0.1], seed=1)
    draws = [mix.get(i) for i in range(2000)]
    assert draws == [mix.get(i) for i in range(2000)]                          # deterministic in the index
    share_b = sum(d >= 100 for d in draws) / len(draws)
    assert 0.06 < share_b < 0.14, share_b
    pol = DatasetIterationPolicy(shuffle=True, seed=3)
    parts = [epoch_order(10, 0, pol, r, 2) for r in range(2)]
    assert sorted(parts[0] + parts[1]) == list(range(10)) and not set(parts[0]) & set(parts[1])   # DP shards partition the epoch
    assert epoch_order(10, 0, pol, 0, 2) != epoch_order(10, 1, pol, 0, 2)                          # reshuffled per epoch
    assert epoch_order(10, 0, DatasetIterationPolicy(shuffle=False), 1, 2) == [1, 3, 5, 7, 9]


def test_prefetch_thread_ends_when_the_cursor_is_restored_or_the_loader_closed(tmp_path):
    import time
    texts = [" ".join(f"w{(i * 7 + j) % 50}" for j in range(20)) for i in range(40)]
    data = tmp_path / "corpus.jsonl"
    data.write_text("\n".join(json.dumps({"text": t}) for t in texts))
    vocab = tmp_path / "vocab.json"
    WhitespaceTokenizer.from_texts(texts).save(str(vocab))
    cfg = DataloaderConfig(dataset="local_jsonl", dataset_path=str(data), tokenizer_path=str(vocab), tokenizer_backend="whitespace",
                           num_prefetch_batches=2)
    dl = build_dataloader(cfg, vocab_size=1000, global_batch=2, seq_len=16, seed=0, dp_rank=0, dp_degree=1, rows_per_rank=2)
    first = [next(dl) for _ in range(3)]
    t1 = dl._thread
    time.sleep(0.1)
    assert t1 is not None and t1.is_alive()                  # blocked on the full queue
    sd = dl.state_dict()
    dl.load_state_dict({**sd, "delivered": 1})
    assert not t1.is_alive()
    assert torch.equal(next(dl)["input"], first[1]["input"])  # the stream restarts at the restored cursor
    t2 = dl._thread
    dl.close()
    assert not t2.is_alive() and dl._thread is None
