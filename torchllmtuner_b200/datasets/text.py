"""Text data loader: source -> processor -> packing -> collator, sharded over data-parallel ranks, with a prefetch
thread and a resumable cursor (reference: llmtuner/datasets/dataloader.py:41-234, loader_builder.py:154-317,
packing/global_rows.py:13-97)."""
from __future__ import annotations

import queue
import threading

from ..components.tokenizer import build_tokenizer
from ..errors import ConfigError
from .collators import TextCollator
from .composition import DatasetIterationPolicy, SingleDataset, epoch_order
from .contracts import BaseDataLoader, DataloaderExhaustedError, require_same_dp_degree
from .corpus_identity import corpus_data_identity
from .packing import concat_then_split, first_fit
from .processors import ChatProcessor, TextProcessor
from .sources import build_source


class TextDataLoader(BaseDataLoader):
    """Deterministic: the stream of packed rows is a pure function of (data, seed, dp coordinates), so the state is just
    the number of batches already delivered; a resume replays the packer up to that point without tokenising twice the
    rows it can skip wholesale (whole epochs)."""

    def __init__(self, dataset, collator, *, seq_len, rows_per_rank, dp_rank, dp_degree, policy, packing, num_bins,
                 max_num_documents, pad_id, identity, prefetch: int = 2):
        self.ds, self.collator = dataset, collator
        self.seq_len, self.rows, self.dp_rank, self.dp_degree = seq_len, rows_per_rank, dp_rank, dp_degree
        self.policy, self.packing, self.num_bins, self.max_docs, self.pad_id = policy, packing, num_bins, max_num_documents, pad_id
        self.identity = identity
        self.delivered = 0
        self.prefetch = prefetch
        self._q: queue.Queue | None = None
        self._thread = None
        self._gen = None
        self._stop = None

    # ------------------------------------------------------------------ stream
    def _sequences(self):
        epoch = 0
        while True:
            order = epoch_order(len(self.ds), epoch, self.policy, self.dp_rank, self.dp_degree)
            if not order:
                return
            for i in order:
                yield self.ds.get(i)
            epoch += 1
            if not self.policy.repeat:
                return

    def _batches(self):
        packer = concat_then_split(self._sequences(), self.seq_len, self.pad_id, self.max_docs) if self.packing == "concat_then_split" \
            else first_fit(self._sequences(), self.seq_len, self.pad_id, self.num_bins)
        rows = []
        for r in packer:
            rows.append(r)
            if len(rows) == self.rows:
                yield self.collator(rows)
                rows = []

    def _start(self):
        gen = self._batches()
        for _ in range(self.delivered):          # replay to the cursor
            next(gen, None)
        if self.prefetch <= 0:
            self._gen = gen
            return
        q, stop = queue.Queue(maxsize=self.prefetch), threading.Event()
        self._q, self._stop = q, stop

        def offer(item) -> bool:                 # a full queue must not hold the thread after the loader moved on
            while not stop.is_set():
                try:
                    q.put(item, timeout=0.2)
                    return True
                except queue.Full:
                    continue
            return False

        def work():
            try:
                for b in gen:
                    if not offer(b):
                        return
                offer(StopIteration)
            except Exception as e:  # noqa: BLE001
                offer(e)
        self._thread = threading.Thread(target=work, daemon=True)
        self._thread.start()

    def _halt(self) -> None:
        """Ends the prefetch thread of the current stream (a restored cursor or a closed loader starts a new one)."""
        if getattr(self, "_stop", None) is not None:
            self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        self._q = self._gen = self._thread = None

    def close(self) -> None:
        self._halt()

    def __iter__(self):
        return self

    def __next__(self):
        if self._q is None and self._gen is None:
            self._start()
        if self._gen is not None:
            b = next(self._gen, None)
            if b is None:
                raise DataloaderExhaustedError("text data exhausted")
        else:
            b = self._q.get()
            if b is StopIteration:
                raise DataloaderExhaustedError("text data exhausted")
            if isinstance(b, Exception):
                raise b
        self.delivered += 1
        return b

    def state_dict(self):
        return {"delivered": self.delivered, "dp_degree": self.dp_degree, "rows": self.rows, "seq_len": self.seq_len,
                "identity": self.identity}

    def load_state_dict(self, sd):
        require_same_dp_degree(int(sd["dp_degree"]), self.dp_degree)
        if sd.get("identity") != self.identity:
            raise ConfigError("the data cursor belongs to a different corpus / tokenizer / packing setup")
        if int(sd["rows"]) != self.rows or int(sd["seq_len"]) != self.seq_len:
            raise ConfigError("batch layout changed since the data cursor was saved")
        self.delivered = int(sd["delivered"])
        self._halt()


def build_text_dataloader(data_cfg, *, vocab_size, seq_len, seed, dp_rank, dp_degree, rows_per_rank, pin_memory=False, split="train"):
    tok = build_tokenizer(data_cfg)
    if tok.vocab_size > vocab_size:
        raise ConfigError(f"tokenizer vocabulary {tok.vocab_size} exceeds the model vocabulary {vocab_size}")
    src = build_source(data_cfg, split)
    if data_cfg.dataset in ("local_jsonl_sft", "local_jsonl_sft_multiturn"):
        proc = ChatProcessor(tok, data_cfg.prompt_field, data_cfg.response_field, data_cfg.messages_field,
                             multiturn=data_cfg.dataset.endswith("multiturn") or data_cfg.chat_renderer is not None,
                             template_kwargs=data_cfg.chat_template_kwargs)
    else:
        proc = TextProcessor(tok, data_cfg.text_field)
    ident = corpus_data_identity(data_cfg, tok.identity(), getattr(src, "paths", ()))
    policy = DatasetIterationPolicy(shuffle=data_cfg.shuffle, seed=seed, repeat=split == "train")
    return TextDataLoader(SingleDataset(src, proc), TextCollator(seq_len, pin_memory), seq_len=seq_len, rows_per_rank=rows_per_rank,
                          dp_rank=dp_rank, dp_degree=dp_degree, policy=policy, packing=data_cfg.packing,
                          num_bins=data_cfg.num_packing_bins, max_num_documents=data_cfg.max_num_documents,
                          pad_id=tok.pad_id or 0, identity=ident, prefetch=data_cfg.num_prefetch_batches)
