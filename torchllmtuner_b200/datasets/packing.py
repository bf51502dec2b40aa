"""Sequence packing (reference: llmtuner/datasets/packing/build.py:37-153, iterators.py:22-312).

  concat_then_split   documents are concatenated into a token stream and cut every `seq_len` tokens; a document that
                      crosses a cut is split (its continuation restarts positions at 0 and is a document of its own for
                      the attention mask; the last token before the cut still predicts the first one after it);
                      `max_num_documents` caps the documents per row (the row is then padded).
  first_fit           documents (truncated to seq_len) go into the first of `num_bins` open rows with room; a row is
                      emitted when no open row fits the next document; rows are padded.
Each packed row carries tokens, shifted labels (no loss across document borders or on padding), per-document positions
and the document cut points from which the attention kernels build their block-causal masks."""
from __future__ import annotations

from dataclasses import dataclass, field

from .contracts import IGNORE_INDEX, TextSequence


@dataclass
class PackedRow:
    tokens: list[int] = field(default_factory=list)
    labels: list[int] = field(default_factory=list)
    positions: list[int] = field(default_factory=list)
    cuts: list[int] = field(default_factory=lambda: [0])     # document boundaries inside the row

    def room(self, seq_len: int) -> int:
        return seq_len - len(self.tokens)

    def add(self, seq: TextSequence, start: int, n: int) -> None:
        self.tokens += seq.tokens[start:start + n]
        lab = seq.labels[start:start + n]
        if start + n >= len(seq.tokens):
            lab[-1:] = [IGNORE_INDEX]          # nothing is predicted across a document border
        # a document cut by the end of the row keeps its last target: the token that opens its continuation in the next
        # row (reference: llmtuner/datasets/packing/iterators.py:178, labels are sliced as they are)
        self.labels += lab
        self.positions += list(range(n))
        self.cuts.append(len(self.tokens))

    def finish(self, seq_len: int, pad_id: int) -> "PackedRow":
        pad = seq_len - len(self.tokens)
        if pad > 0:
            self.tokens += [pad_id] * pad
            self.labels += [IGNORE_INDEX] * pad
            self.positions += list(range(pad))
            self.cuts.append(seq_len)
        return self


def concat_then_split(seqs, seq_len: int, pad_id: int = 0, max_num_documents: int | None = None):
    row = PackedRow()
    for seq in seqs:
        start, total = 0, len(seq.tokens)
        while start < total:
            if max_num_documents is not None and len(row.cuts) - 1 >= max_num_documents:
                yield row.finish(seq_len, pad_id)
                row = PackedRow()
            n = min(row.room(seq_len), total - start)
            row.add(seq, start, n)
            start += n
            if row.room(seq_len) == 0:
                yield row
                row = PackedRow()
    if row.tokens:
        yield row.finish(seq_len, pad_id)


def first_fit(seqs, seq_len: int, pad_id: int = 0, num_bins: int = 8):
    bins: list[PackedRow] = []
    for seq in seqs:
        n = min(len(seq.tokens), seq_len)
        if n == 0:
            continue
        target = next((b for b in bins if b.room(seq_len) >= n), None)
        if target is None:
            if len(bins) >= num_bins:
                fullest = min(range(len(bins)), key=lambda i: bins[i].room(seq_len))
                yield bins.pop(fullest).finish(seq_len, pad_id)
            target = PackedRow()
            bins.append(target)
        target.add(seq, 0, n)
        if target.room(seq_len) == 0:
            bins.remove(target)
            yield target
    for b in bins:
        yield b.finish(seq_len, pad_id)
