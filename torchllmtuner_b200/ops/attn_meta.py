"""Host-side work description for the variable-length attention kernels.

Work is a list of *pieces* `(q0, qlen, k0, klen, off)`: query rows `q0..q0+qlen` attend key rows `k0..k0+klen`, and
query i of the piece sees keys `[0, min(klen, i + off + 1))` when causal. A plain packed batch has one piece per
document (`off = klen - qlen`); context-parallel shards have one piece per (document, local span) with explicit
offsets, and pieces may then share keys. `AttnMeta` cuts the pieces into 128-row tiles and produces the int32 tile
tables the kernels consume: q tiles for the forward and dQ kernels, k tiles for the dK/dV kernel. Pieces that share
keys are spread over several k-tile passes (the dK/dV kernel accumulates from the second pass on). The tables are
built once per batch (the cuts come from the data loader on the host) and reused by every layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

TILE = 128


@dataclass
class AttnMeta:
    pieces: list[tuple[int, int, int, int, int]]
    causal: bool
    q_tiles: torch.Tensor | None          # int32 [nq_tiles, 8] on the compute device (heaviest first)
    k_tile_passes: list[torch.Tensor] = field(default_factory=list)   # int32 [n, 8] per pass
    total_q: int = 0
    total_k: int = 0
    covers_all_keys: bool = True

    @property
    def k_tiles(self):
        return self.k_tile_passes[0] if self.k_tile_passes else None

    # cu_seqlens views kept for the CPU statement of plain batches
    @property
    def cu_q(self):
        return torch.tensor([p[0] for p in self.pieces] + [self.total_q], dtype=torch.int32)

    @classmethod
    def from_pieces(cls, pieces, total_q: int, total_k: int, causal: bool = True, device=None) -> "AttnMeta":
        pieces = [tuple(int(x) for x in p) for p in pieces if p[1] > 0]
        qt, passes, occupied = [], [], []
        covered = 0
        for (q0, qlen, k0, klen, off) in pieces:
            for a in range(0, qlen, TILE):
                nq = min(TILE, qlen - a)
                diag0 = max(0, min(klen, a + off + 1)) if causal else klen
                work = min(klen, diag0 + nq - 1) if causal else klen
                qt.append((work, [q0 + a, nq, k0, klen, diag0, 0, 0, 0]))
            # keys beyond the last query's reach get no gradient from this piece
            kuse = min(klen, qlen + off) if causal else klen
            pi = 0
            while True:
                if pi == len(occupied):
                    occupied.append([])
                    passes.append([])
                if all(k0 + kuse <= s or k0 >= e for s, e in occupied[pi]):
                    break
                pi += 1
            occupied[pi].append((k0, k0 + kuse))
            if pi == 0:
                covered += kuse
            for b in range(0, kuse, TILE):
                nk = min(TILE, kuse - b)
                work = (qlen - max(0, b - off)) if causal else qlen
                passes[pi].append((work, [k0 + b, nk, b, q0, qlen, off, klen, 0]))
        qt.sort(key=lambda t: -t[0])
        dev = torch.device(device) if device is not None else None
        on_dev = dev is not None and dev.type == "cuda"

        def mk(rows):
            rows = sorted(rows, key=lambda t: -t[0])
            return torch.tensor([r[1] for r in rows], dtype=torch.int32).reshape(-1, 8).to(dev)
        return cls(pieces, causal, mk(qt) if on_dev else None, [mk(p) for p in passes] if on_dev else [], total_q, total_k,
                   covered >= total_k and len(passes) <= 1)

    @classmethod
    def build(cls, cu_seqlens_q, cu_seqlens_k=None, q_offsets=None, causal: bool = True, device=None) -> "AttnMeta":
        lq = torch.as_tensor(cu_seqlens_q, dtype=torch.int64).tolist()
        lk = lq if cu_seqlens_k is None else torch.as_tensor(cu_seqlens_k, dtype=torch.int64).tolist()
        n = len(lq) - 1
        pieces = []
        for i in range(n):
            qlen, klen = lq[i + 1] - lq[i], lk[i + 1] - lk[i]
            off = (klen - qlen) if q_offsets is None else int(q_offsets[i])
            pieces.append((lq[i], qlen, lk[i], klen, off))
        return cls.from_pieces(pieces, lq[-1], lk[-1], causal, device)

    @classmethod
    def uniform(cls, batch: int, seqlen: int, causal: bool = True, device=None) -> "AttnMeta":
        return cls.build(torch.arange(0, (batch + 1) * seqlen, seqlen), causal=causal, device=device)
