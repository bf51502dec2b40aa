"""Host-side work description for the variable-length attention kernels.

`AttnMeta.build(cu_seqlens_q, ...)` cuts the packed rows into 128-row tiles per document and produces the two
int32 tile tables that the forward / dQ kernels (q tiles) and the dK/dV kernel (k tiles) consume. It is built
once per batch (the cuts come from the data loader on the host) and reused by every layer.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

TILE = 128


@dataclass
class AttnMeta:
    cu_q: torch.Tensor            # int32 [n+1] host
    cu_k: torch.Tensor            # int32 [n+1] host
    q_offsets: list[int]          # position of each document's first query among its keys
    causal: bool
    q_tiles: torch.Tensor | None  # int32 [nq_tiles, 8] on the compute device (heaviest tiles first)
    k_tiles: torch.Tensor | None  # int32 [nk_tiles, 8]
    total_q: int
    total_k: int
    max_seqlen: int

    @classmethod
    def build(cls, cu_seqlens_q, cu_seqlens_k=None, q_offsets=None, causal: bool = True, device=None) -> "AttnMeta":
        cq = torch.as_tensor(cu_seqlens_q, dtype=torch.int32).cpu()
        ck = cq if cu_seqlens_k is None else torch.as_tensor(cu_seqlens_k, dtype=torch.int32).cpu()
        lq, lk = cq.tolist(), ck.tolist()
        n = len(lq) - 1
        if q_offsets is None:
            offs = [(lk[i + 1] - lk[i]) - (lq[i + 1] - lq[i]) for i in range(n)]
        else:
            offs = [int(x) for x in q_offsets]
        qt, kt = [], []
        for i in range(n):
            qs, qe, ks, ke = lq[i], lq[i + 1], lk[i], lk[i + 1]
            qlen, klen, off = qe - qs, ke - ks, offs[i]
            for a in range(0, qlen, TILE):
                nq = min(TILE, qlen - a)
                diag0 = max(0, min(klen, a + off + 1)) if causal else klen
                work = min(klen, diag0 + nq - 1) if causal else klen
                qt.append((work, [qs + a, nq, ks, klen, diag0, 0, 0, 0]))
            for b in range(0, klen, TILE):
                nk = min(TILE, klen - b)
                work = (qlen - max(0, b - off)) if causal else qlen
                kt.append((work, [ks + b, nk, b, qs, qlen, off, klen, 0]))
        qt.sort(key=lambda t: -t[0])
        kt.sort(key=lambda t: -t[0])
        dev = torch.device(device) if device is not None else None
        mk = (lambda rows: torch.tensor([r[1] for r in rows], dtype=torch.int32).reshape(-1, 8).to(dev)) if dev is not None and dev.type == "cuda" else (lambda rows: None)
        maxlen = max([lq[i + 1] - lq[i] for i in range(n)] + [lk[i + 1] - lk[i] for i in range(n)] + [0])
        return cls(cq, ck, offs, causal, mk(qt), mk(kt), lq[-1], lk[-1], maxlen)

    @classmethod
    def uniform(cls, batch: int, seqlen: int, causal: bool = True, device=None) -> "AttnMeta":
        return cls.build(torch.arange(0, (batch + 1) * seqlen, seqlen, dtype=torch.int32), causal=causal, device=device)
