"""Plain PyTorch fp32-math statements of every hot op.

These are the CPU path and the numerical oracle for the sm_100a kernels: each CUDA kernel test
compares against the function of the same name here (reference for the op set:
llmtuner/kernel/cpu/basic.py:1-96, llmtuner/models/qwen/ops.py:80-131,503,
llmtuner/components/loss.py:35-70). Everything is differentiable through autograd.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.linear(x, w)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """(norm(x + residual), x + residual): the residual stream stays in the input dtype."""
    s = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(s, weight, eps), s


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype=torch.float32):
    """cos/sin of shape [T, head_dim/2] for half-rotation RoPE."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x [T, H, d] fp32; cos/sin [T, d/2]; half rotation: (x1, x2) -> (x1 c - x2 s, x2 c + x1 s)
    d2 = x.shape[-1] // 2
    x1, x2 = x[..., :d2], x[..., d2:]
    c, s = cos.float()[:, None, :], sin.float()[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps: float):
    """Per-head RMSNorm over head_dim (skipped when the weight is None) followed by half-rotation RoPE.
    q [T, Hq, d], k [T, Hkv, d]."""
    def one(x, w):
        xf = x.float()
        if w is not None:
            xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        return _rope(xf, cos, sin).to(x.dtype)
    return one(q, q_weight), one(k, k_weight)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    g = gate.float()
    return (g * torch.sigmoid(g) * up.float()).to(gate.dtype)


def attention_pieces(q, k, v, pieces, causal: bool = True, scale: float | None = None):
    """GQA attention over explicit pieces (q0, qlen, k0, klen, off): query i of a piece sees keys
    [0, min(klen, i + off + 1)) of that piece when causal. q [Tq, Hq, d], k [Tk, Hkv, d], v [Tk, Hkv, dv].
    Returns (out [Tq, Hq, dv], lse [Hq, Tq] fp32)."""
    Tq, Hq, d = q.shape
    g = Hq // k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    d = v.shape[-1]                                        # the output takes the values' width
    outs = torch.zeros(Tq, Hq, d, dtype=torch.float32, device=q.device)
    lses = torch.full((Hq, Tq), float("-inf"), dtype=torch.float32, device=q.device)
    rows_o, rows_i = [], []
    for (q0, qlen, k0, klen, off) in pieces:
        if qlen == 0:
            continue
        qi = q[q0:q0 + qlen].float().transpose(0, 1)
        ki = k[k0:k0 + klen].float().transpose(0, 1).repeat_interleave(g, 0)
        vi = v[k0:k0 + klen].float().transpose(0, 1).repeat_interleave(g, 0)
        s = torch.matmul(qi, ki.transpose(1, 2)) * scale
        if causal:
            qpos = torch.arange(qlen, device=q.device)[:, None] + off
            kpos = torch.arange(klen, device=q.device)[None, :]
            s = s.masked_fill(kpos > qpos, float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.nan_to_num(torch.exp(s - l.unsqueeze(-1)), nan=0.0)
        rows_o.append(torch.matmul(p, vi).transpose(0, 1))
        rows_i.append((q0, qlen, l))
    # assemble without in-place writes so that autograd flows
    order = sorted(range(len(rows_i)), key=lambda t: rows_i[t][0])
    chunks, pos = [], 0
    for t in order:
        q0, qlen, l = rows_i[t]
        if q0 > pos:
            chunks.append(torch.zeros(q0 - pos, Hq, d, dtype=torch.float32, device=q.device))
        chunks.append(rows_o[t])
        lses[:, q0:q0 + qlen] = l.detach()
        pos = q0 + qlen
    if pos < Tq:
        chunks.append(torch.zeros(Tq - pos, Hq, d, dtype=torch.float32, device=q.device))
    out = torch.cat(chunks, 0) if chunks else outs
    return out.to(q.dtype), lses


def _bmm_fp32(a, b):
    """Batched product with an fp32 result: 16-bit inputs on the device keep the tensor cores' fp32 accumulator instead of
    rounding the result to 16 bits first."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16):
        return torch.bmm(a, b, out_dtype=torch.float32)
    return torch.bmm(a, b).float()


def _rows_probs(s, l, n, diag, scale, causal, dtype):
    """P = exp(S * scale - lse) with the causal limit, as tensor expressions (in place on `s`)."""
    l = torch.where(torch.isinf(l), torch.zeros_like(l), l).unsqueeze(-1)       # rows that see no key; masked below
    p = s.mul_(scale).sub_(l).exp_()
    if causal:
        C = p.shape[-1]
        kd = max(0, diag + 1)                                                    # columns below kd are visible to every row
        if kd < C:
            hidden = torch.arange(kd, C, device=p.device)[None, :] > (torch.arange(n, device=p.device) + diag)[:, None]
            p[:, :, kd:].masked_fill_(hidden.repeat(p.shape[1] // n, 1)[None], 0.0)
    return p.to(dtype)


def _rows_ds(dp, p, dl):
    return dp.sub_(dl.unsqueeze(-1)).mul_(p).to(p.dtype)


def attention_backward_rows(q, k, v, o, do, lse, pieces, causal: bool = True, scale: float | None = None, q_chunk: int = 512,
                            probs_fn=None, ds_fn=None):
    """Gradients of `attention_pieces` from its saved output and log-sum-exp, without the [Tq, Tk] probabilities ever
    existing at once: per piece and per chunk of query rows, P = exp(S - lse) is rebuilt, then dV += P^T dO,
    dS = P * (dO V^T - rowsum(dO * O)), dQ = dS K, dK += dS^T Q. The products run in the inputs' dtype (tensor cores
    for bf16) with fp32 results, the key/value accumulators are fp32. Query heads of one key/value group are stacked
    along the row axis, so no head is ever repeated in memory. This is the backward of the head sizes for which the
    device has a forward kernel only; there `probs_fn(s, lse_rows, n, diag, scale, causal)` and `ds_fn(dp, p, delta_rows)`
    are one-pass kernels, here they default to tensor expressions. Returns (dq, dk, dv) in the inputs' dtype."""
    Tq, Hq, d = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    probs_fn = probs_fn or (lambda s, l, n, diag, sc, ca: _rows_probs(s, l, n, diag, sc, ca, q.dtype))
    ds_fn = ds_fn or _rows_ds
    dq = torch.zeros(Tq, Hq, d, dtype=q.dtype, device=q.device)
    dk = torch.zeros(Tk, Hkv, d, dtype=torch.float32, device=q.device)
    dv = torch.zeros(Tk, Hkv, d, dtype=torch.float32, device=q.device)
    delta = (o.float() * do.float()).sum(-1)                                    # [Tq, Hq]
    for (q0, qlen, k0, klen, off) in pieces:
        for a in range(0, qlen, q_chunk):
            n = min(q_chunk, qlen - a)
            kend = min(klen, a + n + off) if causal else klen                    # keys the chunk's last row sees
            if kend <= 0:
                continue
            rows = slice(q0 + a, q0 + a + n)
            keys = slice(k0, k0 + kend)
            qg = q[rows].transpose(0, 1).reshape(Hkv, g * n, d)                 # heads of a group stacked along rows
            dog = do[rows].transpose(0, 1).reshape(Hkv, g * n, d).to(q.dtype)
            ki, vi = k[keys].transpose(0, 1), v[keys].transpose(0, 1)           # [Hkv, kend, d]
            l = lse[:, rows].reshape(Hkv, g * n).contiguous()
            dl = delta[rows].transpose(0, 1).reshape(Hkv, g * n).contiguous()
            p = probs_fn(_bmm_fp32(qg, ki.transpose(1, 2)), l, n, a + off, scale, causal)       # [Hkv, g*n, kend]
            dv[keys] += _bmm_fp32(p.transpose(1, 2), dog).transpose(0, 1)
            ds = ds_fn(_bmm_fp32(dog, vi.transpose(1, 2)), p, dl)                # the softmax scale goes on the outputs
            dq[rows] = _bmm_fp32(ds, ki).mul_(scale).reshape(Hq, n, d).transpose(0, 1).to(q.dtype)
            dk[keys] += _bmm_fp32(ds.transpose(1, 2), qg).mul_(scale).transpose(0, 1)
    return dq, dk.to(k.dtype), dv.to(v.dtype)


def attention(q, k, v, cu_seqlens=None, causal: bool = True, scale: float | None = None, k_cu_seqlens=None, q_offsets=None):
    """Packed-row attention from cumulative document cuts (see `attention_pieces`)."""
    Tq = q.shape[0]
    if cu_seqlens is None:
        cu_seqlens = torch.tensor([0, Tq])
    cq = torch.as_tensor(cu_seqlens).tolist()
    ck = cq if k_cu_seqlens is None else torch.as_tensor(k_cu_seqlens).tolist()
    pieces = []
    for i in range(len(cq) - 1):
        qlen, klen = cq[i + 1] - cq[i], ck[i + 1] - ck[i]
        off = (klen - qlen) if q_offsets is None else int(q_offsets[i])
        pieces.append((cq[i], qlen, ck[i], klen, off))
    return attention_pieces(q, k, v, pieces, causal, scale)


def cross_entropy_sum(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Sum (not mean) of token cross-entropies in fp32; targets == IGNORE_INDEX are skipped."""
    return F.cross_entropy(logits.float(), targets, ignore_index=IGNORE_INDEX, reduction="sum")


def linear_cross_entropy_sum(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, num_chunks: int = 1):
    """Head projection + summed CE without ever holding more than one chunk of logits."""
    total = h.new_zeros((), dtype=torch.float32)
    n = max(1, num_chunks)
    step = -(-h.shape[0] // n)
    for s in range(0, h.shape[0], step):
        total = total + cross_entropy_sum(F.linear(h[s:s + step], w), targets[s:s + step])
    return total


def router_scores(logits: torch.Tensor, score_fn: str) -> torch.Tensor:
    lf = logits.float()
    if score_fn == "softmax":
        return torch.softmax(lf, dim=-1)
    if score_fn == "sigmoid":
        return torch.sigmoid(lf)
    if score_fn == "sqrtsoftplus":
        return torch.sqrt(F.softplus(lf))
    raise ValueError(score_fn)


def router_topk(logits, bias, top_k: int, score_fn: str = "softmax", renorm: bool = True, route_scale: float = 1.0):
    """scores = f(logits); selection on scores (+bias, which never enters the weights); weights are the
    selected scores, optionally renormalised. Returns (weights [T,k] fp32, indices [T,k] int64,
    counts [E] fp32)."""
    scores = router_scores(logits, score_fn)
    sel = scores if bias is None else scores + bias.float()[None, :]
    idx = torch.topk(sel, top_k, dim=-1, sorted=True).indices
    w = scores.gather(-1, idx)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    w = w * route_scale
    counts = torch.zeros(logits.shape[-1], dtype=torch.float32, device=logits.device)
    counts.scatter_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=logits.device))
    return w, idx, counts


def moe_permute(x: torch.Tensor, indices: torch.Tensor, num_experts: int):
    """Sort the T*k token copies by expert (stable). Returns (rows [T*k, D], order [T*k] int64 =
    flat copy index of each sorted row, tokens_per_expert [E] int64)."""
    flat = indices.reshape(-1)
    order = torch.argsort(flat, stable=True)
    rows = x.index_select(0, order // indices.shape[1])
    counts = torch.bincount(flat, minlength=num_experts)
    return rows, order, counts


def moe_unpermute_combine(y: torch.Tensor, order: torch.Tensor, weights: torch.Tensor, num_tokens: int):
    """out[t] = sum_j weights[t, j] * y[row of copy (t, j)], accumulated in fp32."""
    k = weights.shape[1]
    w_sorted = weights.reshape(-1).index_select(0, order).float()
    out = torch.zeros(num_tokens, y.shape[1], dtype=torch.float32, device=y.device)
    out.index_add_(0, order // k, y.float() * w_sorted[:, None])
    return out.to(y.dtype)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Rows of `x` are grouped by expert (counts[e] consecutive rows each); y_e = x_e @ w[e].T with
    w [E, N, K]."""
    outs, s = [], 0
    for e, c in enumerate(counts.tolist()):
        outs.append(F.linear(x[s:s + c], w[e]))
        s += c
    return torch.cat(outs, 0) if outs else x.new_zeros(0, w.shape[1])


def adamw_step_(p_master, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                p_lowp=None, decoupled: bool = True):
    """One AdamW (or Adam when not `decoupled`) update on fp32 master weights; writes the low-precision
    copy when given."""
    g = grad.float() * grad_scale
    if not decoupled and weight_decay:
        g = g + weight_decay * p_master
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    if decoupled and weight_decay:
        p_master.mul_(1 - lr * weight_decay)
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    p_master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if p_lowp is not None:
        p_lowp.copy_(p_master)


def sq_norm(tensors) -> torch.Tensor:
    acc = None
    for t in tensors:
        v = t.float().pow(2).sum()
        acc = v if acc is None else acc + v
    return acc if acc is not None else torch.zeros(())
