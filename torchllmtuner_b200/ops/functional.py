"""Autograd-aware hot ops. CUDA tensors run the hand-written sm_100a kernels (`csrc/*.cu`); CPU tensors run the
plain PyTorch statements in `reference.py`, which are also the numerical oracle of the kernel tests.
There is no library fallback on CUDA: if the extension cannot be loaded the call raises.
"""
from __future__ import annotations

import math
import os

import torch

from . import reference as ref
from ..errors import UnsupportedCombinationError
from .validation import validate_attention_inputs, validate_rms_norm_inputs
from .attn_meta import AttnMeta
from .cuda_ext import load as _ext

IGNORE_INDEX = ref.IGNORE_INDEX


def _comm_queue():
    from ..parallel import symm
    return symm._ACTIVE


def _use_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _2d(t: torch.Tensor) -> torch.Tensor:
    t = t.reshape(-1, t.shape[-1])
    return t if t.stride(-1) == 1 else t.contiguous()


# ----------------------------------------------------------------------------------------------- per-op checkpointing
class SelectiveReplay:
    """Per-op activation checkpointing of one block frame (reference policy: llmtuner/memory/activation_checkpoint.py:203-256).

    The block's first forward runs without a graph in `record` mode and its replay inside backward in `replay` mode. Ops
    the policy keeps store their output while recording and hand it back while replaying, so the replay only rebuilds the
    autograd node (inputs saved, nothing computed); every other op is recomputed. Policy: attention is kept; linears are
    kept except every second one (counted in call order, restarted per frame so that record and replay agree); a linear
    whose weight shape is in `recompute_mm_shapes` is always recomputed and not counted."""

    def __init__(self, recompute_mm_shapes=()):
        self.recompute_mm_shapes = {tuple(s) for s in recompute_mm_shapes}
        self.store: list = []
        self.mode = "record"
        self.mm_count = 0
        self.cursor = 0
        self.kept_bytes = 0

    def begin(self, mode: str) -> None:
        self.mode, self.mm_count, self.cursor = mode, 0, 0

    def keeps_linear(self, w: torch.Tensor) -> bool:
        if tuple(w.shape) in self.recompute_mm_shapes:
            return False
        self.mm_count += 1
        return self.mm_count % 2 == 1

    def put(self, value) -> None:
        self.store.append(value)
        for t in (value if isinstance(value, tuple) else (value,)):
            self.kept_bytes += t.numel() * t.element_size()

    def take(self):
        v = self.store[self.cursor]
        self.cursor += 1
        return v


_SAC: SelectiveReplay | None = None


class sac_frame:
    """Context manager that makes `frame` the active per-op checkpoint frame in `mode` ("record" / "replay")."""

    def __init__(self, frame: SelectiveReplay | None, mode: str):
        self.frame, self.mode = frame, mode

    def __enter__(self):
        global _SAC
        self.prev = _SAC
        _SAC = self.frame
        if self.frame is not None:
            self.frame.begin(self.mode)
        return self.frame

    def __exit__(self, *exc):
        global _SAC
        _SAC = self.prev
        return False


# ----------------------------------------------------------------------------------------------- GEMM
def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, accumulate=False, max_ctas=0):
    """out[M,N] (+)= op(a) @ op(b)^T-style product on the tcgen05 kernel.
    a_mn=False: a is [M,K]; a_mn=True: a is stored [K,M]. b_mn=False: b is [N,K]; b_mn=True: b is stored [K,N]."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
    q = _comm_queue()
    if q:                                   # a pending peer-memory collective rides on this kernel's comm warps
        K = a.shape[0] if a_mn else a.shape[1]
        s, callbacks = q.take(2.0 * M * N * K)
        if s is not None:
            ext = _ext()
            from ..parallel.symm import make_side_job
            ext.gemm(a, b, out, a_mn, b_mn, accumulate, 0, make_side_job(ext, s))
            for cb in callbacks:
                cb()
            return out
    _ext().gemm(a, b, out, a_mn, b_mn, accumulate, max_ctas)
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, y_kept=None):
        x2 = _2d(x)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        if y_kept is not None:              # replay of a kept op: only the graph node is rebuilt
            return y_kept.view(*x.shape[:-1], w.shape[0])
        return gemm(x2, w).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.xshape)                      # dy [M,N] @ W [N,K]
        if ctx.needs_input_grad[1]:
            main = getattr(w, "main_grad", None)
            if main is not None:                                                   # accumulate straight into the owner's buffer
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main, accumulate=getattr(w, "main_grad_initialized", False))
                w.main_grad_initialized = True
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)        # dy^T [N,M] @ x [M,K]
        return dx, dw, None


class _KeptLinear(torch.autograd.Function):
    """Replay of a kept linear off the kernel path (CPU, odd shapes): returns the kept output, backward is the linear's."""

    @staticmethod
    def forward(ctx, x, w, y_kept):
        ctx.save_for_backward(x, w)
        return y_kept.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        return (dy2 @ w.to(dy2.dtype)).reshape(x.shape), (dy2.t() @ x2).to(w.dtype), None


class _MultiLinear(torch.autograd.Function):
    """y_i = x W_i^T for several weights that read the same rows (q / k / v, gate / up). The input gradient is summed by the
    GEMM epilogues themselves (dx = dy_0 W_0, then dx += dy_i W_i with the accumulating epilogue) instead of by one
    elementwise addition per extra consumer, which autograd would otherwise insert."""

    @staticmethod
    def forward(ctx, x, *ws):
        x2 = _2d(x)
        ctx.save_for_backward(x2, *ws)
        ctx.xshape = x.shape
        return tuple(gemm(x2, w).reshape(*x.shape[:-1], w.shape[0]) for w in ws)

    @staticmethod
    def backward(ctx, *dys):
        x2, *ws = ctx.saved_tensors
        dx = None
        if ctx.needs_input_grad[0]:
            for dy, w in zip(dys, ws):
                if dy is None:
                    continue
                if dx is None:
                    dx = gemm(_2d(dy), w, b_mn=True)
                else:
                    gemm(_2d(dy), w, b_mn=True, out=dx, accumulate=True)
            dx = None if dx is None else dx.reshape(ctx.xshape)
        dws = []
        for i, (dy, w) in enumerate(zip(dys, ws)):
            if dy is None or not ctx.needs_input_grad[1 + i]:
                dws.append(None)
                continue
            main = getattr(w, "main_grad", None)
            if main is not None:
                gemm(_2d(dy), x2, a_mn=True, b_mn=True, out=main, accumulate=getattr(w, "main_grad_initialized", False))
                w.main_grad_initialized = True
                dws.append(None)
            else:
                dws.append(gemm(_2d(dy), x2, a_mn=True, b_mn=True, out_dtype=w.dtype))
        return (dx, *dws)


def linears(x: torch.Tensor, *ws: torch.Tensor):
    """Several bias-free projections of the same rows; one autograd node on the kernel path, plain `linear` calls elsewhere
    (CPU, odd shapes, and under per-op checkpointing, whose keep / replay bookkeeping is per projection)."""
    if (_SAC is None and _use_cuda(x) and x.dtype == torch.bfloat16 and len(ws) > 1
            and not any(w.shape[0] % 8 or w.shape[1] % 8 for w in ws)):
        return _MultiLinear.apply(x, *ws)
    return tuple(linear(x, w) for w in ws)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    # a TMA row must start on a 16-byte boundary: projections with fewer than 8 (or an odd number of) features, e.g. one
    # gate value per head, cannot be tiled by the tcgen05 kernel and take the plain library product
    kernel = _use_cuda(x) and x.dtype == torch.bfloat16 and not (w.shape[0] % 8 or w.shape[1] % 8)
    frame = _SAC
    if frame is not None and frame.keeps_linear(w):
        if frame.mode == "record":
            y = _Linear.apply(x, w) if kernel else ref.linear(x, w)
            frame.put(y.detach())
            return y
        kept = frame.take()
        return _Linear.apply(x, w, kept) if kernel else _KeptLinear.apply(x, w, kept)
    return _Linear.apply(x, w) if kernel else ref.linear(x, w)


# ----------------------------------------------------------------------------------------------- RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xc = _c(x)
        y, rstd = _ext().rmsnorm_fwd(xc, None, w, eps)
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _ext().rmsnorm_bwd(_c(dy), x, w, rstd, None)
        return dx, dw.to(w.dtype), None


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, eps):
        y, rstd, s = _ext().rmsnorm_fwd(_c(x), _c(res), w, eps)
        ctx.save_for_backward(s, w, rstd)
        return y, s

    @staticmethod
    def backward(ctx, dy, ds):
        s, w, rstd = ctx.saved_tensors
        dsum, dw = _ext().rmsnorm_bwd(_c(dy), s, w, rstd, _c(ds) if ds is not None else None)
        return dsum, dsum, dw.to(w.dtype), None


def rms_norm(x, weight, eps: float):
    validate_rms_norm_inputs(x, weight)
    if _use_cuda(x) and x.dtype == torch.bfloat16:
        return _RMSNorm.apply(x, weight, eps)
    return ref.rms_norm(x, weight, eps)


def add_rms_norm(x, residual, weight, eps: float):
    """Returns (rms_norm(x + residual), x + residual) with one pass over the data."""
    if _use_cuda(x) and x.dtype == torch.bfloat16:
        return _AddRMSNorm.apply(x, residual, weight, eps)
    return ref.add_rms_norm(x, residual, weight, eps)


# ----------------------------------------------------------------------------------------------- QK-norm + RoPE
rope_tables = ref.rope_tables


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cos, sin, eps):
        y, rstd = _ext().qk_norm_rope_fwd(x, w, cos, sin, eps)
        ctx.save_for_backward(x, w if w is not None else torch.empty(0), cos, sin, rstd)
        ctx.has_w = w is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, cos, sin, rstd = ctx.saved_tensors
        if dy.stride(2) != 1 or dy.stride(1) != dy.shape[2]:
            dy = dy.contiguous()
        out = _ext().qk_norm_rope_bwd(dy, x, w if ctx.has_w else None, cos, sin, rstd)
        return out[0], (out[1].to(w.dtype) if ctx.has_w else None), None, None, None


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps: float):
    """q [T,Hq,d], k [T,Hkv,d] (views with packed heads are fine); cos/sin fp32 [T,d/2]."""
    if _use_cuda(q) and q.dtype == torch.bfloat16:
        return _QKNormRope.apply(q, q_weight, cos, sin, eps), _QKNormRope.apply(k, k_weight, cos, sin, eps)
    return ref.qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps)


# ----------------------------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, row_limit):
        g2, u2 = _2d(gate), _2d(up)
        if g2.stride(0) != u2.stride(0):
            g2, u2 = g2.contiguous(), u2.contiguous()
        ctx.save_for_backward(g2, u2)
        ctx.shape, ctx.row_limit = gate.shape, row_limit
        return _ext().swiglu_fwd(g2, u2, row_limit).reshape(gate.shape)

    @staticmethod
    def backward(ctx, dout):
        g2, u2 = ctx.saved_tensors
        d2 = _2d(dout)
        both = torch.empty(g2.shape[0], 2 * g2.shape[1], dtype=g2.dtype, device=g2.device)
        dg, du = both[:, :g2.shape[1]], both[:, g2.shape[1]:]
        _ext().swiglu_bwd(d2, g2, u2, dg, du, ctx.row_limit)
        return dg.reshape(ctx.shape), du.reshape(ctx.shape), None


def swiglu(gate, up, row_limit=None):
    """silu(gate) * up. `row_limit` (int32 device scalar) bounds the rows that are touched when the operands are
    statically sized buffers whose live row count is only known on the device (expert-parallel receive buffers)."""
    if _use_cuda(gate) and gate.dtype == torch.bfloat16:
        return _SwiGLU.apply(gate, up, row_limit)
    return ref.swiglu(gate, up)


# ----------------------------------------------------------------------------------------------- attention
DEVICE_ATTENTION_HEAD_DIMS = (64, 128, 256)     # 256: forward kernel, backward rebuilt per chunk of rows from the LSE


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta: AttnMeta, scale, kept=None):
        o, lse = kept if kept is not None else _ext().attn_fwd(q, k, v, meta.q_tiles, scale, meta.causal, attention_forward_mode() == "pair")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta, ctx.scale = meta, scale
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse=None):
        q, k, v, o, lse = ctx.saved_tensors
        if do.stride(2) != 1 or do.stride(1) != do.shape[2]:
            do = do.contiguous()
        m = ctx.meta
        if q.shape[-1] not in (64, 128):      # forward kernel only at this head size: rebuild P per chunk of rows from the LSE
            ext = _ext()
            dq, dk, dv = ref.attention_backward_rows(q, k, v, o, do, lse, m.pieces, m.causal, ctx.scale,
                                                     probs_fn=ext.attn_rows_probs, ds_fn=ext.attn_rows_ds)
            return dq, dk, dv, None, None, None
        dq, dk, dv = _ext().attn_bwd(q, k, v, o, do, lse, m.q_tiles, m.k_tile_passes, ctx.scale, m.causal, not m.covers_all_keys,
                                     attention_backward_mode() == "fused")
        return dq, dk, dv, None, None, None


def attention_forward_mode() -> str:
    """"single" (default): one head per CTA. "pair" (`LLMT_ATTN_FWD=pair`): one CTA serves two query heads of a key/value
    group, K/V tiles are loaded once for both and P stays in tensor memory; needs an even group size."""
    return "pair" if os.environ.get("LLMT_ATTN_FWD") == "pair" else "single"


_ATTN_BWD_MODE: str | None = None


def set_attention_backward(mode: str | None) -> None:
    """Choose the attention backward: "fused" (one kernel per key tile, five products, dQ summed in an fp32 accumulator by
    bulk reduce-adds: fastest, dQ reproducible up to fp32 summation order) or "split" (a dK/dV kernel and a dQ kernel,
    seven products, bitwise reproducible). `None` returns to the default: the environment variable `LLMT_ATTN_BWD`, else
    "split" when `torch.use_deterministic_algorithms(True)` is in force, else "fused"."""
    global _ATTN_BWD_MODE
    if mode not in (None, "fused", "split"):
        raise ValueError(f"attention backward mode must be 'fused' or 'split', got {mode!r}")
    _ATTN_BWD_MODE = mode


def attention_backward_mode() -> str:
    if _ATTN_BWD_MODE is not None:
        return _ATTN_BWD_MODE
    env = os.environ.get("LLMT_ATTN_BWD")
    if env in ("fused", "split"):
        return env
    return "split" if torch.are_deterministic_algorithms_enabled() else "fused"


def device_head_dim(d: int) -> int | None:
    """The head size the device kernels run a head of width `d` at (the next supported size), None beyond the largest."""
    return next((s for s in DEVICE_ATTENTION_HEAD_DIMS if s >= d), None)


def attention(q, k, v, meta: AttnMeta, scale: float | None = None):
    """Packed-row GQA attention; documents and masks come from `meta`. q [Tq,Hq,d], k [Tk,Hkv,d], v [Tk,Hkv,dv]
    -> [Tq,Hq,dv]. On the device a head width the kernels have no variant for (72, 192, a value width that differs from
    the key width) is zero-padded to the next one they have: the padded columns add nothing to Q K^T and their outputs are
    cut away again, so only the products grow."""
    validate_attention_inputs(q, k, v)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _use_cuda(q) and q.dtype == torch.bfloat16:
        d, dv = q.shape[-1], v.shape[-1]
        run = device_head_dim(max(d, dv))
        if run is None:
            raise UnsupportedCombinationError(f"attention head width {max(d, dv)} exceeds the device kernels' largest ({DEVICE_ATTENTION_HEAD_DIMS[-1]})")
        if d != run or dv != run:
            pad = torch.nn.functional.pad
            out = attention(pad(q, (0, run - d)), pad(k, (0, run - d)), pad(v, (0, run - dv)), meta, scale)
            return out[..., :dv]
        if meta.q_tiles is None:
            raise ValueError("AttnMeta was built without device tables; pass device= to AttnMeta.build")
        frame = _SAC
        if frame is None:
            return _Attention.apply(q, k, v, meta, scale)[0]
        if frame.mode == "record":                       # attention is always kept by the per-op policy
            o, lse = _Attention.apply(q, k, v, meta, scale)
            frame.put((o.detach(), lse.detach()))
            return o
        return _Attention.apply(q, k, v, meta, scale, frame.take())[0]
    out, _ = ref.attention_pieces(q, k, v, meta.pieces, meta.causal, scale)
    return out


def attention_with_lse(q, k, v, meta: AttnMeta, scale: float | None = None):
    """Forward only, returns (out, lse [Hq, Tq]); used by context-parallel merges."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _use_cuda(q) and q.dtype == torch.bfloat16:
        o, lse = _ext().attn_fwd(q, k, v, meta.q_tiles, scale, meta.causal, attention_forward_mode() == "pair")
        return o, lse
    return ref.attention_pieces(q, k, v, meta.pieces, meta.causal, scale)


# ----------------------------------------------------------------------------------------------- cross-entropy
class _LinearCrossEntropy(torch.autograd.Function):
    """loss_sum = sum_t CE(h_t W^T, y_t), computed chunk by chunk; logits of a chunk are overwritten in place by their
    gradient, from which dh and dW are accumulated, so that the full [T, V] logits never exist
    (reference: llmtuner/components/loss.py:246-316)."""

    @staticmethod
    def forward(ctx, h, w, targets, num_chunks):
        ext = _ext()
        T, D = h.shape
        n = max(1, int(num_chunks))
        step = -(-T // n)
        step = -(-step // 128) * 128
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(h) if need_dh else None
        dw = torch.zeros(w.shape, dtype=torch.float32, device=w.device) if need_dw else None
        loss = torch.zeros((), dtype=torch.float32, device=h.device)
        first = True
        for s in range(0, T, step):
            hc = h[s:s + step]
            logits = gemm(hc, w)                                                   # [c, V] bf16
            row_loss, _ = ext.ce_fwd_bwd(logits, targets[s:s + step].contiguous(), 1.0, None, IGNORE_INDEX,
                                         need_dh or need_dw)
            loss += row_loss.sum()
            if need_dh:
                gemm(logits, w, b_mn=True, out=dh[s:s + step])                     # dlogits [c,V] @ W [V,D]
            if need_dw:
                gemm(logits, hc, a_mn=True, b_mn=True, out=dw, accumulate=not first)  # dlogits^T @ h
            first = False
        ctx.save_for_backward(dh if dh is not None else torch.empty(0), dw if dw is not None else torch.empty(0))
        ctx.flags = (need_dh, need_dw, w.dtype)
        return loss

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        need_dh, need_dw, wdt = ctx.flags
        return ((dh * g.to(dh.dtype)) if need_dh else None, ((dw * g).to(wdt)) if need_dw else None, None, None)


def linear_cross_entropy_sum(h, w, targets, num_chunks: int = 1):
    if _use_cuda(h) and h.dtype == torch.bfloat16:
        return _LinearCrossEntropy.apply(_2d(h), w, targets.reshape(-1), num_chunks)
    return ref.linear_cross_entropy_sum(h.reshape(-1, h.shape[-1]), w, targets.reshape(-1), num_chunks)


class _CrossEntropySum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        work = logits.clone()
        row_loss, _ = _ext().ce_fwd_bwd(work, targets.contiguous(), 1.0, None, IGNORE_INDEX, True)
        ctx.save_for_backward(work)
        return row_loss.sum()

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g.to(d.dtype), None


def cross_entropy_sum(logits, targets):
    if _use_cuda(logits) and logits.dtype == torch.bfloat16:
        return _CrossEntropySum.apply(_2d(logits), targets.reshape(-1))
    return ref.cross_entropy_sum(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))


# ----------------------------------------------------------------------------------------------- optimizer pieces
def adamw_step_(p_master, grad, exp_avg, exp_avg_sq, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                p_lowp=None, decoupled=True, clip_coef=None):
    if p_master.is_cuda:
        _ext().adamw(p_master, p_lowp, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, clip_coef,
                     grad_scale, decoupled)
        return
    gs = grad_scale * (float(clip_coef) if clip_coef is not None else 1.0)
    if not math.isfinite(gs):
        return          # non-finite gradient norm: leave parameters and moments untouched
    ref.adamw_step_(p_master, grad, exp_avg, exp_avg_sq, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                    weight_decay=weight_decay, step=step, grad_scale=gs, p_lowp=p_lowp, decoupled=decoupled)


_scratch: dict = {}


def sq_norm(tensors, out: torch.Tensor | None = None) -> torch.Tensor:
    """Deterministic sum of squares over a list of tensors, fp32, on the tensors' device (no host sync)."""
    tensors = [t for t in tensors if t is not None and t.numel()]
    if not tensors:
        return torch.zeros((), dtype=torch.float32) if out is None else out.zero_()
    dev = tensors[0].device
    if dev.type != "cuda":
        v = ref.sq_norm(tensors)
        return v if out is None else out.copy_(v)
    ext = _ext()
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    if key not in _scratch:
        _scratch[key] = torch.empty(ext.sqnorm_scratch_floats(), dtype=torch.float32, device=dev)
    acc = torch.zeros(1, dtype=torch.float32, device=dev) if out is None else out.reshape(1)
    for i, t in enumerate(tensors):
        t = t if t.is_contiguous() else t.contiguous()
        if t.dtype not in (torch.float32, torch.bfloat16):
            t = t.float()
        ext.sqnorm(t, _scratch[key], acc, i > 0)
    return acc.reshape(())
