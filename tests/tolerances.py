"""Element-wise comparison of a bf16 kernel result with its fp32 PyTorch statement.

`assert_close(out, ref, rtol, atol_rms)` requires, for EVERY element, |out - ref| <= atol_rms * rms(ref) + rtol * |ref|.
The absolute part scales with the root-mean-square of the reference, not with its maximum, so an error confined to
small-magnitude entries (a wrong masked column, a dropped tail block of one row) fails even when the large entries are
right. Bounds by kernel class (bf16 has 8 bits of mantissa, one rounding = 2^-9 relative):

  GEMM_BF16      one rounding of an fp32 accumulator                      rtol 2^-7, atol 1e-3 rms
  GEMM_F32       fp32 accumulation order only                             rtol 1e-5, atol 1e-4 rms
  ELEMENTWISE    fp32 math, one output rounding, inputs rounded once       rtol 2^-6, atol 4e-3 rms
  REDUCED        sums of many bf16-rounded terms (weight gradients)        rtol 2^-6, atol 1e-2 rms
  ATTENTION      probabilities rounded to bf16 before the P V product       rtol 2e-2, atol 3e-2 rms
  ATTENTION_GRAD P and dS rounded to bf16, delta = rowsum(dO * O) from the      rtol 2e-2, atol 1.2e-1 rms
                 bf16-rounded output: rows with few visible keys cancel
                 (dP - delta) to a few percent of the gradient's rms

The fp32 statement must itself be exact to fp32: give it fp32 LEAF copies of the inputs (a `.float()` inside the graph of
a bf16 leaf rounds every gradient contribution to bf16 before they are summed).
"""
import torch

GEMM_BF16 = dict(rtol=2.0 ** -7, atol_rms=1e-3)
GEMM_F32 = dict(rtol=1e-5, atol_rms=1e-4)
ELEMENTWISE = dict(rtol=2.0 ** -6, atol_rms=4e-3)
REDUCED = dict(rtol=2.0 ** -6, atol_rms=1e-2)
ATTENTION = dict(rtol=2e-2, atol_rms=3e-2)
ATTENTION_GRAD = dict(rtol=2e-2, atol_rms=1.2e-1)


def f32_leaves(*tensors):
    """fp32 leaf copies (None passes through) for the reference arm of a gradient comparison."""
    return [None if t is None else t.detach().float().requires_grad_(t.requires_grad) for t in tensors]


def assert_close(out, ref, rtol, atol_rms, name="tensor"):
    out, ref = out.detach().float(), ref.detach().float().to(out.device)
    assert out.shape == ref.shape, f"{name}: shape {tuple(out.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(out).all(), f"{name}: non-finite values"
    rms = ref.pow(2).mean().sqrt().item()
    bound = atol_rms * rms + rtol * ref.abs()
    excess = (out - ref).abs() - bound
    worst = excess.max().item()
    if worst > 0:
        idx = tuple(int(i) for i in torch.unravel_index(excess.argmax(), excess.shape))
        raise AssertionError(f"{name}: element {idx} is {out[idx].item():.6g}, reference {ref[idx].item():.6g} "
                             f"(bound {bound[idx].item():.3g}, rms {rms:.3g}); {(excess > 0).sum().item()} elements out of bound")
