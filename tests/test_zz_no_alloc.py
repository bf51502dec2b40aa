"""The allocation-free RMSNorm backward, reached through its exported C symbol the way a caller without an allocator
would reach it (raw device pointers and a stream), must agree with the regular entry point that gets its scratch
from torch. Two calls in a row share the library's built-in scratch array, so the second call (different data,
different shape) also proves that leftovers of the first do not leak into the result."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from torchllmtuner_b200.ops.cuda_ext import load, so_path
    load()                                    # makes sure the extension (and libtorch) is loaded
    lib = ctypes.CDLL(so_path())
    fn = lib.llmt_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.llmt_noalloc_last_error.restype = ctypes.c_char_p
    lib.llmt_noalloc_scratch_bytes.restype = ctypes.c_size_t
    return lib


def _case(T, D, seed, with_dres):
    from torchllmtuner_b200.ops.cuda_ext import load
    ext = load()
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    dy = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).bfloat16()
    dres = torch.randn(T, D, device="cuda", generator=g).bfloat16() if with_dres else None
    _, rstd = ext.rmsnorm_fwd(x, None, w, 1e-6)
    dx_ref, dw_ref = ext.rmsnorm_bwd(dy, x, w, rstd, dres)          # existing entry point (scratch from torch)
    return x, dy, w, rstd, dres, dx_ref, dw_ref


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    torch.cuda.set_device(0)
    assert lib.llmt_noalloc_scratch_bytes() == 296 * 8192 * 4
    stream = torch.cuda.current_stream().cuda_stream
    for T, D, seed, with_dres in ((777, 4096, 1, False), (130, 1024, 2, True)):
        x, dy, w, rstd, dres, dx_ref, dw_ref = _case(T, D, seed, with_dres)
        dx = torch.empty_like(x)
        dw = torch.empty(D, device="cuda", dtype=torch.float32)
        rc = lib.llmt_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                          dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(), T, D,
                                          ctypes.c_void_p(stream))
        assert rc == 0, lib.llmt_noalloc_last_error()
        torch.cuda.synchronize()
        # same kernels, same launch geometry, same order of additions: the two entry points agree bit for bit
        assert torch.equal(dx, dx_ref)
        assert torch.equal(dw, dw_ref.float()) or torch.equal(dw.to(dw_ref.dtype), dw_ref)
        # and both agree with the fp32 statement of the op within the tolerance of the other kernel tests
        from tolerances import ELEMENTWISE, REDUCED, assert_close, f32_leaves
        from torchllmtuner_b200.ops import reference as ref
        xf, wf = f32_leaves(x.requires_grad_(), w.requires_grad_())
        y = ref.rms_norm(xf, wf, 1e-6)
        gx, gw = torch.autograd.grad(y, [xf, wf], dy.float())
        if dres is not None:
            gx = gx + dres.float()
        assert_close(dx, gx, name="dx", **ELEMENTWISE)
        assert_close(dw, gw, name="dw", **REDUCED)


def test_noalloc_rejects_rows_wider_than_the_scratch():
    lib = _lib()
    torch.cuda.set_device(0)
    rc = lib.llmt_rmsnorm_bwd_noalloc(None, None, None, None, None, None, None, 8, 8192 + 8, None)
    assert rc == -10
    assert b"exceeds" in lib.llmt_noalloc_last_error()
