"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the call site (a fixed memory
budget, a latency-critical path, a binding that only passes raw pointers), so they cannot provide
the scratch matrix the regular entry point asks for. ``pb_rmsnorm_bwd_noalloc`` keeps that scratch
in a static device array inside the library. This test drives it exactly the way such a caller
would — ctypes on the shared object, raw pointers, no helper from the Python package on the call
path — and checks it against the regular entry point twice in a row, because the static scratch
keeps the previous call's contents and the second call must not be affected by them.

The file name sorts last on purpose: if this addition ever breaks, every other test has already run.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from prime_b200 import _build
    lib = C.CDLL(str(_build.build_cuda()))
    vp, i32 = C.c_void_p, C.c_int
    lib.pb_rmsnorm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.pb_rmsnorm_bwd_noalloc.restype = C.c_int
    lib.pb_noalloc_strerror.argtypes = [i32]
    lib.pb_noalloc_strerror.restype = C.c_char_p
    return lib


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_matches_regular_entry_point_twice():
    from prime_b200.ops import kernels as ops
    lib = _lib()
    torch.manual_seed(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (M, N) in enumerate([(3000, 1024), (777, 512)]):   # second call: different shape, stale scratch from the first
        x = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(N, device="cuda")).bfloat16()
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        dres = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        _, rstd = ops.rmsnorm_fwd(x, w, 1e-5)
        dw_ref = torch.zeros(N, device="cuda", dtype=torch.float32)
        dx_ref = ops.rmsnorm_bwd(x, w, rstd, dy, dw_ref, dres=dres, accumulate_dw=False)
        dx = torch.empty_like(x)
        dw = torch.full((N,), 123.0, device="cuda", dtype=torch.float32)   # overwritten, not accumulated
        before = torch.cuda.memory_allocated()
        rc = lib.pb_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr(), dx.data_ptr(),
                                        dw.data_ptr(), 1, 0, M, N, stream)
        assert rc == 0, lib.pb_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel(dx, dx_ref) < 1e-2, f"call {call}: dx"
        assert _rel(dw, dw_ref) < 1e-3, f"call {call}: dw"
        # and against the fp32 PyTorch twin of the op on the CPU, so this test stands on its own
        dw_cpu = torch.zeros(N, dtype=torch.float32)
        dx_cpu = ops.rmsnorm_bwd(x.cpu(), w.cpu(), rstd.cpu(), dy.cpu(), dw_cpu, dres=dres.cpu(), accumulate_dw=False)
        assert _rel(dx.cpu(), dx_cpu) < 1e-2 and _rel(dw.cpu(), dw_cpu) < 1e-2, f"call {call}: CPU twin"


def test_noalloc_rejects_rows_wider_than_the_builtin_scratch():
    lib = _lib()
    t = torch.zeros(8, device="cuda")
    p = t.data_ptr()
    rc = lib.pb_rmsnorm_bwd_noalloc(p, p, p, p, None, p, p, 1, 0, 16, 2048, None)
    assert rc == -3 and b"PB_NOALLOC_MAX_N" in lib.pb_noalloc_strerror(rc)
    assert lib.pb_rmsnorm_bwd_noalloc(p, p, p, p, None, p, p, 1, 0, 16, 300, None) == -1
