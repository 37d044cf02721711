"""The allocation-free linear forward (ls_mxfp4_linear_noalloc) against the
regular two-call path, through the C ABI.

Some callers cannot allocate device memory at call time: a plugin living
inside a host application's fixed memory plan, or a loop where the implicit
device synchronisation of an allocation is not acceptable.  For them the
library keeps the temporaries of the linear forward in an array inside its own
image.  This test calls that entry point twice in a row with different shapes
and data (the array keeps the previous call's bytes, which must not leak into
the next result) and holds each output to the existing entry points' output
bit for bit.  It is collected last so that a failure here cannot hide another
test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(fp4, mg, x, w_pk, w_sf, dt):
    p, sf = fp4.quantize_mxfp4_packed(x)
    return mg.mxfp4_gemm_packed(p, w_pk, sf, w_sf, out_dtype=dt)


def _noalloc(L, x, w_pk, w_sf, N, dt):
    from lockstep_b200._lib import check, dtype_code, ptr, stream
    M, K = x.shape
    c = torch.full((M, N), float("nan"), device="cuda", dtype=dt)
    status = torch.full((1,), 7, device="cuda", dtype=torch.int32)
    check(L.ls_mxfp4_linear_noalloc(ptr(x), dtype_code(x.dtype), ptr(w_pk), ptr(w_sf), ptr(c), dtype_code(dt),
                                    M, N, K, ptr(status), stream()))
    assert int(status.item()) == 0
    return c


def test_no_alloc_linear_matches_regular_path_twice():
    from lockstep_b200 import fp4, mxfp4_gemm as mg
    from lockstep_b200._lib import lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(5)
    cases = [(300, 520, 1024, torch.bfloat16, torch.bfloat16), (130, 256, 384, torch.float32, torch.float32)]
    for M, N, K, xdt, odt in cases:                      # two calls in a row, second one smaller
        x = torch.randn(M, K, device="cuda", generator=g).to(xdt)
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
        w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
        want = _regular(fp4, mg, x, w_pk, w_sf, odt)
        mem_before = torch.cuda.memory_allocated()
        got = _noalloc(L, x, w_pk, w_sf, N, odt)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (M, N, K)
        # only the output and the status word came from the caller's allocator
        assert torch.cuda.memory_allocated() - mem_before <= got.numel() * got.element_size() + 1024
    mg.gemm_status()


def test_no_alloc_linear_rejects_oversize():
    from lockstep_b200._lib import lib
    L = lib()
    x = torch.zeros(8, device="cuda")
    rc = L.ls_mxfp4_linear_noalloc(ctypes.c_void_p(x.data_ptr()), 1, ctypes.c_void_p(x.data_ptr()),
                                   ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 1,
                                   8192, 256, 4096, None, None)        # 2^25 elements > 2^24
    assert rc == -1
    assert b"at most" in L.ls_last_error()
