"""The allocation-free linear forward (ls_mxfp4_linear_noalloc) through the C ABI.

Some callers cannot allocate device memory at call time: a plugin living
inside a host application's fixed memory plan, or a loop where the implicit
device synchronisation of an allocation is not acceptable.  For them the
library keeps the temporaries of the linear forward in an array inside its own
image.  This test calls that entry point several times in a row with different
shapes and data (the array keeps the previous call's bytes, which must not
leak into the next result) and holds each output

* to the existing two-call path (ls_quantize_mxfp4 + ls_mxfp4_gemm) bit for bit,
* to the CPU oracle's dequantize + fp32 matmul within the GEMM tolerance
  (rel-L2 <= 1e-3, max-abs <= 2e-2 * ||row||_inf, same output type),

and checks with the driver's own count of free device memory that a call takes
none: an allocation made inside the library would not show in torch's
allocator statistics, but it does lower cudaMemGetInfo's free bytes.  The cases
cover both GEMM kernels (M <= 128: one CTA per tile; M > 128: CTA pairs).
It is collected last so that a failure here cannot hide another test.
"""

import ctypes

import pytest
import torch

from oracle import ref_port

pytestmark = pytest.mark.gpu

CASES = [(300, 520, 1024, torch.bfloat16, torch.bfloat16), (130, 256, 384, torch.float32, torch.float32),
         (96, 384, 512, torch.bfloat16, torch.bfloat16), (16, 136, 256, torch.bfloat16, torch.float32)]


def _regular(fp4, mg, x, w_pk, w_sf, dt):
    p, sf = fp4.quantize_mxfp4_packed(x)
    return mg.mxfp4_gemm_packed(p, w_pk, sf, w_sf, out_dtype=dt)


def _noalloc(L, x, w_pk, w_sf, c, status):
    from lockstep_b200._lib import check, dtype_code, ptr, stream
    M, K = x.shape
    check(L.ls_mxfp4_linear_noalloc(ptr(x), dtype_code(x.dtype), ptr(w_pk), ptr(w_sf), ptr(c), dtype_code(c.dtype),
                                    M, c.shape[1], K, ptr(status), stream()))


def test_no_alloc_linear_matches_regular_path_and_oracle():
    from lockstep_b200 import fp4, mxfp4_gemm as mg
    from lockstep_b200._lib import lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(5)
    prepared = []
    for M, N, K, xdt, odt in CASES:
        x = torch.randn(M, K, device="cuda", generator=g).to(xdt)
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
        w_pk, w_sf = fp4.quantize_mxfp4_packed(w)
        want = _regular(fp4, mg, x, w_pk, w_sf, odt)
        xc, xs = ref_port.quantize(x.cpu())
        wc, ws = ref_port.quantize(w.cpu())
        oracle = ref_port.gemm_fake_quant(xc, xs, wc, ws, odt)
        c = torch.full((M, N), float("nan"), device="cuda", dtype=odt)
        status = torch.full((1,), 7, device="cuda", dtype=torch.int32)
        prepared.append((x, w_pk, w_sf, c, status, want, oracle))
    # warm-up call: the first call on a device looks the array's address up and loads the kernels
    _noalloc(L, *prepared[0][:5])
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for rounds in range(2):                                  # the whole sequence twice, back to back
        for x, w_pk, w_sf, c, status, want, oracle in prepared:
            c.fill_(float("nan"))
            status.fill_(7)
            _noalloc(L, x, w_pk, w_sf, c, status)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before, f"device memory was taken during the calls: {free_before - free_after} bytes"
    for (M, N, K, _, _), (x, w_pk, w_sf, c, status, want, oracle) in zip(CASES, prepared):
        c.fill_(float("nan"))
        _noalloc(L, x, w_pk, w_sf, c, status)
        assert int(status.item()) == 0
        assert torch.equal(c, want), (M, N, K)
        got, ref = c.float().cpu(), oracle.float()
        rel = ((got - ref).norm() / ref.norm()).item()
        worst = ((got - ref).abs() / ref.abs().amax(1, keepdim=True)).max().item()
        assert rel <= 1e-3 and worst <= 2e-2, (M, N, K, rel, worst)
    mg.gemm_status()


def test_no_alloc_linear_rejects_bad_sizes():
    from lockstep_b200._lib import lib
    L = lib()
    x = torch.zeros(8, device="cuda")
    p = ctypes.c_void_p(x.data_ptr())
    rc = L.ls_mxfp4_linear_noalloc(p, 1, p, p, p, 1, 8192, 256, 4096, None, None)        # 2^25 elements > 2^24
    assert rc == -1 and b"at most" in L.ls_last_error()
    rc = L.ls_mxfp4_linear_noalloc(p, 1, p, p, p, 1, 1 << 62, 256, 1 << 20, None, None)  # M * K overflows int64
    assert rc == -1 and b"at most" in L.ls_last_error()
    rc = L.ls_mxfp4_linear_noalloc(p, 1, p, p, p, 1, -1, 256, 128, None, None)
    assert rc == -1 and b"negative" in L.ls_last_error()
    rc = L.ls_mxfp4_linear_noalloc(p, 1, p, p, p, 1, 8, 256, 100, None, None)
    assert rc == -1 and b"multiple of 128" in L.ls_last_error()
