"""Packed MXFP4 GEMM with the API of lockstep's mxfp4_gemm.py, on tcgen05.

`mxfp4_gemm_packed` and `mxfp4_gemm_fp8` keep the reference signatures
(mxfp4_gemm.py:74-87, :161-174).  The reference emulates the block-scaled
product on Hopper FP8 tensor cores through Triton; here one hand-written
sm_100a kernel feeds packed E2M1 operands and UE8M0 block scales straight to
`tcgen05.mma.kind::mxf4.block_scale`, accumulating in tensor memory.

Scales may be given as the reference does (fp32 powers of two, [rows, K//32])
or, to skip a conversion pass, as the uint8 scale-factor buffer that
`fp4.quantize_mxfp4_packed` produces.
"""

import torch

from . import _lib, fp4
from ._lib import aligned, check, lib, need_cuda, ptr, stream

# The reference exports its Triton launch config under this name
# (mxfp4_gemm.py:23); here it documents the fixed tile shape of the kernel.
CFG = dict(BLOCK_M=128, BLOCK_N=256, BLOCK_K=256, num_stages=4, num_warps=6)


def _sf(scale, rows, K, block=32):
    """fp32 [rows, K//block] scales -> scale-factor bytes; uint8 buffers pass through."""
    if scale.dtype == torch.uint8:
        assert scale.numel() == fp4.sf_bytes(rows, K, block), "scale-factor buffer has the wrong size"
        return aligned(scale)
    assert scale.shape == (rows, K // block), f"scale shape {tuple(scale.shape)} != {(rows, K // block)}"
    sf, _bad = fp4.scales_to_sf(scale, block)
    return sf


def mxfp4_gemm_packed(a_pk, bt_pk, a_scale, b_scale, out_dtype=torch.bfloat16, block=32):
    """a_pk [M, K//2] uint8, bt_pk [N, K//2] uint8 (both K-contiguous, even
    index in the low nibble), a_scale [M, K//32], b_scale [N, K//32].
    Returns C = A @ B_T.T as [M, N] of out_dtype (bf16 or fp32).

    (extension) block = 16 takes operands of fp4.quantize_mxfp4(x, 16): scales
    [M, K//16] and [N, K//16].  The reference's GEMM has no such form
    (mxfp4_gemm.py:136 fixes 32 values per scale); on tcgen05 it is the same
    kernel on `kind::mxf4nvf4.block_scale.block16` with UE8M0 scales."""
    need_cuda(a_pk, bt_pk, a_scale, b_scale)
    assert block in (16, 32)
    M, Kh = a_pk.shape
    N, Kh2 = bt_pk.shape
    K = Kh * 2
    assert Kh == Kh2 and K % 128 == 0, "K must be a multiple of 128 (max BLOCK_K)"
    a_pk, bt_pk = aligned(a_pk), aligned(bt_pk)
    sfa, sfb = _sf(a_scale, M, K, block), _sf(b_scale, N, K, block)
    c = torch.empty((M, N), device=a_pk.device, dtype=out_dtype)
    fn = lib().ls_mxfp4_gemm if block == 32 else lib().ls_mxfp4_gemm_block16
    check(fn(ptr(a_pk), ptr(bt_pk), ptr(sfa), ptr(sfb), ptr(c), _lib.dtype_code(out_dtype), M, N, K, stream()))
    return c


def mxfp4_gemm_packed_quant(a_pk, bt_pk, a_scale, b_scale, out_dtype=torch.bfloat16, act=None, want_c=True):
    """(extension) mxfp4_gemm_packed whose epilogue also quantizes act(C) to MXFP4
    for a following GEMM (act: None or "gelu").  Returns (C or None, packed
    [M, N // 2], scale-factor bytes of a [M, N] operand).  N % 128 == 0."""
    need_cuda(a_pk, bt_pk, a_scale, b_scale)
    M, Kh = a_pk.shape
    N, Kh2 = bt_pk.shape
    K = Kh * 2
    assert Kh == Kh2 and K % 128 == 0, "K must be a multiple of 128 (max BLOCK_K)"
    assert N % 128 == 0, "N must be a multiple of 128 for the quantized output"
    a_pk, bt_pk = aligned(a_pk), aligned(bt_pk)
    sfa, sfb = _sf(a_scale, M, K), _sf(b_scale, N, K)
    c = torch.empty((M, N), device=a_pk.device, dtype=out_dtype) if want_c else None
    q = torch.empty((M, N // 2), device=a_pk.device, dtype=torch.uint8)
    q_sf = torch.empty(fp4.sf_bytes(M, N), device=a_pk.device, dtype=torch.uint8)
    check(lib().ls_mxfp4_gemm_quant(ptr(a_pk), ptr(bt_pk), ptr(sfa), ptr(sfb), ptr(c), _lib.dtype_code(out_dtype),
                                    {None: 0, "gelu": 1}[act], ptr(q), ptr(q_sf), M, N, K, stream()))
    return c, q, q_sf


def mxfp4_gemm_fp8(a_fp8, b_fp8, a_scale, b_scale, out_dtype=torch.bfloat16):
    """a_fp8 [M, K] K-contiguous, b_fp8 [K, N] N-contiguous, both E4M3 bytes
    holding E2M1 values; a_scale [M, K//32], b_scale [K//32, N]
    (mxfp4_gemm.py:74-87).  The reference expands FP4 to FP8 because Hopper's
    tensor cores have no FP4 type; here two small kernels re-encode the bytes to
    packed E2M1 (exactly; b is transposed on the way, its scales go straight to
    the scale-factor layout) and the product runs on the MXFP4 tensor-core kernel
    at the FP4 rate.  Nothing synchronises: a byte that is not an E2M1 value is
    reported by `gemm_status()`."""
    need_cuda(a_fp8, b_fp8, a_scale, b_scale)
    M, K = a_fp8.shape
    K2, N = b_fp8.shape
    assert K == K2 and K % 128 == 0, "K must be a multiple of 128 (max BLOCK_K)"
    assert a_scale.shape == (M, K // 32) and b_scale.shape == (K // 32, N)
    a_fp8, b_fp8 = aligned(a_fp8), aligned(b_fp8)
    dev = a_fp8.device
    a_pk = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    b_pk = torch.empty((N, K // 2), dtype=torch.uint8, device=dev)
    check(lib().ls_e4m3_to_packed(ptr(a_fp8), M, K, ptr(a_pk), stream()))
    check(lib().ls_e4m3_to_packed_t(ptr(b_fp8), K, N, ptr(b_pk), stream()))
    sfb = torch.empty(fp4.sf_bytes(N, K), dtype=torch.uint8, device=dev)
    check(lib().ls_scales_to_sf_t(ptr(aligned(b_scale.float())), N, K, ptr(sfb), None, stream()))
    return mxfp4_gemm_packed(a_pk, b_pk, a_scale, sfb, out_dtype)


def gemm_status():
    """Raises if a GEMM kernel launched since the last call gave up on a
    bounded wait (a protocol fault; results are then undefined)."""
    check(lib().ls_gemm_status(None))
