"""Dual-batch GEMM with the API of lockstep's dual_gemm.py.

The reference file is an experiment on whether two FP4 GEMMs can share one
fp32 accumulator (acc = C1 + 2^s * C2); its own conclusion is that they cannot
beyond K ~ 14 and that two activation batches against one shared weight are
"one GEMM with a taller M" (dual_gemm.py:1-15, train_step.py:186-188).  What
the hot path needs from it is that shared-weight case, which
`dual_mxfp4_packed` runs in one launch on packed MXFP4 operands: both batches'
tiles walk the same weight stream back to back, two fp32 accumulators live in
tensor memory.

The reference's own entry points are kept with their signatures.  They take
bf16/fp8 operands without block scales, i.e. they are not MXFP4 work; they
run as fp32-accumulating library matmuls so that callers keep working.
"""

import math

import torch

from . import _lib, fp4, mxfp4_gemm
from ._lib import aligned, check, lib, need_cuda, ptr, stream

CFG = dict(BLOCK_M=128, BLOCK_N=256, BLOCK_K=256, num_stages=4, num_warps=6)


def slot_offset(K: int) -> int:
    """Minimum 2^s separation for a K-deep FP4 dot product (dual_gemm.py:23-25)."""
    return int(math.floor(math.log2(144 * K))) + 2


def unpack_dual(acc: torch.Tensor, s: int):
    """Split acc = C1 + 2^s * C2 back into the two results (dual_gemm.py:28-32)."""
    w = float(2 ** s)
    c2 = torch.round(acc / w)
    return acc - c2 * w, c2


def dual_mxfp4_packed(a1_pk, a2_pk, bt_pk, a1_scale, a2_scale, b_scale, out_dtype=torch.bfloat16, out=None):
    """Two activation batches against one MXFP4 weight in one launch.

    a1_pk, a2_pk [M, K//2] uint8; bt_pk [N, K//2] uint8; scales as in
    mxfp4_gemm.mxfp4_gemm_packed.  Returns (C1, C2), each [M, N]; `out` may
    give the two output tensors (contiguous, 16-byte aligned)."""
    need_cuda(a1_pk, a2_pk, bt_pk)
    M, Kh = a1_pk.shape
    N, Kh2 = bt_pk.shape
    K = Kh * 2
    assert a2_pk.shape == a1_pk.shape and Kh == Kh2 and K % 128 == 0
    a1_pk, a2_pk, bt_pk = aligned(a1_pk), aligned(a2_pk), aligned(bt_pk)
    sfa1, sfa2 = mxfp4_gemm._sf(a1_scale, M, K), mxfp4_gemm._sf(a2_scale, M, K)
    sfb = mxfp4_gemm._sf(b_scale, N, K)
    if out is not None:
        c1, c2 = out
        assert c1.shape == (M, N) and c2.shape == (M, N) and c1.dtype == out_dtype and c2.dtype == out_dtype
        assert c1.is_contiguous() and c2.is_contiguous()
    else:
        c1 = torch.empty((M, N), device=a1_pk.device, dtype=out_dtype)  # two allocations: both 16-byte aligned
        c2 = torch.empty((M, N), device=a1_pk.device, dtype=out_dtype)
    check(lib().ls_mxfp4_gemm_dual(ptr(a1_pk), ptr(a2_pk), ptr(bt_pk), ptr(sfa1), ptr(sfa2), ptr(sfb),
                                   ptr(c1), ptr(c2), _lib.dtype_code(out_dtype), M, N, K, stream()))
    return c1, c2


def dual_mxfp4(x1, x2, w_pk, w_sf, out_dtype=torch.bfloat16):
    """Quantize two bf16/fp32 activation batches on the fly and multiply both
    by a pre-quantized weight (packed bytes + scale-factor buffer).

    When the two batches are the two halves of one allocation (as the
    reference's train_step.py:97-103 lays its microbatches out) and the batch
    height is a multiple of 128, both are quantized by a single launch.
    (Splitting the rows to run the second half's quantizer under the first
    half's GEMM was tried and lost: 236 us against 210 us per step at
    2 x 4096 x 8192 -- two shorter persistent GEMM launches cost more than the
    overlap hides.)"""
    M, K = x1.shape
    adjacent = (x1.is_contiguous() and x2.is_contiguous() and x1.dtype == x2.dtype and x1.shape == x2.shape
                and M % 128 == 0 and x2.data_ptr() == x1.data_ptr() + x1.numel() * x1.element_size()
                and x1.untyped_storage().data_ptr() == x2.untyped_storage().data_ptr())
    if adjacent:
        both = torch.as_strided(x1, (2 * M, K), (K, 1))
        p, sf = fp4.quantize_mxfp4_packed(both)
        half = sf.numel() // 2
        return dual_mxfp4_packed(p[:M], p[M:], w_pk, sf[:half], sf[half:], w_sf, out_dtype)
    p1, s1 = fp4.quantize_mxfp4_packed(x1)
    p2, s2 = fp4.quantize_mxfp4_packed(x2)
    return dual_mxfp4_packed(p1, p2, w_pk, s1, s2, w_sf, out_dtype)


# ---- reference signatures (bf16 / fp8 operands, fp32 out) -------------------
def _mm(a, b):
    need_cuda(a, b)
    return a.float() @ b.float()


def gemm(a, b):
    """Single GEMM, fp32 out. a [M, K], b [K, N] (dual_gemm.py:215-226)."""
    assert a.shape[1] % 64 == 0, "K must be a multiple of 64 (max BLOCK_K); zero-pad if shorter"
    return _mm(a, b)


def dual_packed(a1, a2s, b1, b2):
    """The PACKED fp32 tile C1 + C2s; split with unpack_dual (dual_gemm.py:230-241)."""
    assert a1.shape[1] % 64 == 0, "K must be a multiple of 64 (max BLOCK_K); zero-pad if shorter"
    return _mm(a1, b1) + _mm(a2s, b2)


def dual_separate(a1, a2, b1, b2):
    """(a1 @ b1, a2 @ b2), fp32 (dual_gemm.py:244-255)."""
    assert a1.shape[1] % 64 == 0, "K must be a multiple of 64 (max BLOCK_K); zero-pad if shorter"
    return _mm(a1, b1), _mm(a2, b2)


def splitk_packed(a1, a2s, b1, b2, splits=8, **kw):
    """dual_gemm.py:261-274; the split only changes the summation order."""
    assert a1.shape[1] % (splits * kw.get("BK", 64)) == 0, "K must divide splits*BK"
    return dual_packed(a1, a2s, b1, b2)


def splitk_separate(a1, a2, b1, b2, splits=8, **kw):
    """dual_gemm.py:277-289."""
    assert a1.shape[1] % (splits * kw.get("BK", 64)) == 0, "K must divide splits*BK"
    return dual_separate(a1, a2, b1, b2)
