"""NVFP4 (blocks of 16 E2M1 values under one E4M3 scale) on the tensor cores.

lockstep states this format in its study of block formats
(rig_sm75/quant_sim.cuh:90-97 `nv_scale_e2m1`, :20-33 `quant_e4m3`, :57-69
`quant_e2m1_code`; applied per block in rig_q.cu:348-363) and measures its
accuracy in simulation, but ships no kernel for it.  Here the quantizer follows
those rules bit for bit and the product runs on
`tcgen05.mma.kind::mxf4nvf4.block_scale.block16` with the E4M3 scale bytes.
"""

import torch

from . import _lib, fp4
from ._lib import aligned, check, lib, need_cuda, ptr, stream


def quantize_nvfp4(x: torch.Tensor, want_bytes: bool = False):
    """x [..., K] bf16/fp32, K % 128 == 0 -> (packed uint8 [..., K // 2], scale fp32 [..., K // 16],
    scale-factor bytes for the GEMM[, E4M3 scale bytes [..., K // 16]])."""
    need_cuda(x)
    x, lead, K, rows = fp4._as_rows(x, 16)
    assert K % 128 == 0, "K must be a multiple of 128"
    dev = x.device
    packed = torch.empty((*lead, K // 2), dtype=torch.uint8, device=dev)
    scale = torch.empty((*lead, K // 16), dtype=torch.float32, device=dev)
    sf = torch.empty(fp4.sf_bytes(rows, K, 16), dtype=torch.uint8, device=dev)
    u8 = torch.empty((*lead, K // 16), dtype=torch.uint8, device=dev) if want_bytes else None
    check(lib().ls_quantize_nvfp4(ptr(x), _lib.dtype_code(x.dtype), rows, K, ptr(packed), ptr(u8), ptr(scale), ptr(sf),
                                  stream()))
    return (packed, scale, sf, u8) if want_bytes else (packed, scale, sf)


def dequantize_nvfp4(packed: torch.Tensor, scale_u8: torch.Tensor, out_dtype=torch.float32):
    """value[code] * scale; packed [..., K // 2], scale_u8 [..., K // 16] E4M3 bytes."""
    need_cuda(packed, scale_u8)
    packed, scale_u8 = aligned(packed), aligned(scale_u8)
    *lead, Kh = packed.shape
    K = Kh * 2
    rows = packed.numel() // Kh if Kh else 0
    assert scale_u8.numel() * 16 == packed.numel() * 2
    out = torch.empty((*lead, K), dtype=out_dtype, device=packed.device)
    check(lib().ls_dequantize_nvfp4(ptr(packed), ptr(scale_u8), rows, K, ptr(out), _lib.dtype_code(out_dtype), stream()))
    return out


def nvfp4_gemm_packed(a_pk, bt_pk, a_sf, b_sf, out_dtype=torch.bfloat16):
    """a_pk [M, K // 2], bt_pk [N, K // 2] packed E2M1 (K-contiguous); a_sf, b_sf the scale-factor
    buffers of quantize_nvfp4.  Returns C = A @ B_T.T [M, N] in out_dtype (bf16 or fp32)."""
    need_cuda(a_pk, bt_pk, a_sf, b_sf)
    M, Kh = a_pk.shape
    N, Kh2 = bt_pk.shape
    K = Kh * 2
    assert Kh == Kh2 and K % 128 == 0, "K must be a multiple of 128"
    assert a_sf.dtype == torch.uint8 and a_sf.numel() == fp4.sf_bytes(M, K, 16), "a_sf has the wrong size"
    assert b_sf.dtype == torch.uint8 and b_sf.numel() == fp4.sf_bytes(N, K, 16), "b_sf has the wrong size"
    a_pk, bt_pk, a_sf, b_sf = aligned(a_pk), aligned(bt_pk), aligned(a_sf), aligned(b_sf)
    c = torch.empty((M, N), device=a_pk.device, dtype=out_dtype)
    check(lib().ls_nvfp4_gemm(ptr(a_pk), ptr(bt_pk), ptr(a_sf), ptr(b_sf), ptr(c), _lib.dtype_code(out_dtype),
                              M, N, K, stream()))
    return c


def nvfp4_gemm_dual(a1_pk, a2_pk, bt_pk, a1_sf, a2_sf, b_sf, out_dtype=torch.bfloat16):
    """Two activation batches against one weight in one launch (the NVFP4 form of dual_gemm.dual_mxfp4's GEMM)."""
    need_cuda(a1_pk, a2_pk, bt_pk, a1_sf, a2_sf, b_sf)
    M, Kh = a1_pk.shape
    N, _ = bt_pk.shape
    K = Kh * 2
    assert a2_pk.shape == a1_pk.shape and bt_pk.shape[1] == Kh and K % 128 == 0
    ts = [aligned(t) for t in (a1_pk, a2_pk, bt_pk, a1_sf, a2_sf, b_sf)]
    c1 = torch.empty((M, N), device=a1_pk.device, dtype=out_dtype)
    c2 = torch.empty_like(c1)
    check(lib().ls_nvfp4_gemm_dual(*map(ptr, ts), ptr(c1), ptr(c2), _lib.dtype_code(out_dtype), M, N, K, stream()))
    return c1, c2
