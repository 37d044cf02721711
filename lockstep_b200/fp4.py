"""MXFP4 primitives with the API of lockstep's fp4.py, computed by sm_100a kernels.

Same names, argument meaning and return types as the reference module
(fp4.py:20-125): E2M1 tables, quantize / dequantize, pack / unpack, the fp64
reference GEMM and the exact integer block dot.  Tensors must live on a CUDA
device; there is no CPU path.  Layout conventions are the reference's:
A [M, K] K-contiguous, B_T [N, K] K-contiguous, scales [rows, K // 32].

Additions that the reference does not have are marked "(extension)".
"""

import torch

from . import _lib
from ._lib import aligned, check, lib, need_cuda, ptr, stream

# ---------------------------------------------------------------- E2M1 tables
_E2M1_MAG = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
FP4_MAX = 6.0
FP4_EMAX = 2

E2M1_VALUES = torch.tensor(_E2M1_MAG + [-v for v in _E2M1_MAG], dtype=torch.float32)
_E4M3_POS = [0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C]
E2M1_TO_E4M3 = torch.tensor(_E4M3_POS + [b | 0x80 for b in _E4M3_POS], dtype=torch.uint8)
E2M1_Q = torch.tensor([int(2 * v) for v in E2M1_VALUES.tolist()], dtype=torch.int32)

_ROUNDING = {"ref": 0, "rne": 1}


def random_codes(shape, device="cpu") -> torch.Tensor:
    """Uniform over the 15 distinct E2M1 codes, negative zero excluded (fp4.py:37-40)."""
    pick = torch.tensor([c for c in range(16) if c != 8], device=device, dtype=torch.uint8)
    return pick[torch.randint(0, 15, shape, device=device)]


def _round_to_e2m1(q: torch.Tensor, rounding: str = "ref") -> torch.Tensor:
    """Nearest E2M1 code of each element (fp4.py:43-54).  A value halfway
    between two grid points keeps the smaller magnitude; rounding="rne"
    (extension) sends it to the even code instead."""
    need_cuda(q)
    q = aligned(q.float())
    codes = torch.empty(q.shape, dtype=torch.uint8, device=q.device)
    check(lib().ls_round_e2m1(ptr(q), q.numel(), _ROUNDING[rounding], ptr(codes), stream()))
    return codes


def _as_rows(x, block):
    *lead, K = x.shape
    assert K % block == 0, f"K={K} must be a multiple of block={block}"
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x = aligned(x, 32)                         # the kernels read 32-byte words
    return x, lead, K, (x.numel() // K if K else 0)


def quantize_mxfp4(x: torch.Tensor, block: int = 32, rounding: str = "ref"):
    """MXFP4 quantize along the last dim (fp4.py:57-72).

    Returns (codes uint8 [..., K], scale fp32 [..., K // block]); the scale is
    2^(floor(log2(amax)) - 2), 1.0 for an all-zero block."""
    need_cuda(x)
    x, lead, K, rows = _as_rows(x, block)
    codes = torch.empty((*lead, K), dtype=torch.uint8, device=x.device)
    scale = torch.empty((*lead, K // block), dtype=torch.float32, device=x.device)
    check(lib().ls_quantize_mxfp4(ptr(x), _lib.dtype_code(x.dtype), rows, K, block, _ROUNDING[rounding],
                                  ptr(codes), None, ptr(scale), None, None, stream()))
    return codes, scale


def quantize_mxfp4_packed(x: torch.Tensor, rounding: str = "ref", want_scale: bool = False, block: int = 32):
    """(extension) One pass from bf16/fp32 to what the tensor-core GEMM reads:
    packed nibbles [..., K // 2] and E8M0 scale bytes in the tcgen05
    scale-factor layout (see sf_bytes).  Fuses quantize_mxfp4 + pack_fp4 +
    the scale re-layout.  K must be a multiple of 128.  With want_scale the
    fp32 scales [..., K // block] are returned as a third value.  block = 16
    gives the operands of mxfp4_gemm_packed(..., block=16)."""
    need_cuda(x)
    assert block in (16, 32)
    x, lead, K, rows = _as_rows(x, block)
    assert K % 128 == 0, "K must be a multiple of 128"
    packed = torch.empty((*lead, K // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, K, block), dtype=torch.uint8, device=x.device)
    scale = torch.empty((*lead, K // block), dtype=torch.float32, device=x.device) if want_scale else None
    check(lib().ls_quantize_mxfp4(ptr(x), _lib.dtype_code(x.dtype), rows, K, block, _ROUNDING[rounding],
                                  None, ptr(packed), ptr(scale), None, ptr(sf), stream()))
    return (packed, sf, scale) if want_scale else (packed, sf)


def quantize_mxfp4_packed_t(x: torch.Tensor, rounding: str = "ref", want_scale: bool = False):
    """(extension) quantize_mxfp4_packed(x.t().contiguous()) without the copy:
    x [R, C] -> packed [C, R // 2] and the scale-factor buffer of a [C, R]
    operand, blocks of 32 running down the columns of x.  R % 128 == 0."""
    need_cuda(x)
    assert x.dim() == 2 and x.shape[0] % 128 == 0, "rows must be a multiple of 128"
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x = aligned(x)
    R, C = x.shape
    packed = torch.empty((C, R // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(C, R), dtype=torch.uint8, device=x.device)
    scale = torch.empty((C, R // 32), dtype=torch.float32, device=x.device) if want_scale else None
    check(lib().ls_quantize_mxfp4_t(ptr(x), _lib.dtype_code(x.dtype), R, C, _ROUNDING[rounding],
                                    ptr(packed), ptr(scale), ptr(sf), stream()))
    return (packed, sf, scale) if want_scale else (packed, sf)


def layernorm_quantize(x: torch.Tensor, weight, bias, eps: float = 1e-5):
    """(extension) layer_norm(x) over the last dim, rounded to bf16, and its MXFP4 form in one
    pass.  x [rows, D] fp32 or bf16; returns (y bf16 [rows, D], packed [rows, D // 2], sf,
    mean [rows], rstd [rows]).  D % 256 == 0 and D <= 8192."""
    need_cuda(x)
    assert x.dim() == 2 and x.dtype in (torch.float32, torch.bfloat16)
    rows, D = x.shape
    assert D % 256 == 0 and D <= 8192, "D must be a multiple of 256, at most 8192"
    x = aligned(x)
    w = None if weight is None else aligned(weight.float())
    b = None if bias is None else aligned(bias.float())
    y = torch.empty((rows, D), dtype=torch.bfloat16, device=x.device)
    packed = torch.empty((rows, D // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(rows, D), dtype=torch.uint8, device=x.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    check(lib().ls_layernorm_quantize(ptr(x), _lib.dtype_code(x.dtype), ptr(w), ptr(b), float(eps), rows, D,
                                      ptr(y), ptr(packed), ptr(sf), ptr(mean), ptr(rstd), stream()))
    return y, packed, sf, mean, rstd


def layernorm_backward(g_y: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, rstd: torch.Tensor, weight, want_bias=True):
    """(extension) Backward of layer_norm from the statistics layernorm_quantize kept: returns
    (gx in x's dtype, gweight fp32 [D] or None, gbias fp32 [D] or None).  g_y fp32 or bf16 [rows, D]."""
    need_cuda(g_y, x, mean, rstd)
    rows, D = x.shape
    assert g_y.shape == x.shape and D % 256 == 0 and D <= 8192
    if g_y.dtype not in (torch.float32, torch.bfloat16):
        g_y = g_y.float()
    g_y, x = aligned(g_y), aligned(x)
    w = None if weight is None else aligned(weight.float())
    gx = torch.empty_like(x)
    gw = torch.empty(D, dtype=torch.float32, device=x.device) if weight is not None else None
    gb = torch.empty(D, dtype=torch.float32, device=x.device) if want_bias else None
    scratch = torch.empty(int(lib().ls_layernorm_backward_scratch(rows, D)), dtype=torch.float32, device=x.device)
    check(lib().ls_layernorm_backward(ptr(g_y), _lib.dtype_code(g_y.dtype), ptr(x), _lib.dtype_code(x.dtype), ptr(aligned(mean)),
                                      ptr(aligned(rstd)), ptr(w), rows, D, ptr(gx), ptr(gw), ptr(gb), ptr(scratch), stream()))
    return gx, gw, gb


def quantize_mxfp4_packed_t_gelu(x: torch.Tensor, rounding: str = "ref"):
    """(extension) quantize_mxfp4_packed_t(gelu(x)) for bf16 x [R, C] without the elementwise
    pass: the activation is applied to the tile inside the kernel.  R % 128 == 0."""
    need_cuda(x)
    assert x.dim() == 2 and x.shape[0] % 128 == 0 and x.dtype == torch.bfloat16
    x = aligned(x)
    R, C = x.shape
    packed = torch.empty((C, R // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(C, R), dtype=torch.uint8, device=x.device)
    check(lib().ls_quantize_mxfp4_t_act(ptr(x), _lib.dtype_code(x.dtype), R, C, _ROUNDING[rounding], 1,
                                        ptr(packed), None, ptr(sf), stream()))
    return packed, sf


def quantize_mxfp4_both(x: torch.Tensor, rounding: str = "ref", act=None):
    """(extension) quantize_mxfp4_packed(x) and quantize_mxfp4_packed_t(x) from one read
    of x [R, C]: returns (packed, sf, packed_t, sf_t).  R % 128 == 0 and C % 128 == 0.
    act="gelu" (bf16 x) quantizes gelu(x) instead, without the elementwise pass."""
    need_cuda(x)
    assert x.dim() == 2 and x.shape[0] % 128 == 0 and x.shape[1] % 128 == 0, "both dimensions must be multiples of 128"
    assert act in (None, "gelu") and (act is None or x.dtype == torch.bfloat16)
    if x.dtype not in (torch.float32, torch.bfloat16):
        x = x.float()
    x = aligned(x)
    R, C = x.shape
    packed = torch.empty((R, C // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty(sf_bytes(R, C), dtype=torch.uint8, device=x.device)
    packed_t = torch.empty((C, R // 2), dtype=torch.uint8, device=x.device)
    sf_t = torch.empty(sf_bytes(C, R), dtype=torch.uint8, device=x.device)
    check(lib().ls_quantize_mxfp4_both_act(ptr(x), _lib.dtype_code(x.dtype), R, C, _ROUNDING[rounding], 1 if act else 0,
                                           ptr(packed), ptr(sf), ptr(packed_t), ptr(sf_t), stream()))
    return packed, sf, packed_t, sf_t


def sf_bytes(rows: int, K: int, block: int = 32) -> int:
    """(extension) Size of the scale-factor buffer of a [rows, K] operand."""
    return int(lib().ls_sf_bytes_block(rows, K, block))


def scales_to_sf(scale: torch.Tensor, block: int = 32) -> torch.Tensor:
    """(extension) fp32 power-of-two scales [rows, K // block] -> scale-factor
    layout bytes.  Raises if a scale is not a power of two."""
    need_cuda(scale)
    scale = aligned(scale.float())
    rows, kb = scale.shape
    K = kb * block
    assert K % 128 == 0, "K must be a multiple of 128"
    sf = torch.empty(sf_bytes(rows, K, block), dtype=torch.uint8, device=scale.device)
    bad = torch.zeros(1, dtype=torch.int32, device=scale.device)
    check(lib().ls_scales_to_sf_block(ptr(scale), rows, K, block, ptr(sf), ptr(bad), stream()))
    return sf, bad


def dequantize_mxfp4(codes: torch.Tensor, scale: torch.Tensor, block: int = 32):
    """value[code] * scale (fp4.py:75-78); fp32 out, same shape as codes."""
    need_cuda(codes, scale)
    *lead, K = codes.shape
    assert K % block == 0
    codes = aligned(codes)
    scale = aligned(scale.float())
    out = torch.empty((*lead, K), dtype=torch.float32, device=codes.device)
    rows = codes.numel() // K if K else 0
    check(lib().ls_dequantize_mxfp4(ptr(codes), 0, ptr(scale), None, rows, K, block, ptr(out), 0, stream()))
    return out


def codes_to_e4m3(codes: torch.Tensor) -> torch.Tensor:
    """Lossless FP4 -> FP8 (E4M3) cast by table (fp4.py:81-83)."""
    return E2M1_TO_E4M3.to(codes.device)[codes.long()].view(torch.float8_e4m3fn)


def codes_to_q(codes: torch.Tensor) -> torch.Tensor:
    """FP4 code -> 2 * value as int32, the exact integer grid (fp4.py:86-88)."""
    return E2M1_Q.to(codes.device)[codes.long()]


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] codes -> [..., K // 2] bytes, even index in the low nibble (fp4.py:91-94)."""
    assert codes.shape[-1] % 2 == 0
    need_cuda(codes)
    codes = aligned(codes)
    out = torch.empty((*codes.shape[:-1], codes.shape[-1] // 2), dtype=torch.uint8, device=codes.device)
    check(lib().ls_pack_fp4(ptr(codes), ptr(out), codes.numel(), stream()))
    return out


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of pack_fp4 (fp4.py:97-99)."""
    need_cuda(packed)
    packed = aligned(packed)
    out = torch.empty((*packed.shape[:-1], packed.shape[-1] * 2), dtype=torch.uint8, device=packed.device)
    check(lib().ls_unpack_fp4(ptr(packed), ptr(out), packed.numel(), stream()))
    return out


# ------------------------------------------------------------------ references
def reference_mxfp4_gemm(a_codes, a_scale, b_codes, b_scale, block=32):
    """fp64 check value for C = A @ B with A [M, K], B [K, N] quantized along K
    (fp4.py:103-112).  A verification helper, not a fast path."""
    A = dequantize_mxfp4(a_codes, a_scale, block).double()
    Bt = dequantize_mxfp4(b_codes.t().contiguous(), b_scale.t().contiguous(), block).double()
    return (A @ Bt.t()).float()


def blockwise_exact_dot(qa: torch.Tensor, qb: torch.Tensor, block: int = 32):
    """Exact integer dot products per block from the integer grid (fp4.py:115-125)."""
    p = qa.long() * qb.long()
    *lead, K = p.shape
    return p.reshape(*lead, K // block, block).sum(-1)
