"""CPU restatement of lockstep's NVFP4 format rules.  Test infrastructure only.

NVFP4 = blocks of 16 E2M1 values under one E4M3 scale.  lockstep states the
rules in rig_sm75/quant_sim.cuh and applies them per block in
rig_sm75/rig_q.cu:348-363 (a host-side simulation; there is no kernel).  Each
function below cites the lines it follows.  numpy, float32 arithmetic
throughout, as the C code computes in `float`.

Pinned against the reference's own header compiled here (oracle/_ref, built by
`make -C oracle ref`) through the golden vectors tests/golden/nvfp4_*.npz.
"""

import numpy as np

E4M3_MAX = np.float32(448.0)
E4M3_MIN_SUB = np.float32(2.0 ** -9)
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def quant_e4m3(x):
    """quant_sim.cuh:20-33: round-half-even onto E4M3 (bias 7, subnormals at 2^-9), saturating at
    448; zero gives 0.  (A NaN passes the `!(x != 0.f)` test and comes out as NaN; the block
    maximum that reaches this function is never NaN.)"""
    x = np.asarray(x, np.float32)
    a = np.abs(x)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(a, dtype=np.float32))
    e = np.where(np.isfinite(e), e, 0).astype(np.int32)
    e = np.maximum(e, -6)
    step = np.ldexp(np.float32(1.0), e - 3).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        r = (np.rint(a / step) * step).astype(np.float32)
    r = np.minimum(r, E4M3_MAX)
    r = np.where(a >= E4M3_MAX, E4M3_MAX, r)
    r = np.where(x < 0, -r, r)                                              # s * r: a negative input that rounds to 0 gives -0.0
    r = np.where(a < E4M3_MIN_SUB * np.float32(0.5), np.float32(0), r)     # the early `return 0.f`
    return np.where(x != 0, r, np.float32(0)).astype(np.float32)


def nv_scale(amax):
    """quant_sim.cuh:93-97: E4M3(amax / 6), 2^-9 where that is 0, 1.0 without a positive maximum."""
    amax = np.asarray(amax, np.float32)
    with np.errstate(invalid="ignore"):
        s = quant_e4m3(amax / np.float32(6.0))
    s = np.where(s > 0, s, E4M3_MIN_SUB)
    return np.where(amax > 0, s, np.float32(1.0)).astype(np.float32)


def e2m1_code(x):
    """quant_sim.cuh:57-69: first candidate with the strictly smallest |a - m|, i.e. nearest with
    ties to the smaller magnitude; NaN and infinite inputs never beat candidate 0."""
    x = np.asarray(x, np.float32)
    a = np.abs(x)
    with np.errstate(invalid="ignore"):
        d = np.abs(a[..., None] - E2M1)                # inf - m = inf, NaN stays NaN
    best = np.zeros(a.shape, np.int64)
    bd = d[..., 0].copy()
    for i in range(1, 8):
        with np.errstate(invalid="ignore"):
            take = d[..., i] < bd
        best = np.where(take, i, best)
        bd = np.where(take, d[..., i], bd)
    with np.errstate(invalid="ignore"):
        neg = x < 0
    return (best | np.where(neg, 8, 0)).astype(np.uint8)


def block_amax(xb):
    """rig_q.cu:351-352: std::max(amax, fabsf(v)) from 0 -- a NaN never replaces the running maximum."""
    a = np.abs(xb)
    return np.max(np.where(np.isnan(a), np.float32(0), a), axis=-1).astype(np.float32)


def quantize(x):
    """rig_q.cu:348-363 for F_NVFP4.  x [..., K] float32, K % 16 == 0.
    Returns (codes uint8 [..., K], scale float32 [..., K // 16])."""
    x = np.ascontiguousarray(x, np.float32)
    *lead, K = x.shape
    xb = x.reshape(*lead, K // 16, 16)
    s = nv_scale(block_amax(xb))
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        q = (xb / s[..., None]).astype(np.float32)
    return e2m1_code(q).reshape(*lead, K), s


def e4m3_byte(s):
    """E4M3 byte of a positive E4M3-representable value."""
    s = np.asarray(s, np.float32)
    m, e = np.frexp(s)                                  # s = m * 2^e, m in [0.5, 1)
    be = e - 1 + 7                                      # biased exponent of the normal form
    normal = be >= 1
    mant = np.where(normal, np.rint((m * 2 - 1) * 8), np.rint(s / E4M3_MIN_SUB)).astype(np.int64)
    return np.where(normal, (be << 3) | mant, mant).astype(np.uint8)


def dequantize(codes, scale):
    """rig_q.cu:361: e2m1_value(code) * s."""
    v = np.where(codes & 8, -E2M1[codes & 7], E2M1[codes & 7]).astype(np.float32)
    *lead, K = v.shape
    return (v.reshape(*lead, K // 16, 16) * scale[..., None]).reshape(*lead, K).astype(np.float32)


def pack(codes):
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)
