"""CPU oracle: a restatement of lockstep's MXFP4 hot path in torch CPU ops.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file;
only the tests, the smoke check and the CPU-baseline leg of the benchmark do,
and only as the checker or the timed CPU baseline.

Every function names the reference code it restates (paths are relative to
the lockstep project root).  The reference's arithmetic lives in torch's CPU
kernels (log2, floor, exp2, bucketize, sgemm), so this port calls the same
torch ops in the same order: on the same torch build it reproduces the
reference bit for bit, including the fp32 ``log2`` rounding that makes the
block exponent one larger than the mathematical one for maxima a few ulps
below a power of two.  Pinning: ``tests/golden/`` holds outputs of the real
reference modules on seeded inputs; ``tests/test_oracle_golden.py`` holds this
port (and the C restatement in ``mxfp4_ref.c``) to them.

The MXFP4 gradient wire at the end has no counterpart in the reference (its
wire.py offers fp32/bf16/int16/int8ef only): it is the reference's
owner-reduces protocol (wire.py:104-138) with fp4.py's codec substituted for
the integer grid.  Its byte format is pinned by the codec; its protocol is
"parity unpinned".
"""

import torch

E2M1_MAG = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# Decision thresholds between neighbouring magnitudes (fp4.py:50).
E2M1_MID = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
E2M1_E4M3 = (0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C)


def value_table():
    """code -> value, codes 8..15 are the negatives (fp4.py:24)."""
    return torch.tensor(list(E2M1_MAG) + [-m for m in E2M1_MAG], dtype=torch.float32)


def round_e2m1(q, rounding="ref"):
    """fp4.py:43-54.  Nearest E2M1 code; a value exactly between two grid
    points keeps the SMALLER magnitude ("ref", what torch.bucketize's
    right-closed buckets give).  "rne" is the OCP tie rule (even mantissa),
    offered by the product as an option; it has no reference counterpart."""
    mid = torch.tensor(E2M1_MID, dtype=torch.float32)
    a = q.abs().clamp(max=6.0)
    if rounding == "ref":
        idx = torch.bucketize(a, mid)
    else:
        # ties at .25 .75 1.25 1.75 2.5 3.5 5 -> even code: 0,2,2,4,4,6,6
        idx = torch.bucketize(a, mid)
        tie = torch.zeros_like(idx, dtype=torch.bool)
        for m in E2M1_MID:
            tie |= a == m
        idx = torch.where(tie & (idx % 2 == 1), idx + 1, idx)
    return idx.to(torch.uint8) | (torch.signbit(q).to(torch.uint8) << 3)


def quantize(x, block=32, rounding="ref"):
    """fp4.py:57-72.  Returns (codes u8 [..., K], scale f32 [..., K/block])."""
    x = x.float()
    *lead, K = x.shape
    assert K % block == 0
    xb = x.reshape(*lead, K // block, block)
    amax = xb.abs().amax(dim=-1)
    e = torch.floor(torch.log2(amax.clamp(min=1e-30))) - 2
    scale = torch.exp2(e.clamp(-127, 127))
    scale = torch.where(amax == 0, torch.ones_like(scale), scale)
    codes = round_e2m1(xb / scale.unsqueeze(-1), rounding).reshape(*lead, K)
    return codes, scale


def dequantize(codes, scale, block=32):
    """fp4.py:75-78."""
    v = value_table()[codes.long()]
    *lead, K = v.shape
    return (v.reshape(*lead, K // block, block) * scale.unsqueeze(-1)).reshape(*lead, K)


def pack(codes):
    """fp4.py:91-94: even index in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def unpack(packed):
    """fp4.py:97-99."""
    return torch.stack([packed & 0x0F, packed >> 4], dim=-1).reshape(*packed.shape[:-1], -1)


def scale_to_e8m0(scale):
    """Biased exponent byte of a power-of-two fp32 scale (exact; no reference
    counterpart: the reference keeps scales as fp32)."""
    bits = scale.contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF).to(torch.uint8)


def gemm_fake_quant(a_codes, a_scale, w_codes, w_scale, out_dtype=torch.bfloat16):
    """fp4_linear.py:40: F.linear on dequantized operands, fp32, then cast.
    This is the path the reference itself takes on any GPU that is not an
    H100, and the one the GEMM tolerance is stated against."""
    a = dequantize(a_codes, a_scale)
    w = dequantize(w_codes, w_scale)
    return torch.nn.functional.linear(a, w).to(out_dtype)


def gemm_fp64(a_codes, a_scale, w_codes, w_scale):
    """fp4.py:103-112 with B given K-contiguous ([N,K], scales [N,K/32])."""
    a = dequantize(a_codes, a_scale).double()
    w = dequantize(w_codes, w_scale).double()
    return a @ w.t()


def linear_forward(x, w):
    """fp4_linear.py:33-40 on the non-H100 branch."""
    xc, xs = quantize(x)
    wc, ws = quantize(w)
    return torch.nn.functional.linear(dequantize(xc, xs), dequantize(wc, ws)).to(x.dtype)


def linear_backward_ste(gy, x, w):
    """fp4_linear.py:42-45: straight-through, in the incoming grad's dtype."""
    return (gy @ w.to(gy.dtype)).to(x.dtype), (gy.t() @ x.to(gy.dtype)).to(w.dtype)


def slot_offset(K):
    """dual_gemm.py:23-25."""
    import math
    return int(math.floor(math.log2(144 * K))) + 2


def unpack_dual(acc, s):
    """dual_gemm.py:28-32."""
    w = float(2 ** s)
    c2 = torch.round(acc / w)
    return acc - c2 * w, c2


# --------------------------------------------------------------------------
# Reference integer wires (wire.py:92-138), restated for one process with the
# peers' payloads passed in explicitly: `exchange` objects below carry them.
# --------------------------------------------------------------------------
CHUNK = 64


def padded_len(numel, world, unit=CHUNK):
    """wire.py:86-87."""
    span = world * unit
    return -(-numel // span) * span


def wire_int_step(gs, lim, res=None, ores=None, reverse=False):
    """wire.py:104-138 for every rank at once.  gs: list of fp32 gradients
    (one per rank, equal length).  res/ores: lists of residual tensors or
    None (no error feedback).  Returns the list of averaged outputs."""
    world = len(gs)
    n = gs[0].numel()
    padded = padded_len(n, world)
    vs = []
    for r in range(world):
        v = torch.zeros(padded)
        v[:n] = gs[r]
        if res is not None:
            v += res[r]
        vs.append(v)
    m = torch.stack([v.view(-1, CHUNK).abs().amax(1) for v in vs]).amax(0)
    s = torch.where(m > 0, lim / m, torch.ones_like(m))
    qs = []
    for r in range(world):
        q = torch.round(vs[r].view(-1, CHUNK) * s[:, None]).clamp_(-lim, lim)
        if res is not None:
            res[r].copy_(vs[r] - (q / s[:, None]).view(-1))
        qs.append(q)
    own = padded // CHUNK // world
    q2s, s2s = [], []
    for o in range(world):
        parts = torch.stack([qs[r][o * own:(o + 1) * own] for r in range(world)])
        if reverse:
            parts = parts.flip(0)
        val = parts.to(torch.int32).sum(0).float()
        val /= s[o * own:(o + 1) * own, None]
        if ores is not None:
            val += ores[o]
        m2 = val.abs().amax(1)
        s2 = torch.where(m2 > 0, lim / m2, torch.ones_like(m2))
        q2 = torch.round(val * s2[:, None]).clamp_(-lim, lim)
        if ores is not None:
            ores[o].copy_(val - q2 / s2[:, None])
        q2s.append(q2)
        s2s.append(s2)
    q2 = torch.cat(q2s)
    s2 = torch.cat(s2s)
    out = (q2 / s2[:, None]).view(-1)[:n] / world
    return [out.clone() for _ in range(world)]


# --------------------------------------------------------------------------
# Derived MXFP4 wire: structure of wire.py:104-138, codec of fp4.py.
# --------------------------------------------------------------------------
WIRE_BLOCK = 32


def wire_mxfp4_encode(g, n, padded, res):
    """Sender half (wire.py:106-119 with the fp4 codec): pad, add the sender
    residual, quantize per 32, update the residual.  Returns (packed bytes
    [padded/2] u8, e8m0 [padded/32] u8)."""
    v = torch.zeros(padded)
    v[:n] = g
    if res is not None:
        v += res
    codes, scale = quantize(v.view(-1, WIRE_BLOCK))
    if res is not None:
        res.copy_(v - dequantize(codes, scale).view(-1))
    return pack(codes).view(-1), scale_to_e8m0(scale.view(-1))


def wire_mxfp4_decode(packed, e8m0):
    """bytes -> fp32 values: value * 2^(e-127), exact."""
    codes = unpack(packed.view(-1, WIRE_BLOCK // 2))
    scale = torch.exp2(e8m0.float() - 127.0)
    return dequantize(codes, scale.view(-1, 1)).view(-1)


def wire_mxfp4_owner(slots, ores, reverse=False):
    """Owner half (wire.py:121-135): decode every sender's shard, add them in
    ascending sender order starting from +0.0 (each add a separately rounded
    fp32 op), add the owner residual, re-encode, update the residual.
    slots: list over senders of (packed, e8m0) for this owner's shard."""
    order = range(len(slots) - 1, -1, -1) if reverse else range(len(slots))
    val = torch.zeros(slots[0][0].numel() * 2)
    for s in order:
        val = val + wire_mxfp4_decode(*slots[s])
    if ores is not None:
        val = val + ores
    codes, scale = quantize(val.view(-1, WIRE_BLOCK))
    if ores is not None:
        ores.copy_(val - dequantize(codes, scale).view(-1))
    return pack(codes).view(-1), scale_to_e8m0(scale.view(-1))


def wire_mxfp4_step(gs, res=None, ores=None, reverse=False, return_bytes=False):
    """One all-reduce step for every rank at once.  gs: per-rank fp32
    gradients.  res/ores: per-rank residual lists (error feedback) or None.
    Returns the per-rank outputs (identical on every rank) and, optionally,
    the bytes that crossed the wire: sender payloads and owner payloads."""
    world = len(gs)
    n = gs[0].numel()
    padded = padded_len(n, world)
    shard = padded // world
    sent = [wire_mxfp4_encode(gs[r], n, padded, None if res is None else res[r])
            for r in range(world)]
    owned = []
    for o in range(world):
        lo_b, hi_b = o * shard // 2, (o + 1) * shard // 2
        lo_s, hi_s = o * shard // WIRE_BLOCK, (o + 1) * shard // WIRE_BLOCK
        slots = [(sent[r][0][lo_b:hi_b], sent[r][1][lo_s:hi_s]) for r in range(world)]
        owned.append(wire_mxfp4_owner(slots, None if ores is None else ores[o], reverse))
    full_p = torch.cat([p for p, _ in owned])
    full_s = torch.cat([s for _, s in owned])
    out = wire_mxfp4_decode(full_p, full_s)[:n] / world
    outs = [out.clone() for _ in range(world)]
    if return_bytes:
        return outs, sent, owned
    return outs
