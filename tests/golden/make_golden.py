"""Generates tests/golden/*.npz by running the REAL reference modules.

Run once, in a container that has the lockstep sources:

    python tests/golden/make_golden.py /path/to/lockstep

It imports fp4.py, fp4_linear.py and wire.py from that path (CPU torch only),
feeds them seeded inputs and stores inputs + outputs as small numpy archives.
The test-suite never needs the lockstep sources: it reads the archives.
bf16 tensors are stored as their uint16 bit patterns.

The "wire_mxfp4" archive is not an output of reference wire.py (which has no
FP4 method): it is the owner-reduces protocol of wire.py:104-138 composed here
from the reference's own quantize_mxfp4 / pack_fp4 / dequantize_mxfp4, all
ranks simulated in this one process.
"""

import struct
import sys
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/lockstep")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF))
import fp4            # noqa: E402  (the reference's)
import fp4_linear     # noqa: E402
import wire           # noqa: E402

OUT = Path(__file__).resolve().parent
torch.set_num_threads(4)


def bits16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def f32_from_bits(u):
    return struct.unpack("<f", struct.pack("<I", u & 0xFFFFFFFF))[0]


def adversarial_f32():
    """One value per 32-block decides the scale; the rest probe the rounding."""
    rows = []
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    grid = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    # (a) every midpoint and grid value, both signs, +-1 ulp, at many block exponents
    for e in (-100, -60, -20, -3, -1, 0, 1, 2, 7, 40, 100, 120):
        vals = []
        for m in mids + grid:
            u = struct.unpack("<I", struct.pack("<f", m))[0]
            for d in (-1, 0, 1):
                if m == 0.0 and d == -1:
                    continue
                vals.append(f32_from_bits(u + d))
        vals = vals[:29]
        row = vals + [-vals[3], -vals[10]] + [4.0]          # 4.0 pins amax/scale = 4
        sc = 2.0 ** e
        rows.append([v * sc for v in row[:31]] + [4.0 * sc])
    # (b) block maxima a few ulps below a power of two (fp32 log2 rounds up)
    for k in list(range(-98, 127, 3)) + [1, 2, 3, 4, 5, 8, 9, 16, 17, 32, 33, 64, 65]:
        top = struct.unpack("<I", struct.pack("<f", 2.0 ** k))[0] if k < 128 else None
        for n in (1, 2, 3, 5, 6, 11, 12, 22, 23, 44, 45, 46):
            amax = f32_from_bits(top - n)
            row = [amax * f for f in (1.0, -0.5, 0.375, 0.25, -0.1875, 0.125, 0.0625, 0.03125)]
            rows.append((row * 4)[:32])
    # (c) zeros, signed zeros, subnormals, the 1e-30 clamp, huge, infinities
    z = [0.0] * 32
    rows.append(z)
    rows.append([-0.0] * 32)
    rows.append([0.0, -0.0] * 16)
    rows.append([1e-45 * (i + 1) for i in range(32)])
    rows.append([(-1) ** i * 1e-39 * (i + 1) for i in range(32)])
    rows.append([9.9e-31 * (i + 1) / 32 for i in range(32)])
    rows.append([1.0e-30] + [2.5e-31 * (i % 5) for i in range(31)])
    rows.append([1.0000001e-30] + [-3e-31] * 31)
    rows.append([3.4028234e38] + [(-1) ** i * 1e38 * (i % 4) for i in range(31)])
    rows.append([float("inf")] + [(-1) ** i * 3e38 * (i % 3) / 2 for i in range(31)])
    rows.append([float("-inf"), float("inf")] + [1.0] * 30)
    rows.append([1000.0] + [0.1 * i for i in range(31)])              # one outlier
    x = torch.tensor(rows, dtype=torch.float64).to(torch.float32)
    return x


def main():
    g = torch.Generator().manual_seed(0)

    # ---- quantizer, fp32 adversarial rows
    x = adversarial_f32()
    codes, scale = fp4.quantize_mxfp4(x)
    np.savez_compressed(OUT / "quant_adversarial_f32.npz", x=x.numpy().view(np.uint32),
                        codes=codes.numpy(), scale=scale.numpy().view(np.uint32),
                        packed=fp4.pack_fp4(codes).numpy())

    # ---- NaN block (kept apart: scale is NaN)
    xn = torch.randn(2, 64, generator=g)
    xn[0, 5] = float("nan")
    xn[1, 40] = float("-nan")
    cn, sn = fp4.quantize_mxfp4(xn)
    np.savez_compressed(OUT / "quant_nan_f32.npz", x=xn.numpy().view(np.uint32),
                        codes=cn.numpy(), scale=sn.numpy().view(np.uint32))

    # ---- bf16 activations / weights (shapes of the CPU config, cropped)
    a = torch.randn(64, 1024, generator=g).bfloat16()
    w = (torch.randn(96, 1024, generator=g) * 0.02).bfloat16()
    ac, asc = fp4.quantize_mxfp4(a)
    wc, wsc = fp4.quantize_mxfp4(w)
    c16, s16 = fp4.quantize_mxfp4(a, 16)
    out_bf16 = torch.nn.functional.linear(fp4.dequantize_mxfp4(ac, asc),
                                          fp4.dequantize_mxfp4(wc, wsc)).bfloat16()
    out_f64 = fp4.reference_mxfp4_gemm(ac, asc, wc.t(), wsc.t())
    np.savez_compressed(
        OUT / "quant_gemm_bf16.npz", a=bits16(a), w=bits16(w),
        a_codes=ac.numpy(), a_scale=asc.numpy(), w_codes=wc.numpy(), w_scale=wsc.numpy(),
        a_packed=fp4.pack_fp4(ac).numpy(), a_unpacked=fp4.unpack_fp4(fp4.pack_fp4(ac)).numpy(),
        a_codes16=c16.numpy(), a_scale16=s16.numpy(),
        a_deq=fp4.dequantize_mxfp4(ac, asc).numpy(),
        out_bf16=bits16(out_bf16), out_ref_f32=out_f64.numpy())

    # ---- fp32 wide-range data (reference test recipe, tests/test_fp4.py:56-57)
    torch.manual_seed(0)
    xr = torch.randn(64, 256) * torch.logspace(-3, 3, 64).unsqueeze(1)
    for blk in (16, 32):
        c, s = fp4.quantize_mxfp4(xr, blk)
        np.savez_compressed(OUT / f"quant_logspace_b{blk}.npz", x=xr.numpy(), codes=c.numpy(),
                            scale=s.numpy())

    # ---- tables and the tie vector (tests/test_fp4.py:48-51, fp4.py:20-34)
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    np.savez_compressed(OUT / "tables.npz", values=fp4.E2M1_VALUES.numpy(),
                        e4m3=fp4.E2M1_TO_E4M3.numpy(), q=fp4.E2M1_Q.numpy(),
                        mids=mids.numpy(), mid_codes=fp4._round_to_e2m1(mids).numpy(),
                        neg_mid_codes=fp4._round_to_e2m1(-mids).numpy())

    # ---- linear layer forward + straight-through backward (fp4_linear.py:32-59)
    torch.manual_seed(3)
    lin = fp4_linear.MXFP4Linear(256, 160)
    xin = torch.randn(4, 24, 256, generator=g).bfloat16().requires_grad_(True)
    y = lin(xin)
    gy = torch.randn(y.shape, generator=g).bfloat16()
    y.backward(gy)
    np.savez_compressed(OUT / "linear_ste.npz", w=lin.weight.detach().numpy(), x=bits16(xin.detach()),
                        gy=bits16(gy), y=bits16(y.detach()), gx=bits16(xin.grad),
                        gw=lin.weight.grad.numpy())

    # ---- reference integer wires, one rank, three steps (wire.py:104-138)
    gw = torch.randn(5000, generator=g)
    for method in ("int16", "int8", "int8ef"):
        wobj = wire.Wire(method, gw.numel())
        outs = [wobj(gw.clone() * (1 + 0.5 * s)).numpy().copy() for s in range(3)]
        np.savez_compressed(OUT / f"wire_{method}_w1.npz", g=gw.numpy(), outs=np.stack(outs))

    # ---- derived MXFP4 wire from reference codec functions; worlds 1, 2, 4
    def e8m0(s):
        return ((s.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)

    def decode(p, e):
        return fp4.dequantize_mxfp4(fp4.unpack_fp4(p.view(-1, 16)),
                                    torch.exp2(e.float() - 127).view(-1, 1)).view(-1)

    for world in (1, 2, 4):
        n = 4000 + 37 * world
        span = world * wire.CHUNK
        padded = -(-n // span) * span
        shard = padded // world
        tdist = torch.distributions.StudentT(3.0)
        torch.manual_seed(100 + world)
        grads = [[(tdist.sample((n,)) * 1e-3) for _ in range(world)] for _ in range(3)]
        for ef in (False, True):
            res = [torch.zeros(padded) for _ in range(world)]
            ores = [torch.zeros(shard) for _ in range(world)]
            rec = {}
            for step in range(3):
                sent = []
                for r in range(world):
                    v = torch.zeros(padded)
                    v[:n] = grads[step][r]
                    if ef:
                        v += res[r]
                    c, s = fp4.quantize_mxfp4(v.view(-1, 32))
                    if ef:
                        res[r] = v - fp4.dequantize_mxfp4(c, s).view(-1)
                    sent.append((fp4.pack_fp4(c).view(-1), e8m0(s.view(-1))))
                owned = []
                for o in range(world):
                    val = torch.zeros(shard)
                    for r in range(world):
                        val = val + decode(sent[r][0][o * shard // 2:(o + 1) * shard // 2],
                                           sent[r][1][o * shard // 32:(o + 1) * shard // 32])
                    if ef:
                        val = val + ores[o]
                    c2, s2 = fp4.quantize_mxfp4(val.view(-1, 32))
                    if ef:
                        ores[o] = val - fp4.dequantize_mxfp4(c2, s2).view(-1)
                    owned.append((fp4.pack_fp4(c2).view(-1), e8m0(s2.view(-1))))
                allp = torch.cat([p for p, _ in owned])
                alle = torch.cat([e for _, e in owned])
                out = decode(allp, alle)[:n] / world
                rec[f"sent_p{step}"] = np.stack([p.numpy() for p, _ in sent])
                rec[f"sent_e{step}"] = np.stack([e.numpy() for _, e in sent])
                rec[f"own_p{step}"] = allp.numpy()
                rec[f"own_e{step}"] = alle.numpy()
                rec[f"out{step}"] = out.numpy()
            rec["grads"] = np.stack([np.stack([t.numpy() for t in st]) for st in grads])
            np.savez_compressed(OUT / f"wire_mxfp4{'ef' if ef else ''}_w{world}.npz", **rec)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
