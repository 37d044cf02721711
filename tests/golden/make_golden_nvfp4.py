"""Generates tests/golden/nvfp4_*.npz from lockstep's own NVFP4 format functions.

Run where the reference's sources are present (`make -C oracle ref` builds
oracle/_ref/libnvfp4_ref.so around rig_sm75/quant_sim.cuh):

    python tests/golden/make_golden_nvfp4.py

Each file holds inputs (float32 bit patterns) and, from the reference, the E2M1
codes, the block scales and the dequantized values.
"""

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE = HERE.parent.parent / "oracle"


def ref_lib():
    subprocess.run(["make", "-C", str(ORACLE), "ref"], check=True, capture_output=True)
    lib = ctypes.CDLL(str(ORACLE / "_ref" / "libnvfp4_ref.so"))
    lib.ref_quant_e4m3.restype = ctypes.c_float
    lib.ref_quant_e4m3.argtypes = [ctypes.c_float]
    lib.ref_nv_scale.restype = ctypes.c_float
    lib.ref_nv_scale.argtypes = [ctypes.c_float]
    lib.ref_e2m1_code.restype = ctypes.c_int
    lib.ref_e2m1_code.argtypes = [ctypes.c_float]
    return lib


def blocks(lib, x):
    x = np.ascontiguousarray(x, np.float32)
    nb = x.size // 16
    codes = np.empty(x.size, np.uint8)
    scale = np.empty(nb, np.float32)
    deq = np.empty(x.size, np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    lib.ref_nvfp4_blocks(p(x), ctypes.c_int64(nb), p(codes), p(scale), p(deq))
    return codes.reshape(x.shape), scale.reshape(*x.shape[:-1], x.shape[-1] // 16), deq.reshape(x.shape)


def main():
    lib = ref_lib()
    rng = np.random.default_rng(20240607)

    # scalar functions on a dense set of inputs: every E4M3 value, the midpoints between
    # neighbours, one ulp either side of each, the subnormal range, saturation, zeros
    e4 = np.array([((8 + m) * 2.0 ** (e - 10)) if e else m * 2.0 ** -9 for e in range(16) for m in range(8)][:-1], np.float32)
    mids = (e4[:-1].astype(np.float64) + e4[1:]) / 2
    pts = np.concatenate([e4, mids.astype(np.float32), np.nextafter(mids.astype(np.float32), np.float32(0)),
                          np.nextafter(mids.astype(np.float32), np.float32(1e9)),
                          np.array([0, 2.0 ** -10, 2.0 ** -11, 447.9, 448, 463.9, 464, 480, 1e6, np.inf], np.float32),
                          np.exp(rng.uniform(np.log(1e-4), np.log(600), 4000)).astype(np.float32)])
    pts = np.concatenate([pts, -pts]).astype(np.float32)
    q = np.array([lib.ref_quant_e4m3(float(v)) for v in pts], np.float32)
    amax = np.abs(pts) * np.float32(6)
    amax = np.concatenate([amax, np.array([0, 1e-30, 1e-4, 2.0 ** -9 * 6, 2.0 ** -10 * 6, 2687.9, 2688, 3000, 1e30, np.inf],
                                          np.float32)]).astype(np.float32)
    sc = np.array([lib.ref_nv_scale(float(v)) for v in amax], np.float32)
    grid = np.array([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7, 100], np.float32)
    xs = np.concatenate([grid, np.nextafter(grid, np.float32(-1)), np.nextafter(grid, np.float32(1e9)),
                         rng.uniform(0, 8, 2000).astype(np.float32), np.array([np.inf, np.nan], np.float32)])
    xs = np.concatenate([xs, -xs]).astype(np.float32)
    cd = np.array([lib.ref_e2m1_code(float(v)) for v in xs], np.uint8)
    np.savez_compressed(HERE / "nvfp4_scalar.npz", e4m3_in=pts.view(np.uint32), e4m3_out=q.view(np.uint32),
                        amax=amax.view(np.uint32), scale=sc.view(np.uint32), code_in=xs.view(np.uint32), code_out=cd)

    # whole blocks: normal data with outliers (fp32 and values that are exactly bf16)
    x = rng.standard_normal((96, 512)).astype(np.float32)
    x = np.where(rng.uniform(size=x.shape) < 0.01, x * 50, x).astype(np.float32)
    xb = (x.view(np.uint32) & 0xFFFF0000).view(np.float32)
    for name, data in (("normal_f32", x), ("normal_bf16", xb)):
        c, s, d = blocks(lib, data)
        np.savez_compressed(HERE / f"nvfp4_{name}.npz", x=data.view(np.uint32), codes=c, scale=s.view(np.uint32), deq=d.view(np.uint32))

    # adversarial blocks: magnitudes over 60 binades, quotients on the rounding midpoints of E2M1
    # for scales with a mantissa, maxima that put amax / 6 on E4M3 midpoints, zero blocks, blocks
    # of tiny values (scale floor 2^-9), huge values (scale saturates), NaN and infinities
    rows = []
    mag = np.exp2(rng.uniform(-30, 30, (64, 1))).astype(np.float32)
    rows.append((rng.standard_normal((64, 128)) * mag).astype(np.float32))
    scales = np.array([((8 + m) * 2.0 ** (e - 10)) for e in range(4, 12) for m in range(8)], np.float32)      # 64 scales
    mid = np.array([.25, .75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    t = np.zeros((64, 128), np.float32)
    for i, s in enumerate(scales):
        for b in range(8):
            blk = np.empty(16, np.float32)
            blk[0] = 6 * s                                   # fixes the block scale at s
            m = np.resize(mid, 15) * s
            wiggle = rng.integers(-1, 2, 15)
            m = np.where(wiggle < 0, np.nextafter(m, np.float32(0)), np.where(wiggle > 0, np.nextafter(m, np.float32(1e9)), m))
            blk[1:] = m * rng.choice([-1, 1], 15)
            t[i, b * 16:(b + 1) * 16] = blk
    rows.append(t)
    t = rng.standard_normal((32, 128)).astype(np.float32)
    for i in range(32):
        for b in range(8):
            k = rng.integers(0, len(mids))
            v = np.float32(mids[k]) * np.float32(6)
            v = [np.nextafter(v, np.float32(0)), v, np.nextafter(v, np.float32(1e9))][rng.integers(0, 3)]
            blk = t[i, b * 16:(b + 1) * 16]
            blk *= v / (np.abs(blk).max() * 1.01)
            blk[rng.integers(0, 16)] = v
    rows.append(t)
    t = np.zeros((18, 128), np.float32)
    t[1] = rng.standard_normal(128) * 1e-4
    t[2] = rng.standard_normal(128) * 1e-6
    t[3] = rng.standard_normal(128) * 1e5
    t[4] = rng.standard_normal(128) * 3000
    t[5, ::7] = -0.0
    t[6] = rng.standard_normal(128); t[6, 5] = np.nan; t[6, 40] = -np.nan
    t[7] = rng.standard_normal(128); t[7, 3] = np.inf; t[7, 20] = -np.inf
    t[8, :16] = np.nan
    t[9] = rng.standard_normal(128) * 2.0 ** -9
    t[10] = rng.standard_normal(128) * 2.0 ** -11
    t[11, 17] = 1e-38
    t[12] = 448 * 6
    t[13] = rng.uniform(-6, 6, 128) * 448
    t[14] = rng.standard_normal(128) * np.exp2(rng.uniform(20, 40, 128))       # quotients around and beyond 2^23:
    t[15] = rng.standard_normal(128) * 1e30                                     # the candidate loop's distances collapse
    t[16] = np.exp2(rng.integers(28, 36, 128)) * rng.choice([-1, 1, 1.5, -1.25], 128)
    t[17, :16] = 3e38; t[17, 3] = -3.4e38
    rows.append(t)
    x = np.concatenate(rows).astype(np.float32)
    c, s, d = blocks(lib, x)
    np.savez_compressed(HERE / "nvfp4_adversarial.npz", x=x.view(np.uint32), codes=c, scale=s.view(np.uint32), deq=d.view(np.uint32))
    print("wrote", sorted(p.name for p in HERE.glob("nvfp4_*.npz")))


if __name__ == "__main__":
    main()
