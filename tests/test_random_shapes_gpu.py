"""Seeded random-shape sweeps on the GPU: quantizer bit-exact against the C oracle,
GEMM within the stated tolerance against the oracle's dequantize + fp32 matmul."""

import numpy as np
import pytest
import torch

from oracle import cref, ref_port

pytestmark = pytest.mark.gpu


def test_quantizer_random_shapes():
    from lockstep_b200 import fp4
    rng = np.random.default_rng(2024)
    for _ in range(40):
        block = int(rng.choice([16, 32]))
        rows = int(rng.integers(1, 300))
        K = block * int(rng.integers(1, 40))
        dtype = torch.bfloat16 if rng.random() < 0.5 else torch.float32
        x = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float32) *
                             np.exp2(rng.integers(-60, 60, (rows, 1))).astype(np.float32)).to(dtype)
        x[rng.integers(0, rows), :block] = 0                     # an all-zero block somewhere
        want = cref.quantize(x.float().numpy(), block=block)
        codes, scale = fp4.quantize_mxfp4(x.cuda(), block)
        assert np.array_equal(codes.cpu().numpy(), want["codes"]), (rows, K, block, dtype)
        assert np.array_equal(scale.cpu().numpy(), want["scale"]), (rows, K, block, dtype)
        rt = fp4.unpack_fp4(fp4.pack_fp4(codes))
        assert torch.equal(rt, codes)


def test_gemm_random_shapes():
    from lockstep_b200 import dual_gemm, fp4, mxfp4_gemm
    rng = np.random.default_rng(7)
    for i in range(16):
        M = int(rng.integers(1, 700))
        N = int(rng.integers(1, 900))
        K = 128 * int(rng.integers(1, 12))
        g = torch.Generator().manual_seed(i)
        a = torch.randn(M, K, generator=g).bfloat16()
        a2 = torch.randn(M, K, generator=g).bfloat16()
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
        wc, ws = ref_port.quantize(w)
        pw, sfw = fp4.quantize_mxfp4_packed(w.cuda())
        c1, c2 = dual_gemm.dual_mxfp4(a.cuda(), a2.cuda(), pw, sfw)
        single = mxfp4_gemm.mxfp4_gemm_packed(*fp4.quantize_mxfp4_packed(a.cuda())[:1], pw,
                                              fp4.quantize_mxfp4_packed(a.cuda())[1], sfw)
        for x, c in ((a, c1), (a2, c2), (a, single)):
            xc, xs = ref_port.quantize(x)
            ref = ref_port.gemm_fake_quant(xc, xs, wc, ws).float()
            got = c.float().cpu()
            rel = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
            worst = ((got - ref).abs() / ref.abs().amax(1, keepdim=True).clamp_min(1e-30)).max().item()
            assert rel <= 1e-3 and worst <= 2e-2, (M, N, K, rel, worst)
    mxfp4_gemm.gemm_status()
