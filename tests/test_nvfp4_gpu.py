"""NVFP4 (blocks of 16, E4M3 scales) on the GPU through the C ABI.

The quantizer is held bit for bit to the golden vectors made by lockstep's own
format header (tests/golden/make_golden_nvfp4.py) and to the numpy oracle on
fresh data; the GEMM first to known answers (E4M3 scales with mantissas whose
products stay exact in fp32) and then to dequantize + fp32 matmul of the same
operands -- the checker lockstep itself uses for its MXFP4 product
(fp4_linear.py:38-40) -- within rel-L2 <= 1e-3 and max-abs <= 2e-2 *
||row||_inf, both sides in the same output type."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nvfp4_ref as R

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def mods():
    from lockstep_b200 import fp4, mxfp4_gemm, nvfp4
    yield fp4, nvfp4, mxfp4_gemm
    mxfp4_gemm.gemm_status()


def _check(c, ref, what=""):
    c, ref = c.float().cpu(), ref.float().cpu()
    rel = ((c - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    row_inf = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    worst = ((c - ref).abs() / row_inf).max().item()
    assert rel <= 1e-3 and worst <= 2e-2, f"{what}: rel-L2 {rel:.3e}, max-abs/row-inf {worst:.3e}"


def _sf_offsets(rows, K):
    r = torch.arange(rows).unsqueeze(1)
    kb = torch.arange(K // 16).unsqueeze(0)
    return (((r // 128) * (K // 64) + kb // 4) * 512 + (r % 32) * 16 + (r % 128 // 32) * 4 + kb % 4).reshape(-1)


@pytest.mark.parametrize("name", ["normal_f32", "normal_bf16", "adversarial"])
def test_quantizer_equals_reference_golden(mods, name):
    fp4, nv, _ = mods
    z = np.load(G / f"nvfp4_{name}.npz")
    x = torch.from_numpy(z["x"].view(np.float32).copy())
    dts = [torch.float32] + ([torch.bfloat16] if name == "normal_bf16" else [])
    for dt in dts:
        packed, scale, sf, u8 = nv.quantize_nvfp4(x.cuda().to(dt), want_bytes=True)
        assert np.array_equal(fp4.unpack_fp4(packed).cpu().numpy(), z["codes"]), (name, dt)
        assert np.array_equal(scale.cpu().numpy().view(np.uint32), z["scale"]), (name, dt)
        assert np.array_equal(u8.cpu().numpy(), R.e4m3_byte(z["scale"].view(np.float32)))
        rows, K = x.shape
        assert torch.equal(sf.cpu()[_sf_offsets(rows, K)], u8.cpu().reshape(-1))
        deq = nv.dequantize_nvfp4(packed, u8).cpu().numpy()
        want = R.dequantize(z["codes"], z["scale"].view(np.float32))
        assert np.array_equal(deq, want)


@pytest.mark.parametrize("rows,K,dt", [(300, 1024, torch.float32), (1000, 384, torch.bfloat16), (1, 128, torch.float32)])
def test_quantizer_equals_oracle_on_fresh_data(mods, rows, K, dt):
    fp4, nv, _ = mods
    g = torch.Generator(device="cuda").manual_seed(rows + K)
    x = torch.randn(rows, K, device="cuda", generator=g) * torch.exp2(torch.randint(-12, 12, (rows, 1), device="cuda", generator=g).float())
    x = torch.where(torch.rand(rows, K, device="cuda", generator=g) < 0.01, x * 50, x).to(dt)
    packed, scale, _ = nv.quantize_nvfp4(x)
    codes, want_scale = R.quantize(x.float().cpu().numpy())
    assert np.array_equal(fp4.unpack_fp4(packed).cpu().numpy(), codes)
    assert np.array_equal(scale.cpu().numpy(), want_scale)
    out = nv.dequantize_nvfp4(packed, torch.from_numpy(R.e4m3_byte(want_scale)).cuda(), out_dtype=torch.bfloat16)
    assert torch.equal(out.cpu(), torch.from_numpy(R.dequantize(codes, want_scale)).bfloat16())


def _sf_of(u8, rows, K):
    sf = torch.zeros(((rows + 127) // 128) * (K // 64) * 512, dtype=torch.uint8)
    sf[_sf_offsets(rows, K)] = u8.reshape(-1)
    return sf.cuda()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 64, 256), (256, 384, 640), (40, 200, 1152)])
def test_gemm_exact_with_e4m3_scales(mods, M, N, K):
    fp4, nv, mg = mods
    g = torch.Generator().manual_seed(M + N + K)
    ac = torch.randint(0, 16, (M, K), dtype=torch.uint8, generator=g)
    bc = torch.randint(0, 16, (N, K), dtype=torch.uint8, generator=g)
    # scale bytes 0x38 .. 0x3F: 1, 1.125 .. 1.875 -- every mantissa, one binade, so that each partial sum
    # (block dot <= 2304 quarter units x a significand product <= 225 / 64, 72 blocks at most) fits 24 bits
    sa = torch.randint(0x38, 0x40, (M, K // 16), dtype=torch.uint8, generator=g)
    sb = torch.randint(0x38, 0x40, (N, K // 16), dtype=torch.uint8, generator=g)
    c = nv.nvfp4_gemm_packed(fp4.pack_fp4(ac.cuda()), fp4.pack_fp4(bc.cuda()), _sf_of(sa, M, K), _sf_of(sb, N, K),
                             out_dtype=torch.float32)
    mg.gemm_status()
    dec = lambda b: ((8 + (b & 7)).double() * torch.exp2((b >> 3).double() - 10))
    A = torch.from_numpy(R.dequantize(ac.numpy(), np.ones((M, K // 16), np.float32))).double().reshape(M, K // 16, 16) * dec(sa).unsqueeze(-1)
    B = torch.from_numpy(R.dequantize(bc.numpy(), np.ones((N, K // 16), np.float32))).double().reshape(N, K // 16, 16) * dec(sb).unsqueeze(-1)
    want = A.reshape(M, K) @ B.reshape(N, K).t()
    assert torch.equal(c.double().cpu(), want)


@pytest.mark.parametrize("M,N,K,dt", [(256, 512, 1024, torch.bfloat16), (300, 520, 1024, torch.float32),
                                      (16, 1024, 2048, torch.bfloat16), (2048, 2048, 2048, torch.bfloat16)])
def test_gemm_against_dequantized_product(mods, M, N, K, dt):
    fp4, nv, mg = mods
    g = torch.Generator(device="cuda").manual_seed(M * 3 + N + K)
    a = torch.randn(M, K, device="cuda", generator=g)
    a = torch.where(torch.rand(M, K, device="cuda", generator=g) < 0.01, a * 50, a).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    pa, _, sfa = nv.quantize_nvfp4(a)
    pw, _, sfw = nv.quantize_nvfp4(w)
    c = nv.nvfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=dt)
    mg.gemm_status()
    ac, asc = R.quantize(a.float().cpu().numpy())
    wc, wsc = R.quantize(w.float().cpu().numpy())
    assert np.array_equal(fp4.unpack_fp4(pa).cpu().numpy(), ac)
    ref = torch.nn.functional.linear(torch.from_numpy(R.dequantize(ac, asc)), torch.from_numpy(R.dequantize(wc, wsc))).to(dt)
    _check(c, ref, f"NVFP4 {M} x {N} x {K}")


def test_gemm_dual_equals_two_singles(mods):
    fp4, nv, mg = mods
    M, N, K = 384, 640, 512
    g = torch.Generator(device="cuda").manual_seed(11)
    xs = [torch.randn(M, K, device="cuda", generator=g).bfloat16() for _ in range(2)]
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    q = [nv.quantize_nvfp4(x) for x in xs]
    pw, _, sfw = nv.quantize_nvfp4(w)
    singles = [nv.nvfp4_gemm_packed(p, pw, sf, sfw) for p, _, sf in q]
    c1, c2 = nv.nvfp4_gemm_dual(q[0][0], q[1][0], pw, q[0][2], q[1][2], sfw)
    mg.gemm_status()
    assert torch.equal(c1, singles[0]) and torch.equal(c2, singles[1])


def test_nvfp4_is_closer_to_the_unquantized_product_than_mxfp4(mods):
    # the point of the format (quant_sim.cuh:90-92): a scale with a mantissa wastes less of a block's range
    fp4, nv, mg = mods
    M, N, K = 512, 512, 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    exact = a @ w.t()
    pa, sfa = fp4.quantize_mxfp4_packed(a)
    pw, sfw = fp4.quantize_mxfp4_packed(w)
    e_mx = ((mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=torch.float32) - exact).norm() / exact.norm()).item()
    pa, _, sfa = nv.quantize_nvfp4(a)
    pw, _, sfw = nv.quantize_nvfp4(w)
    e_nv = ((nv.nvfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=torch.float32) - exact).norm() / exact.norm()).item()
    mg.gemm_status()
    assert e_nv < e_mx, (e_nv, e_mx)


def test_quantizer_on_every_bf16_pattern(mods):
    # all 65536 bf16 bit patterns (zeros, subnormals, infinities, NaNs included), in order (neighbours of like
    # magnitude: realistic scales) and in blocks that mix a few binades; bf16 input and the same values as fp32
    fp4, nv, _ = mods
    bits = torch.arange(65536, dtype=torch.int32)
    ordered = (bits << 16).view(torch.float32).reshape(32, 2048)
    g = torch.Generator().manual_seed(1)
    near = bits.reshape(-1, 256)[:, torch.randperm(256, generator=g)].reshape(-1)        # shuffled within +-2 binades
    mixed = (near << 16).view(torch.float32).reshape(32, 2048)
    for x in (ordered, mixed):
        codes, want_scale = R.quantize(x.numpy())
        for dt in (torch.bfloat16, torch.float32):
            packed, scale, _ = nv.quantize_nvfp4(x.cuda().to(dt))
            assert np.array_equal(scale.cpu().numpy().view(np.uint32), want_scale.view(np.uint32)), dt
            assert np.array_equal(fp4.unpack_fp4(packed).cpu().numpy(), codes), dt
