"""The MXFP4 GEMM on operands quantized in blocks of 16 (fp4.py:57,
quantize_mxfp4(x, 16)) through the C ABI.

lockstep's quantizer takes any block size but its GEMM only 32 values per
scale (mxfp4_gemm.py:136); the checker for this form is therefore the same
dequantize + fp32 matmul that checks the block-32 GEMM (fp4_linear.py:38-40),
given the oracle's block-16 codes and scales.  Known-answer cases first
(power-of-two scales that differ between neighbouring blocks of 16: exact in
fp32, and wrong if a scale were applied to 32 values or to the wrong k-block),
then the stated tolerance: rel-L2 <= 1e-3 and max-abs <= 2e-2 * ||row||_inf
with both sides in the same output type."""

import pytest
import torch

from oracle import ref_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    from lockstep_b200 import fp4, mxfp4_gemm
    yield fp4, mxfp4_gemm
    mxfp4_gemm.gemm_status()


def _check(c, ref, what=""):
    c, ref = c.float().cpu(), ref.float().cpu()
    rel = ((c - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    row_inf = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    worst = ((c - ref).abs() / row_inf).max().item()
    assert rel <= 1e-3 and worst <= 2e-2, f"{what}: rel-L2 {rel:.3e}, max-abs/row-inf {worst:.3e}"


def test_quantizer_scale_factor_bytes_block16(mods):
    # the scale-factor buffer of the fused pass holds the oracle's exponents at the
    # documented offsets: tile (row / 128, kblock / 4), byte (row % 32) * 16 + (row % 128 / 32) * 4 + kblock % 4
    fp4, _ = mods
    rows, K = 200, 384
    x = torch.randn(rows, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)) * 3
    packed, sf, scale = fp4.quantize_mxfp4_packed(x, want_scale=True, block=16)
    codes, want_scale = ref_port.quantize(x.cpu(), block=16)
    assert torch.equal(fp4.unpack_fp4(packed).cpu(), codes)
    assert torch.equal(scale.cpu(), want_scale)
    assert sf.numel() == 2 * (K // 64) * 512 == fp4.sf_bytes(rows, K, 16)
    e = (want_scale.log2().round().to(torch.int32) + 127).to(torch.uint8)
    r = torch.arange(rows).unsqueeze(1)
    kb = torch.arange(K // 16).unsqueeze(0)
    off = ((r // 128) * (K // 64) + kb // 4) * 512 + (r % 32) * 16 + (r % 128 // 32) * 4 + kb % 4
    assert torch.equal(sf.cpu()[off.reshape(-1)], e.reshape(-1))
    sf2, bad = fp4.scales_to_sf(scale, block=16)
    assert int(bad.item()) == 0
    assert torch.equal(sf2.cpu()[off.reshape(-1)], e.reshape(-1))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 64, 256), (256, 384, 640), (40, 200, 1152)])
def test_block16_power_of_two_scales_exact(mods, M, N, K):
    fp4, mg = mods
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    ac = torch.randint(0, 16, (M, K), dtype=torch.uint8, device="cuda", generator=g)
    bc = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    sa = torch.exp2(torch.randint(-3, 4, (M, K // 16), device="cuda", generator=g).float())
    sb = torch.exp2(torch.randint(-3, 4, (N, K // 16), device="cuda", generator=g).float())
    c = mg.mxfp4_gemm_packed(fp4.pack_fp4(ac), fp4.pack_fp4(bc), sa, sb, out_dtype=torch.float32, block=16)
    mg.gemm_status()
    want = fp4.dequantize_mxfp4(ac, sa, 16).double() @ fp4.dequantize_mxfp4(bc, sb, 16).double().t()
    assert torch.equal(c.double(), want)


def test_block16_one_scaled_block_lands_on_its_k_range(mods):
    # one block of 16 of one row of A carries scale 8: only products from that k range grow
    fp4, mg = mods
    M, N, K = 128, 128, 256
    ac = torch.full((M, K), 2, dtype=torch.uint8, device="cuda")       # 1.0
    ones_b = torch.ones(N, K // 16, device="cuda")
    for blk in (0, 1, 3, 4, 7, 9, 15):
        bc = torch.zeros(N, K, dtype=torch.uint8, device="cuda")
        bc[:, blk * 16:(blk + 1) * 16] = 2                                # W is 1.0 on that block only
        sa = torch.ones(M, K // 16, device="cuda")
        sa[77, blk] = 8.0
        c = mg.mxfp4_gemm_packed(fp4.pack_fp4(ac), fp4.pack_fp4(bc), sa, ones_b, out_dtype=torch.float32, block=16)
        want = torch.full((M, N), 16.0)
        want[77] = 128.0
        assert torch.equal(c.cpu(), want), blk
        sa[77, blk] = 1.0
        sa[77, (blk + 1) % (K // 16)] = 8.0                               # a neighbour's scale must not leak in
        c = mg.mxfp4_gemm_packed(fp4.pack_fp4(ac), fp4.pack_fp4(bc), sa, ones_b, out_dtype=torch.float32, block=16)
        assert torch.equal(c.cpu(), torch.full((M, N), 16.0)), blk


@pytest.mark.parametrize("M,N,K,dt", [(256, 512, 1024, torch.bfloat16), (300, 520, 1024, torch.float32),
                                      (16, 1024, 2048, torch.bfloat16), (1000, 192, 384, torch.bfloat16),
                                      (2048, 2048, 2048, torch.bfloat16)])
def test_block16_against_oracle(mods, M, N, K, dt):
    fp4, mg = mods
    g = torch.Generator(device="cuda").manual_seed(M * 3 + N + K)
    a = torch.randn(M, K, device="cuda", generator=g)
    a = torch.where(torch.rand(M, K, device="cuda", generator=g) < 0.01, a * 50, a).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    pa, sfa = fp4.quantize_mxfp4_packed(a, block=16)
    pw, sfw = fp4.quantize_mxfp4_packed(w, block=16)
    c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=dt, block=16)
    mg.gemm_status()
    ac, asc = ref_port.quantize(a.cpu(), block=16)
    wc, wsc = ref_port.quantize(w.cpu(), block=16)
    assert torch.equal(fp4.unpack_fp4(pa).cpu(), ac) and torch.equal(fp4.unpack_fp4(pw).cpu(), wc)
    ref = torch.nn.functional.linear(ref_port.dequantize(ac, asc, 16), ref_port.dequantize(wc, wsc, 16)).to(dt)
    _check(c, ref, f"block 16, {M} x {N} x {K}")


def test_block16_dual_equals_two_singles(mods):
    fp4, mg = mods
    from lockstep_b200._lib import check, dtype_code, lib, ptr, stream
    M, N, K = 384, 640, 512
    g = torch.Generator(device="cuda").manual_seed(11)
    xs = [torch.randn(M, K, device="cuda", generator=g).bfloat16() for _ in range(2)]
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    q = [fp4.quantize_mxfp4_packed(x, block=16) for x in xs]
    pw, sfw = fp4.quantize_mxfp4_packed(w, block=16)
    singles = [mg.mxfp4_gemm_packed(p, pw, sf, sfw, block=16) for p, sf in q]
    c = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    check(lib().ls_mxfp4_gemm_dual_block16(ptr(q[0][0]), ptr(q[1][0]), ptr(pw), ptr(q[0][1]), ptr(q[1][1]), ptr(sfw),
                                           ptr(c[0]), ptr(c[1]), dtype_code(torch.bfloat16), M, N, K, stream()))
    mg.gemm_status()
    assert torch.equal(c[0], singles[0]) and torch.equal(c[1], singles[1])


def test_block16_is_at_least_as_close_to_the_unquantized_product(mods):
    # finer scale blocks cannot lose accuracy on data with outliers: the quantization error of the
    # product against the unquantized fp32 product is smaller with blocks of 16 than with 32
    fp4, mg = mods
    M, N, K = 512, 512, 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(M, K, device="cuda", generator=g)
    a = torch.where(torch.rand(M, K, device="cuda", generator=g) < 0.02, a * 30, a)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    exact = a @ w.t()
    errs = {}
    for block in (32, 16):
        pa, sfa = fp4.quantize_mxfp4_packed(a, block=block)
        pw, sfw = fp4.quantize_mxfp4_packed(w, block=block)
        c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=torch.float32, block=block)
        errs[block] = ((c - exact).norm() / exact.norm()).item()
    mg.gemm_status()
    assert errs[16] < errs[32], errs


@pytest.mark.parametrize("fmt", ["mx16", "nvfp4"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 640, 1152), (1000, 520, 2048)])
def test_block16_kernels_agree(mods, fmt, M, N, K):
    # the CTA-pair kernel (the default above 128 rows; 256- and 192-column tiles) and the single-CTA kernel with 128- and 64-column tiles
    # issue the same MMAs in the same order over K: identical bits, and within tolerance of the oracle
    fp4, mg = mods
    from lockstep_b200 import nvfp4
    from lockstep_b200._lib import lib
    from oracle import nvfp4_ref
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    if fmt == "mx16":
        pa, sfa = fp4.quantize_mxfp4_packed(a, block=16)
        pw, sfw = fp4.quantize_mxfp4_packed(w, block=16)
        run = lambda: mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=torch.float32, block=16)
        ac, asc = ref_port.quantize(a.cpu(), block=16)
        wc, wsc = ref_port.quantize(w.cpu(), block=16)
        ref = torch.nn.functional.linear(ref_port.dequantize(ac, asc, 16), ref_port.dequantize(wc, wsc, 16))
    else:
        pa, _, sfa = nvfp4.quantize_nvfp4(a)
        pw, _, sfw = nvfp4.quantize_nvfp4(w)
        run = lambda: nvfp4.nvfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=torch.float32)
        ac, asc = nvfp4_ref.quantize(a.float().cpu().numpy())
        wc, wsc = nvfp4_ref.quantize(w.float().cpu().numpy())
        ref = torch.nn.functional.linear(torch.from_numpy(nvfp4_ref.dequantize(ac, asc)),
                                         torch.from_numpy(nvfp4_ref.dequantize(wc, wsc)))
    outs = {}
    try:
        for variant in (2, 6, 3, 5):
            lib().ls_gemm_set_variant(variant)
            outs[variant] = run()
    finally:
        lib().ls_gemm_set_variant(0)
    mg.gemm_status()
    _check(outs[2], ref, f"{fmt} pair kernel {M} x {N} x {K}")
    assert torch.equal(outs[2], outs[3]) and torch.equal(outs[2], outs[5]) and torch.equal(outs[2], outs[6])
