"""GPU parity of the tcgen05 MXFP4 GEMM (single and dual batch) through the
C ABI.  Known-answer first (unit scales, integer-valued products: bit-exact),
then the reference's dequantize + fp32 matmul path within the stated
tolerance: rel-L2 <= 1e-3 and max-abs <= 2e-2 * ||row||_inf, both outputs in
the same dtype."""

import numpy as np
import pytest
import torch

from oracle import ref_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    from lockstep_b200 import dual_gemm, fp4, mxfp4_gemm
    yield fp4, mxfp4_gemm, dual_gemm
    mxfp4_gemm.gemm_status()


def _check(c, ref, what=""):
    c, ref = c.float().cpu(), ref.float().cpu()
    rel = ((c - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    row_inf = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    worst = ((c - ref).abs() / row_inf).max().item()
    assert rel <= 1e-3 and worst <= 2e-2, f"{what}: rel-L2 {rel:.3e}, max-abs/row-inf {worst:.3e}"


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 256, 256), (256, 256, 128), (128, 512, 1024)])
def test_unit_scale_bit_exact(mods, M, N, K):
    # design of the reference's bench.py:41-57: unit scales, integer grid, exact
    fp4, mg, _ = mods
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    ac = torch.randint(0, 16, (M, K), dtype=torch.uint8, device="cuda", generator=g)
    bc = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    ones_a = torch.ones(M, K // 32, device="cuda")
    ones_b = torch.ones(N, K // 32, device="cuda")
    c = mg.mxfp4_gemm_packed(fp4.pack_fp4(ac), fp4.pack_fp4(bc), ones_a, ones_b, out_dtype=torch.float32)
    mg.gemm_status()
    want = (fp4.codes_to_q(ac).double() @ fp4.codes_to_q(bc).double().t()) / 4
    assert torch.equal(c.double(), want)


def test_one_hot_nibble_order(mods):
    # a single non-zero code at an odd and an even K index must land on the right product
    fp4, mg, _ = mods
    M, N, K = 128, 256, 128
    for ka in (0, 1, 33, 126):
        ac = torch.zeros(M, K, dtype=torch.uint8, device="cuda")
        bc = torch.zeros(N, K, dtype=torch.uint8, device="cuda")
        ac[5, ka] = 6           # 4.0
        bc[:, :] = 2            # 1.0 everywhere
        bc[7, ka] = 13          # -3.0
        sa = torch.ones(M, K // 32, device="cuda")
        sb = torch.ones(N, K // 32, device="cuda")
        c = mg.mxfp4_gemm_packed(fp4.pack_fp4(ac), fp4.pack_fp4(bc), sa, sb, out_dtype=torch.float32)
        want = torch.zeros(M, N)
        want[5, :] = 4.0
        want[5, 7] = -12.0
        assert torch.equal(c.cpu(), want), ka


def test_block_scales_exact_powers(mods):
    # random power-of-two scales: products stay exactly representable in fp32
    fp4, mg, _ = mods
    M, N, K = 256, 512, 512
    g = torch.Generator(device="cuda").manual_seed(7)
    ac = torch.randint(0, 16, (M, K), dtype=torch.uint8, device="cuda", generator=g)
    bc = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    sa = torch.exp2(torch.randint(-3, 4, (M, K // 32), device="cuda", generator=g).float())
    sb = torch.exp2(torch.randint(-3, 4, (N, K // 32), device="cuda", generator=g).float())
    c = mg.mxfp4_gemm_packed(fp4.pack_fp4(ac), fp4.pack_fp4(bc), sa, sb, out_dtype=torch.float32)
    mg.gemm_status()
    want = fp4.dequantize_mxfp4(ac, sa).double() @ fp4.dequantize_mxfp4(bc, sb).double().t()
    assert torch.equal(c.double(), want)       # |sum| < 2^24 quarter units: exact


def test_config1_against_oracle(mods):
    # A 256x1024 N(0,1) seed 0, W 1024x1024 N(0,0.02) seed 1, bf16
    fp4, mg, _ = mods
    a = torch.randn(256, 1024, generator=torch.Generator().manual_seed(0)).bfloat16()
    w = (torch.randn(1024, 1024, generator=torch.Generator().manual_seed(1)) * 0.02).bfloat16()
    ac, asc = ref_port.quantize(a)
    wc, wsc = ref_port.quantize(w)
    ref = ref_port.gemm_fake_quant(ac, asc, wc, wsc)                 # bf16
    pa, sfa = fp4.quantize_mxfp4_packed(a.cuda())
    pw, sfw = fp4.quantize_mxfp4_packed(w.cuda())
    assert torch.equal(pa.cpu(), ref_port.pack(ac)) and torch.equal(pw.cpu(), ref_port.pack(wc))
    c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw)
    mg.gemm_status()
    _check(c, ref, "config 1")
    c32 = mg.mxfp4_gemm_packed(pa, pw, asc.cuda(), wsc.cuda(), out_dtype=torch.float32)
    _check(c32, ref_port.gemm_fp64(ac, asc, wc, wsc), "config 1 fp32 vs fp64")
    assert torch.equal(c32.bfloat16(), c)       # epilogue rounding = torch's round-to-nearest-even


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (16, 384, 256), (130, 200, 384), (257, 1000, 640),
                                   (128, 8, 128), (300, 264, 1152)])
def test_ragged_shapes(mods, M, N, K):
    fp4, mg, _ = mods
    g = torch.Generator().manual_seed(M * 7 + N)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    ac, asc = ref_port.quantize(a)
    wc, wsc = ref_port.quantize(w)
    pa, sfa = fp4.quantize_mxfp4_packed(a.cuda())
    pw, sfw = fp4.quantize_mxfp4_packed(w.cuda())
    for dt in (torch.bfloat16, torch.float32):
        guard = torch.full((M + 2, N), 777.0, device="cuda", dtype=dt)
        c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=dt)
        mg.gemm_status()
        _check(c, ref_port.gemm_fake_quant(ac, asc, wc, wsc, dt), f"{M}x{N}x{K} {dt}")
        assert (guard == 777.0).all()


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 2048, 8192), (100, 512, 2048), (128, 1000, 1152)])
def test_skinny_shapes(mods, M, N, K):
    # few rows and a long K: 128-column tiles, an A box of only M rows (K splits are forced in the next test)
    fp4, mg, _ = mods
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g)
    a = torch.where(torch.rand(M, K, generator=g) < 0.01, a * 50, a).bfloat16()       # 1 % outliers x 50
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    ac, asc = ref_port.quantize(a)
    wc, wsc = ref_port.quantize(w)
    pa, sfa = fp4.quantize_mxfp4_packed(a.cuda())
    pw, sfw = fp4.quantize_mxfp4_packed(w.cuda())
    for dt in (torch.bfloat16, torch.float32):
        c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=dt)
        mg.gemm_status()
        _check(c, ref_port.gemm_fake_quant(ac, asc, wc, wsc, dt), f"{M}x{N}x{K} {dt}")
    assert torch.equal(mg.mxfp4_gemm_packed(pa, pw, sfa, sfw), mg.mxfp4_gemm_packed(pa, pw, sfa, sfw))   # deterministic


@pytest.mark.parametrize("variant,M,N,K,splits", [(1, 128, 512, 2048, 3), (1, 100, 300, 1152, 16), (2, 512, 512, 2048, 2), (3, 40, 300, 1152, 2), (1, 700, 520, 1024, 1), (3, 300, 264, 512, 2),
                                                  (2, 300, 520, 4096, 5), (2, 1024, 1024, 16384, 0),
                                                  (5, 16, 4096, 512, 1), (5, 1, 1000, 1152, 1), (5, 100, 300, 1152, 2),
                                                  (5, 128, 264, 640, 3), (5, 40, 8192, 256, 1), (5, 130, 200, 384, 1),
                                                  (6, 256, 384, 128, 1), (6, 512, 520, 2048, 1), (6, 300, 1000, 1152, 2),
                                                  (6, 1024, 200, 640, 3), (6, 130, 8192, 256, 1), (6, 2048, 448, 4096, 0)])
def test_forced_k_splits_exact_and_dual(mods, variant, M, N, K, splits):
    # power-of-two scales on an integer grid: every partial sum is exact, so a split
    # product must equal the unsplit one bit for bit, on both kernels and both batches
    fp4, mg, dg = mods
    from lockstep_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(K + splits)
    ac = torch.randint(0, 16, (2, M, K), dtype=torch.uint8, device="cuda", generator=g)
    bc = torch.randint(0, 16, (N, K), dtype=torch.uint8, device="cuda", generator=g)
    sa = torch.exp2(torch.randint(-2, 3, (2, M, K // 32), device="cuda", generator=g).float())
    sb = torch.exp2(torch.randint(-2, 3, (N, K // 32), device="cuda", generator=g).float())
    pa, pb = fp4.pack_fp4(ac), fp4.pack_fp4(bc)
    want = [fp4.dequantize_mxfp4(ac[i], sa[i]).double() @ fp4.dequantize_mxfp4(bc, sb).double().t() for i in range(2)]
    try:
        assert L.ls_gemm_set_variant(variant) == 0 and L.ls_gemm_set_splits(splits) == 0
        c = mg.mxfp4_gemm_packed(pa[0], pb, sa[0], sb, out_dtype=torch.float32)
        guard = torch.full((4, N), 777.0, device="cuda")
        c1, c2 = dg.dual_mxfp4_packed(pa[0], pa[1], pb, sa[0], sa[1], sb, out_dtype=torch.float32)
        cb = mg.mxfp4_gemm_packed(pa[1], pb, sa[1], sb)
        mg.gemm_status()
    finally:
        L.ls_gemm_set_variant(0), L.ls_gemm_set_splits(0)
    if K <= 4096:
        assert torch.equal(c.double(), want[0]) and torch.equal(c1.double(), want[0]) and torch.equal(c2.double(), want[1])
        assert torch.equal(cb, want[1].float().bfloat16())
    else:       # sums may pass 2^24 units: fp32 rounding of the partial sums is allowed
        for got, ref in ((c, want[0]), (c1, want[0]), (c2, want[1]), (cb, want[1])):
            _check(got, ref.float().to(got.dtype), f"{M}x{N}x{K} splits {splits}")
    assert (guard == 777.0).all()
    assert L.ls_gemm_set_splits(17) < 0 and L.ls_gemm_set_splits(-1) < 0 and L.ls_gemm_set_variant(4) < 0 and L.ls_gemm_set_variant(7) < 0


@pytest.mark.parametrize("M,N,K,dt", [(256, 512, 384, torch.bfloat16), (130, 256, 256, torch.bfloat16),
                                      (4096, 1024, 1024, torch.bfloat16), (64, 128, 128, torch.float32)])
def test_quantizing_epilogue_equals_separate_pass(mods, M, N, K, dt):
    fp4, mg, _ = mods
    g = torch.Generator(device="cuda").manual_seed(M + K)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    pa, sfa = fp4.quantize_mxfp4_packed(a)
    pw, sfw = fp4.quantize_mxfp4_packed(w)
    plain = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, out_dtype=dt)

    def valid_sf(t):                        # rows past M in the last 128-row tile are padding
        rows = np.arange(M)
        return t.cpu().numpy().reshape(-1, N // 128, 32, 4, 4)[rows // 128, :, rows % 32, (rows % 128) // 32]

    c, q, q_sf = mg.mxfp4_gemm_packed_quant(pa, pw, sfa, sfw, out_dtype=dt)
    mg.gemm_status()
    assert torch.equal(c, plain)
    want_q, want_sf = fp4.quantize_mxfp4_packed(plain)
    assert torch.equal(q, want_q) and np.array_equal(valid_sf(q_sf), valid_sf(want_sf))

    c2, q2, q2_sf = mg.mxfp4_gemm_packed_quant(pa, pw, sfa, sfw, out_dtype=dt, act="gelu", want_c=False)
    mg.gemm_status()
    assert c2 is None
    want_q, want_sf = fp4.quantize_mxfp4_packed(torch.nn.functional.gelu(plain))
    differ = (q2 != want_q).float().mean().item()       # erf of this library vs torch's kernel: same formula
    assert differ <= 1e-4, differ
    if differ == 0:
        assert np.array_equal(valid_sf(q2_sf), valid_sf(want_sf))


def test_fused_mlp_chain(mods):
    # fc -> GELU -> quantize -> out with the activations never leaving MXFP4 between the GEMMs
    fp4, mg, _ = mods
    T, D = 512, 256
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    w1 = (torch.randn(4 * D, D, device="cuda", generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(D, 4 * D, device="cuda", generator=g) * 0.05).bfloat16()
    px, sx = fp4.quantize_mxfp4_packed(x)
    p1, s1 = fp4.quantize_mxfp4_packed(w1)
    p2, s2 = fp4.quantize_mxfp4_packed(w2)
    h = mg.mxfp4_gemm_packed(px, p1, sx, s1)
    ph, sh = fp4.quantize_mxfp4_packed(torch.nn.functional.gelu(h))
    y_ref = mg.mxfp4_gemm_packed(ph, p2, sh, s2)
    _, qh, qsf = mg.mxfp4_gemm_packed_quant(px, p1, sx, s1, act="gelu", want_c=False)
    y = mg.mxfp4_gemm_packed(qh, p2, qsf, s2)
    mg.gemm_status()
    _check(y, y_ref, "fused mlp")


def test_unaligned_views_are_accepted(mods):
    # contiguous slices that start at odd byte offsets: the host layer re-aligns them
    fp4, mg, dg = mods
    g = torch.Generator(device="cuda").manual_seed(1)
    big = torch.randn(129 * 256 + 3, device="cuda", generator=g).bfloat16()
    x = big[3:3 + 129 * 256].view(129, 256)                  # 6 bytes into the allocation
    w = (torch.randn(72, 256, device="cuda", generator=g) * 0.02).bfloat16()
    want = mg.mxfp4_gemm_packed(*sum((list(fp4.quantize_mxfp4_packed(t.clone())) for t in (x, w)), [])[::2],
                                *sum((list(fp4.quantize_mxfp4_packed(t.clone())) for t in (x, w)), [])[1::2])
    pa, sa = fp4.quantize_mxfp4_packed(x)
    pw, sw = fp4.quantize_mxfp4_packed(w)
    pa_off = torch.cat([torch.zeros(1, dtype=torch.uint8, device="cuda"), pa.flatten()])[1:].view_as(pa)
    got = mg.mxfp4_gemm_packed(pa_off, pw, sa, sw)
    assert torch.equal(got, want)
    codes = fp4.unpack_fp4(pa_off)
    assert torch.equal(fp4.pack_fp4(codes), pa)


@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (130, 200, 384), (16, 1000, 1152), (300, 72, 128)])
def test_fp8_entry(mods, M, N, K):
    # reference signature (mxfp4_gemm.py:74-87): A [M, K] and B [K, N] as E4M3 bytes, b_scale [K/32, N];
    # expected value from the oracle's fp64 product of the dequantized operands
    fp4, mg, _ = mods
    g = torch.Generator(device="cuda").manual_seed(3)
    ac = fp4.random_codes((M, K), device="cuda")
    bc = fp4.random_codes((K, N), device="cuda")
    ac[0, :16] = torch.arange(16, dtype=torch.uint8, device="cuda")           # every code, negative zero included
    bc[:16, 0] = torch.arange(16, dtype=torch.uint8, device="cuda")
    sa = torch.exp2(torch.randint(-2, 3, (M, K // 32), device="cuda", generator=g).float())
    sb = torch.exp2(torch.randint(-2, 3, (K // 32, N), device="cuda", generator=g).float())
    c = mg.mxfp4_gemm_fp8(fp4.codes_to_e4m3(ac), fp4.codes_to_e4m3(bc), sa, sb, out_dtype=torch.float32)
    mg.gemm_status()
    want = ref_port.gemm_fp64(ac.cpu(), sa.cpu(), bc.t().contiguous().cpu(), sb.t().contiguous().cpu())
    assert torch.equal(c.cpu().double(), want)              # power-of-two scales, short K: every sum is exact
    cb = mg.mxfp4_gemm_fp8(fp4.codes_to_e4m3(ac), fp4.codes_to_e4m3(bc), sa, sb)
    assert cb.dtype == torch.bfloat16 and torch.equal(cb.cpu(), want.float().bfloat16())


def test_fp8_entry_reports_bytes_off_the_e2m1_grid(mods):
    fp4, mg, _ = mods
    M, N, K = 128, 128, 128
    a = fp4.codes_to_e4m3(fp4.random_codes((M, K), device="cuda"))
    b = fp4.codes_to_e4m3(fp4.random_codes((K, N), device="cuda"))
    ones = torch.ones(M, K // 32, device="cuda")
    for bad_a in (True, False):
        aa, bb = a.clone(), b.clone()
        (aa if bad_a else bb).view(torch.uint8)[5, 7] = 0x31              # 0.5625: an E4M3 value, not an E2M1 one
        mg.mxfp4_gemm_fp8(aa, bb, ones, ones.t().contiguous())
        with pytest.raises(RuntimeError, match="E2M1"):
            mg.gemm_status()
    mg.mxfp4_gemm_fp8(a, b, ones, ones.t().contiguous())
    mg.gemm_status()                                        # clean again


def test_dual_matches_two_singles_and_oracle(mods):
    fp4, mg, dg = mods
    M, N, K = 384, 768, 1024
    g = torch.Generator().manual_seed(11)
    x1 = torch.randn(M, K, generator=g).bfloat16()
    x2 = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    pw, sfw = fp4.quantize_mxfp4_packed(w.cuda())
    c1, c2 = dg.dual_mxfp4(x1.cuda(), x2.cuda(), pw, sfw)
    mg.gemm_status()
    wc, wsc = ref_port.quantize(w)
    for x, c in ((x1, c1), (x2, c2)):
        xc, xs = ref_port.quantize(x)
        _check(c, ref_port.gemm_fake_quant(xc, xs, wc, wsc), "dual")
        p, sf = fp4.quantize_mxfp4_packed(x.cuda())
        assert torch.equal(mg.mxfp4_gemm_packed(p, pw, sf, sfw), c)     # same kernel, same order: same bits


def test_linearity_full_size(mods):
    """Config-2 sized property check (2 x 4096x8192 @ 8192x8192): scaling a
    batch's block scales by 2 doubles its output exactly; the other batch is
    untouched; a sampled set of rows agrees with the oracle."""
    fp4, mg, dg = mods
    M, N, K = 4096, 8192, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    x1 = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    x2 = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    pw, sfw = fp4.quantize_mxfp4_packed(w)
    p1, s1, sc1 = fp4.quantize_mxfp4_packed(x1, want_scale=True)
    p2, s2 = fp4.quantize_mxfp4_packed(x2)
    c1, c2 = dg.dual_mxfp4_packed(p1, p2, pw, s1, s2, sfw, out_dtype=torch.float32)
    d1, d2 = dg.dual_mxfp4_packed(p1, p2, pw, sc1 * 2, s2, sfw, out_dtype=torch.float32)
    mg.gemm_status()
    assert torch.equal(d1, c1 * 2) and torch.equal(d2, c2)
    rows = torch.tensor([0, 1, 127, 128, 2047, 4095])
    wc, wsc = ref_port.quantize(w.cpu())
    for x, c in ((x1, c1), (x2, c2)):
        xc, xs = ref_port.quantize(x[rows.cuda()].cpu())
        _check(c[rows.cuda()], ref_port.gemm_fake_quant(xc, xs, wc, wsc, torch.float32), "config 2 rows")


def test_dependent_launch_chain_matches_ordinary_launches(mods):
    # Short-M products are launched with programmatic stream serialization: a chain in which each
    # product reads what the one before wrote (re-quantized) must give the same bits either way,
    # eagerly and replayed from a CUDA graph
    fp4, mg, _ = mods
    from lockstep_b200 import _lib
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn(16, 1024, device="cuda", generator=g).bfloat16()
    ws = [fp4.quantize_mxfp4_packed((torch.randn(1024, 1024, device="cuda", generator=g) * 0.05).bfloat16()) for _ in range(6)]

    def chain(h):
        for pw, sw in ws:
            ph, sh = fp4.quantize_mxfp4_packed(h)
            h = mg.mxfp4_gemm_packed(ph, pw, sh, sw)
        return h

    def gemm_only_chain(ph, sh):
        outs = []
        for pw, sw in ws:                                    # back-to-back GEMM launches, nothing in between
            outs.append(mg.mxfp4_gemm_packed(ph, pw, sh, sw))
        return outs

    try:
        assert L.ls_gemm_set_pdl(0) == 0
        want = chain(x)
        ph, sh = fp4.quantize_mxfp4_packed(x)
        want_outs = gemm_only_chain(ph, sh)
        assert L.ls_gemm_set_pdl(1) == 0
        got = chain(x)
        got_outs = gemm_only_chain(ph, sh)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            replayed = gemm_only_chain(ph, sh)
            replayed_chain = chain(x)
        graph.replay()
        torch.cuda.synchronize()
        mg.gemm_status()
    finally:
        L.ls_gemm_set_pdl(1)
    assert torch.equal(got, want) and torch.equal(replayed_chain, want)
    for a, b, c in zip(want_outs, got_outs, replayed):
        assert torch.equal(a, b) and torch.equal(a, c)


def test_mma_only_ceiling_kernel_runs_and_counts_its_flops(mods):
    # the measurement aid behind the benchmark's roofline peak: returns the FLOPs of the launch,
    # finishes, and leaves the error word clean
    import ctypes
    from lockstep_b200 import _lib
    L = _lib.lib()
    flop = ctypes.c_double()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _lib.check(L.ls_fp4_mma_peak(64, ctypes.byref(flop), _lib.stream()))
    a.record()
    _lib.check(L.ls_fp4_mma_peak(400, ctypes.byref(flop), _lib.stream()))
    b.record()
    torch.cuda.synchronize()
    mods[1].gemm_status()
    pairs = torch.cuda.get_device_properties(0).multi_processor_count // 2
    assert flop.value == pairs * 400 * 4 * 2.0 * 256 * 256 * 64
    tflops = flop.value / (a.elapsed_time(b) * 1e-3) / 1e12
    assert 1000 < tflops < 9500, tflops                      # between a bf16-class rate and the dense FP4 spec
    assert L.ls_fp4_mma_peak(0, None, None) < 0


def test_split_k_on_two_streams_and_two_host_threads(mods):
    # The split-K scratch is one buffer per device.  Products with forced K splits issued alternately on two
    # streams, and from two host threads at once, give the bits of the same products issued one after another.
    import threading
    fp4, mg, _ = mods
    from lockstep_b200._lib import lib
    g = torch.Generator(device="cuda").manual_seed(31)
    shapes = [(128, 512, 4096), (100, 300, 2304)]
    ops = []
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
        ops.append((*fp4.quantize_mxfp4_packed(a), *fp4.quantize_mxfp4_packed(w)))
    run = lambda o: mg.mxfp4_gemm_packed(o[0], o[2], o[1], o[3], out_dtype=torch.float32)
    try:
        lib().ls_gemm_set_variant(1)
        lib().ls_gemm_set_splits(4)
        want = [run(o) for o in ops]
        torch.cuda.synchronize()
        streams = [torch.cuda.Stream(), torch.cuda.Stream()]
        got = [[], []]
        for it in range(40):                                   # one host thread, alternating streams
            i = it & 1
            with torch.cuda.stream(streams[i]):
                got[i].append(run(ops[i]))
        torch.cuda.synchronize()
        assert all(torch.equal(c, want[i]) for i in (0, 1) for c in got[i])

        def worker(i, out):
            with torch.cuda.stream(streams[i]):
                for _ in range(40):
                    out.append(run(ops[i]))
        outs = [[], []]
        ts = [threading.Thread(target=worker, args=(i, outs[i])) for i in (0, 1)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        torch.cuda.synchronize()
        assert all(len(outs[i]) == 40 and all(torch.equal(c, want[i]) for c in outs[i]) for i in (0, 1))
    finally:
        lib().ls_gemm_set_variant(0)
        lib().ls_gemm_set_splits(0)
    mg.gemm_status()


def test_split_eligible_product_inside_a_cuda_graph(mods):
    # 1024 x 1024 x 16384 is a shape the library splits along K on its own.  Captured into a CUDA graph (after an
    # eager call on another stream has used the split-K scratch) it runs unsplit: the replay gives the bits of
    # the unsplit eager product, and the capture is not invalidated.
    fp4, mg, _ = mods
    from lockstep_b200._lib import lib
    g = torch.Generator(device="cuda").manual_seed(77)
    a = torch.randn(1024, 16384, device="cuda", generator=g).bfloat16()
    w = (torch.randn(1024, 16384, device="cuda", generator=g) * 0.02).bfloat16()
    pa, sa = fp4.quantize_mxfp4_packed(a)
    pw, sw = fp4.quantize_mxfp4_packed(w)
    split = mg.mxfp4_gemm_packed(pa, pw, sa, sw, out_dtype=torch.float32)          # eager, split by the library
    try:
        lib().ls_gemm_set_splits(1)
        unsplit = mg.mxfp4_gemm_packed(pa, pw, sa, sw, out_dtype=torch.float32)
    finally:
        lib().ls_gemm_set_splits(0)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        c = mg.mxfp4_gemm_packed(pa, pw, sa, sw, out_dtype=torch.float32)
    graph.replay()
    torch.cuda.synchronize()
    mg.gemm_status()
    assert torch.equal(c, unsplit)
    _check(c, split, "graph replay against the split product")
