"""GPU parity of the MXFP4 codec kernels (through the C ABI via
lockstep_b200.fp4) against the CPU oracle and the golden vectors: bit-exact."""

import numpy as np
import pytest
import torch

from oracle import cref, ref_port

pytestmark = pytest.mark.gpu
E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


@pytest.fixture(scope="module")
def fp4():
    from lockstep_b200 import fp4 as m
    return m


def _bf16(u16):
    return torch.from_numpy(u16.view(np.int16).copy()).view(torch.bfloat16)


def _np(t):
    return t.cpu().numpy()


def test_tables(fp4, golden):
    t = golden("tables")
    assert fp4.E2M1_VALUES.tolist() == t["values"].tolist()
    assert fp4.E2M1_TO_E4M3.tolist() == t["e4m3"].tolist()
    assert fp4.E2M1_Q.tolist() == t["q"].tolist()
    codes = torch.arange(16, dtype=torch.uint8, device="cuda")
    assert torch.equal(fp4.codes_to_e4m3(codes).float().cpu(), fp4.E2M1_VALUES)
    assert torch.equal(fp4.codes_to_q(codes).float().cpu(), 2 * fp4.E2M1_VALUES)


def test_ties_go_to_smaller_magnitude(fp4):
    # reference tests/test_fp4.py:48-51
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device="cuda")
    got = fp4.E2M1_VALUES[fp4._round_to_e2m1(mids).long().cpu()]
    assert torch.equal(got, torch.tensor(E2M1[:7]))
    assert fp4._round_to_e2m1(-mids).tolist() == [8, 9, 10, 11, 12, 13, 14]
    assert fp4._round_to_e2m1(mids, "rne").tolist() == [0, 2, 2, 4, 4, 6, 6]


def test_round_e2m1_dense_sweep(fp4):
    # every fp32 within 3 ulps of every grid point and midpoint, both signs, + random
    pts = np.array([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6, 7, 8], np.float32)
    u = pts.view(np.uint32)[:, None] + np.arange(-3, 4, dtype=np.int64)[None, :]
    u = u[u >= 0].astype(np.uint32)
    vals = np.concatenate([u.view(np.float32), -u.view(np.float32),
                           np.random.default_rng(1).normal(0, 3, 100000).astype(np.float32),
                           np.array([np.inf, -np.inf, 1e-45, -1e-45, 1e30], np.float32)])
    q = torch.from_numpy(vals)
    for mode in ("ref", "rne"):
        want = ref_port.round_e2m1(q, mode)
        got = fp4._round_to_e2m1(q.cuda(), mode).cpu()
        assert torch.equal(got, want), mode


def test_pack_unpack_roundtrip(fp4):
    # reference tests/test_fp4.py:34-39
    codes = fp4.random_codes((7, 64), device="cuda")
    packed = fp4.pack_fp4(codes)
    assert packed.shape == (7, 32)
    assert torch.equal(fp4.unpack_fp4(packed), codes)
    assert torch.equal(packed[0, 0] & 0x0F, codes[0, 0])
    for shape in [(1, 2), (3, 6), (5, 46), (1, 16), (129, 258), (1024, 4096)]:
        c = torch.randint(0, 16, shape, dtype=torch.uint8, device="cuda")
        p = fp4.pack_fp4(c)
        assert np.array_equal(_np(p), cref.pack(_np(c)))
        assert torch.equal(fp4.unpack_fp4(p), c)
    assert fp4.pack_fp4(torch.empty(0, 32, dtype=torch.uint8, device="cuda")).shape == (0, 16)


def test_random_codes_skip_negative_zero(fp4):
    codes = fp4.random_codes((20000,), device="cuda")
    assert not (codes == 8).any()
    assert set(codes.unique().tolist()) == {c for c in range(16) if c != 8}


def test_quantize_adversarial_f32(fp4, golden):
    gd = golden("quant_adversarial_f32")
    x = torch.from_numpy(gd["x"].view(np.float32).copy()).cuda()
    codes, scale = fp4.quantize_mxfp4(x)
    assert np.array_equal(_np(codes), gd["codes"])
    assert np.array_equal(_np(scale).view(np.uint32), gd["scale"])
    assert np.array_equal(_np(fp4.pack_fp4(codes)), gd["packed"])


def test_quantize_adversarial_as_bf16(fp4, golden):
    # the same rows rounded to bf16 exercise the converter path of the bf16 kernel
    gd = golden("quant_adversarial_f32")
    xb = torch.from_numpy(gd["x"].view(np.float32).copy()).bfloat16()
    want_c, want_s = ref_port.quantize(xb)
    codes, scale = fp4.quantize_mxfp4(xb.cuda())
    assert torch.equal(scale.cpu(), want_s)
    assert torch.equal(codes.cpu(), want_c)
    want_c, want_s = ref_port.quantize(xb, rounding="rne")
    codes, scale = fp4.quantize_mxfp4(xb.cuda(), rounding="rne")
    assert torch.equal(codes.cpu(), want_c)


def test_quantize_every_bf16_tie(fp4):
    # all bf16 values whose quotient by the block scale is an E2M1 midpoint or
    # grid point, at several exponents, with the block maximum pinned at 4.0*2^e
    mids = torch.tensor([.25, .75, 1.25, 1.75, 2.5, 3.5, 5.0, 0, .5, 1, 1.5, 2, 3, 6, 7, 7.5])
    rows = []
    for e in (-120, -30, -2, 0, 3, 60, 120):
        for sgn in (1.0, -1.0):
            r = torch.cat([mids * sgn, -mids[:15] * sgn, torch.tensor([4.0])]) * 2.0 ** e
            rows.append(r)
    x = torch.stack(rows).bfloat16()
    assert x.shape[1] == 32
    want_c, want_s = ref_port.quantize(x)
    codes, scale = fp4.quantize_mxfp4(x.cuda())
    assert torch.equal(scale.cpu(), want_s) and torch.equal(codes.cpu(), want_c)


def test_quantize_nan_block(fp4, golden):
    gd = golden("quant_nan_f32")
    x = torch.from_numpy(gd["x"].view(np.float32).copy())
    for inp in (x, x.bfloat16()):
        want_c, want_s = ref_port.quantize(inp)
        codes, scale = fp4.quantize_mxfp4(inp.cuda())
        codes, scale = codes.cpu(), scale.cpu()
        assert torch.equal(torch.isnan(scale), torch.isnan(want_s))
        ok = ~torch.isnan(want_s)
        assert torch.equal(scale[ok], want_s[ok])
        okb = ok.repeat_interleave(32, -1)
        assert torch.equal(codes[okb], want_c[okb])
        assert ((codes[~okb] & 7) == 7).all()


def test_quantize_bf16_golden(fp4, golden):
    gd = golden("quant_gemm_bf16")
    a = _bf16(gd["a"]).cuda()
    codes, scale = fp4.quantize_mxfp4(a)
    assert np.array_equal(_np(codes), gd["a_codes"]) and np.array_equal(_np(scale), gd["a_scale"])
    assert np.array_equal(_np(fp4.pack_fp4(codes)), gd["a_packed"])
    assert np.array_equal(_np(fp4.dequantize_mxfp4(codes, scale)), gd["a_deq"])
    c16, s16 = fp4.quantize_mxfp4(a, 16)
    assert np.array_equal(_np(c16), gd["a_codes16"]) and np.array_equal(_np(s16), gd["a_scale16"])
    w = _bf16(gd["w"]).cuda()
    wc, ws = fp4.quantize_mxfp4(w)
    assert np.array_equal(_np(wc), gd["w_codes"]) and np.array_equal(_np(ws), gd["w_scale"])
    ref = fp4.reference_mxfp4_gemm(codes, scale, wc.t(), ws.t())
    assert torch.allclose(ref.cpu(), torch.from_numpy(gd["out_ref_f32"]), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("block", [16, 32])
def test_quantize_logspace_properties(fp4, golden, block):
    # reference tests/test_fp4.py:54-68
    gd = golden(f"quant_logspace_b{block}")
    x = torch.from_numpy(gd["x"]).cuda()
    codes, scale = fp4.quantize_mxfp4(x, block)
    assert np.array_equal(_np(codes), gd["codes"]) and np.array_equal(_np(scale), gd["scale"])
    assert torch.equal(torch.exp2(torch.log2(scale).round()), scale)
    xb = x.reshape(64, -1, block)
    amax = xb.abs().amax(-1)
    assert ((amax / scale >= 4 * (1 - 1e-6)) & (amax / scale < 8)).all()
    y = fp4.dequantize_mxfp4(codes, scale, block).reshape(64, -1, block)
    assert (((y - xb).abs() / scale.unsqueeze(-1)) <= 2.0 + 1e-6).all()


def test_zero_block_is_exact(fp4):
    # reference tests/test_fp4.py:71-74
    codes, scale = fp4.quantize_mxfp4(torch.zeros(2, 32, device="cuda"))
    assert torch.equal(scale.cpu(), torch.ones(2, 1))
    assert torch.equal(fp4.dequantize_mxfp4(codes, scale).cpu(), torch.zeros(2, 32))
    assert fp4.quantize_mxfp4(torch.zeros(0, 64, device="cuda"))[0].shape == (0, 64)


def test_block_must_divide(fp4):
    with pytest.raises(AssertionError):
        fp4.quantize_mxfp4(torch.zeros(2, 48, device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 32), (3, 96), (257, 1024), (2048, 4096)])
def test_quantize_random_vs_c_oracle(fp4, dtype, shape):
    g = torch.Generator().manual_seed(hash((str(dtype), shape)) % 2 ** 31)
    x = torch.randn(shape, generator=g) * torch.exp2(torch.randint(-40, 40, (shape[0], 1), generator=g).float())
    mask = torch.rand(shape, generator=g) < 0.01
    x = torch.where(mask, x * 50, x).to(dtype)
    want = cref.quantize(x.float().numpy())
    codes, scale = fp4.quantize_mxfp4(x.cuda())
    assert np.array_equal(_np(codes), want["codes"])
    assert np.array_equal(_np(scale), want["scale"])
    if shape[1] % 128 == 0:
        packed, sf, sc = fp4.quantize_mxfp4_packed(x.cuda(), want_scale=True)
        assert np.array_equal(_np(packed), want["packed"])
        assert np.array_equal(_np(sc), want["scale"])
        # scale-factor layout: 128-row x 4-block tiles, k-tiles innermost
        rows, K = shape
        e = want["e8m0"]
        sf = _np(sf).reshape(-1, K // 128, 32, 4, 4)          # [rt, kt, r%32, r/32, kb%4]
        r = np.arange(rows)
        for kb in range(K // 32):
            assert np.array_equal(sf[r // 128, kb // 4, r % 32, (r % 128) // 32, kb % 4], e[:, kb])
        sf2, bad = fp4.scales_to_sf(sc)
        assert int(bad.item()) == 0
        sf2 = _np(sf2).reshape(-1, K // 128, 32, 4, 4)
        for kb in range(K // 32):
            assert np.array_equal(sf2[r // 128, kb // 4, r % 32, (r % 128) // 32, kb % 4], e[:, kb])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,C", [(128, 64), (256, 100), (384, 1000), (1024, 4096), (2048, 4100), (4096, 2048)])
def test_transposed_quantizer_equals_quantizer_of_transpose(fp4, dtype, R, C, golden):
    g = torch.Generator().manual_seed(R + C)
    x = torch.randn(R, C, generator=g) * torch.exp2(torch.randint(-20, 20, (1, C), generator=g).float())
    x = torch.where(torch.rand(R, C, generator=g) < 0.01, x * 50, x)
    if R == 128:                                   # adversarial rows of the golden set as columns
        adv = torch.from_numpy(golden("quant_adversarial_f32")["x"].view(np.float32).copy())[:C * 4]
        x = adv.reshape(C, 4 * 32).t().contiguous()
    x = x.to(dtype)
    want = cref.quantize(x.t().contiguous().float().numpy())
    packed, sf, scale = fp4.quantize_mxfp4_packed_t(x.cuda(), want_scale=True)
    assert np.array_equal(_np(packed), want["packed"])
    assert np.array_equal(_np(scale), want["scale"])
    p2, sf2 = fp4.quantize_mxfp4_packed(x.t().contiguous().cuda())
    assert torch.equal(packed, p2)
    rows = np.arange(C)                            # rows past C in the last 128-row tile are padding
    a, b = (_np(t).reshape(-1, R // 128, 32, 4, 4)[rows // 128, :, rows % 32, (rows % 128) // 32] for t in (sf, sf2))
    assert np.array_equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,C", [(128, 128), (256, 384), (1024, 4096), (4096, 1024)])
def test_both_orientations_from_one_read(fp4, dtype, R, C, golden):
    # one kernel, x read once: bit-identical to the row-wise and the transposed quantizer
    g = torch.Generator().manual_seed(R * 3 + C)
    x = torch.randn(R, C, generator=g) * torch.exp2(torch.randint(-20, 20, (R, 1), generator=g).float())
    x = torch.where(torch.rand(R, C, generator=g) < 0.01, x * 50, x)
    if R == 128:                                   # adversarial rows of the golden set (ties, exponent quirk, inf)
        adv = torch.from_numpy(golden("quant_adversarial_f32")["x"].view(np.float32).copy()).reshape(-1)
        k = min(R, adv.numel() // C)
        x[:k] = adv[:k * C].reshape(k, C)
    x = x.to(dtype).cuda()
    for rounding in ("ref", "rne"):
        p, s, pt, st = fp4.quantize_mxfp4_both(x, rounding)
        p1, s1 = fp4.quantize_mxfp4_packed(x, rounding=rounding)
        p2, s2 = fp4.quantize_mxfp4_packed_t(x, rounding=rounding)
        assert torch.equal(p, p1) and torch.equal(pt, p2)
        assert torch.equal(s, s1) and torch.equal(st, s2)          # both dimensions are multiples of 128: no padding bytes
    with pytest.raises(AssertionError):
        fp4.quantize_mxfp4_both(x[:, :96].contiguous())


def test_fp32_exponent_rule_on_gpu(fp4):
    # block maxima a few ulps below powers of two: fp32 log2 rounds up
    vals = []
    for k in range(-98, 128):
        top = np.array([2.0 ** k], np.float32).view(np.uint32)[0]
        vals += [top - n for n in range(0, 48)]
    a = np.array(vals, np.uint32).view(np.float32)
    x = np.zeros((a.size, 32), np.float32)
    x[:, 0] = a
    x[:, 1] = -a / 3
    want = cref.quantize(x)
    codes, scale = fp4.quantize_mxfp4(torch.from_numpy(x).cuda())
    assert np.array_equal(_np(scale), want["scale"]) and np.array_equal(_np(codes), want["codes"])


def test_dequantize_matches_oracle(fp4):
    codes = torch.randint(0, 16, (64, 256), dtype=torch.uint8)
    scale = torch.exp2(torch.randint(-20, 20, (64, 8)).float())
    want = ref_port.dequantize(codes, scale)
    got = fp4.dequantize_mxfp4(codes.cuda(), scale.cuda()).cpu()
    assert torch.equal(got, want)
    assert torch.equal(torch.signbit(got), torch.signbit(want))      # code 8 is -0.0


def test_large_roundtrip_property(fp4):
    """Full-size property check (4096 x 8192 bf16): dequantize(quantize(x)) is
    a fixed point of the quantizer, and pack/unpack round-trips."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(4096, 8192, device="cuda", generator=g, dtype=torch.float32).bfloat16()
    codes, scale = fp4.quantize_mxfp4(x)
    y = fp4.dequantize_mxfp4(codes, scale)
    codes2, scale2 = fp4.quantize_mxfp4(y)
    nz = (codes & 7) != 0                      # a block whose maximum rounds up renormalises
    same = torch.equal(scale2, scale)
    assert torch.equal(fp4.unpack_fp4(fp4.pack_fp4(codes)), codes)
    amax = x.float().reshape(4096, -1, 32).abs().amax(-1)
    assert ((amax / scale >= 4) & (amax / scale < 8) | (amax == 0)).all()
    assert (((y - x.float()).abs().reshape(4096, -1, 32) / scale.unsqueeze(-1)) <= 2.0).all()
    if same:
        assert torch.equal(codes2[nz], codes[nz])
    packed, sf = fp4.quantize_mxfp4_packed(x)
    assert torch.equal(packed, fp4.pack_fp4(codes))
