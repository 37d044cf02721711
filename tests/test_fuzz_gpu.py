"""Seeded random shapes through every GEMM entry of the C ABI: M and N of any
residue (odd output widths, single rows, one past a tile edge), K any multiple
of 128, both output types, single and dual batch, scale blocks of 32 and 16 and
NVFP4.  Each case is held to the oracle's dequantize + fp32 matmul within the
GEMM tolerance (rel-L2 <= 1e-3, max-abs <= 2e-2 * ||row||_inf, same output
type), and a guard band around the output buffer must come back untouched."""

import numpy as np
import pytest
import torch

from oracle import nvfp4_ref, ref_port

pytestmark = pytest.mark.gpu


def _cases(n, seed):
    rng = np.random.default_rng(seed)
    edges = [1, 2, 7, 16, 31, 33, 64, 65, 127, 128, 129, 255, 256, 257, 383, 385, 511, 513]
    out = []
    for i in range(n):
        M = int(rng.choice(edges)) if rng.random() < 0.6 else int(rng.integers(1, 700))
        N = int(rng.choice(edges)) if rng.random() < 0.6 else int(rng.integers(1, 900))
        K = 128 * int(rng.integers(1, 14))
        out.append((M, N, K, ["mxfp4", "mxfp4-b16", "nvfp4"][i % 3], bool(rng.random() < 0.35), bool(rng.random() < 0.5)))
    return out


def _check(c, ref, what):
    c, ref = c.float().cpu(), ref.float().cpu()
    rel = ((c - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    row_inf = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    worst = ((c - ref).abs() / row_inf).max().item()
    assert rel <= 1e-3 and worst <= 2e-2, f"{what}: rel-L2 {rel:.3e}, max-abs/row-inf {worst:.3e}"


@pytest.mark.parametrize("M,N,K,fmt,dual,f32", _cases(48, 2024))
def test_random_shape(M, N, K, fmt, dual, f32):
    from lockstep_b200 import fp4, mxfp4_gemm as mg, nvfp4
    from lockstep_b200._lib import check, dtype_code, lib, ptr, stream
    g = torch.Generator().manual_seed(M * 1000003 + N * 1009 + K)
    dt = torch.float32 if f32 else torch.bfloat16
    xs = [torch.randn(M, K, generator=g).bfloat16() for _ in range(2 if dual else 1)]
    xs = [torch.where(torch.rand(M, K, generator=g) < 0.01, x * 50, x) for x in xs]
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    if fmt == "nvfp4":
        quant = lambda t: nvfp4.quantize_nvfp4(t.cuda())[::2]
        def oracle(a):
            ac, asc = nvfp4_ref.quantize(a.float().numpy())
            wc, wsc = nvfp4_ref.quantize(w.float().numpy())
            return torch.nn.functional.linear(torch.from_numpy(nvfp4_ref.dequantize(ac, asc)),
                                              torch.from_numpy(nvfp4_ref.dequantize(wc, wsc))).to(dt)
        single, both = lib().ls_nvfp4_gemm, lib().ls_nvfp4_gemm_dual
    else:
        block = 16 if fmt == "mxfp4-b16" else 32
        quant = lambda t: fp4.quantize_mxfp4_packed(t.cuda(), block=block)
        def oracle(a):
            ac, asc = ref_port.quantize(a, block=block)
            wc, wsc = ref_port.quantize(w, block=block)
            return torch.nn.functional.linear(ref_port.dequantize(ac, asc, block), ref_port.dequantize(wc, wsc, block)).to(dt)
        single = lib().ls_mxfp4_gemm if block == 32 else lib().ls_mxfp4_gemm_block16
        both = lib().ls_mxfp4_gemm_dual if block == 32 else lib().ls_mxfp4_gemm_dual_block16
    pw, sfw = quant(w)
    qs = [quant(x) for x in xs]
    # outputs inside one buffer with guard rows before, between and after
    pad = 16
    buf = torch.full(((M + pad) * len(xs) + pad, N), 777.0, device="cuda", dtype=dt)
    outs = [buf[pad + i * (M + pad): pad + i * (M + pad) + M] for i in range(len(xs))]
    assert all(o.data_ptr() % 16 == 0 for o in outs) or N % 8 != 0
    if any(o.data_ptr() % 16 for o in outs):                   # odd widths: the guard layout would misalign the outputs
        outs = [torch.full((M, N), 777.0, device="cuda", dtype=dt) for _ in xs]
    if dual:
        check(both(ptr(qs[0][0]), ptr(qs[1][0]), ptr(pw), ptr(qs[0][1]), ptr(qs[1][1]), ptr(sfw), ptr(outs[0]), ptr(outs[1]),
                   dtype_code(dt), M, N, K, stream()))
    else:
        check(single(ptr(qs[0][0]), ptr(pw), ptr(qs[0][1]), ptr(sfw), ptr(outs[0]), dtype_code(dt), M, N, K, stream()))
    mg.gemm_status()
    for x, o in zip(xs, outs):
        _check(o, oracle(x), f"{fmt} {M}x{N}x{K} dual={dual} {dt}")
    if outs[0].data_ptr() >= buf.data_ptr() and outs[0].data_ptr() < buf.data_ptr() + buf.numel() * buf.element_size():
        mask = torch.ones(buf.shape[0], dtype=torch.bool)
        for i in range(len(xs)):
            mask[pad + i * (M + pad): pad + i * (M + pad) + M] = False
        assert (buf[mask.cuda()] == 777.0).all(), "a store landed outside the output rows"


def _special_mix(rows, K, seed):
    """Normal data over many binades with zeros, signed zeros, subnormals, huge values, infinities and NaNs sprinkled in."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, K, generator=g) * torch.exp2(torch.randint(-20, 20, (rows, 1), generator=g).float())
    u = torch.rand(rows, K, generator=g)
    x = torch.where(u < 0.02, torch.zeros(()), x)
    x = torch.where((u >= 0.02) & (u < 0.03), -torch.zeros(()), x)
    x = torch.where((u >= 0.03) & (u < 0.035), x * 1e-38, x)
    x = torch.where((u >= 0.035) & (u < 0.04), x * 1e30, x)
    x = torch.where((u >= 0.04) & (u < 0.042), torch.full((), float("inf")), x)
    x = torch.where((u >= 0.042) & (u < 0.044), torch.full((), float("-inf")), x)
    x = torch.where((u >= 0.044) & (u < 0.046), torch.full((), float("nan")), x)
    # whole blocks of zeros and of one repeated value (ties everywhere)
    x[0, :32] = 0
    x[-1, -32:] = 1.75
    return x


@pytest.mark.parametrize("case", range(12))
def test_random_quantizer_inputs_bit_exact(case):
    from lockstep_b200 import fp4, nvfp4
    rng = np.random.default_rng(100 + case)
    rows, K = int(rng.integers(1, 300)), 128 * int(rng.integers(1, 9))
    x = _special_mix(rows, K, case)
    for dt in (torch.float32, torch.bfloat16):
        xd = x.to(dt)
        for block in (32, 16):
            packed, sf, scale = fp4.quantize_mxfp4_packed(xd.cuda(), want_scale=True, block=block)
            codes, want = ref_port.quantize(xd, block=block)
            got = scale.cpu()
            same = (got == want) | (got.isnan() & want.isnan())
            assert same.all(), (case, dt, block)
            live = ~want.isnan().repeat_interleave(block, dim=-1)                       # codes of a NaN block are unspecified
            assert torch.equal(fp4.unpack_fp4(packed).cpu()[live], codes[live]), (case, dt, block)
        packed, scale, _ = nvfp4.quantize_nvfp4(xd.cuda())
        codes, want = nvfp4_ref.quantize(xd.float().numpy())
        assert np.array_equal(scale.cpu().numpy().view(np.uint32), want.view(np.uint32)), (case, dt)
        assert np.array_equal(fp4.unpack_fp4(packed).cpu().numpy(), codes), (case, dt)
