"""Parity at the sizes the benchmark times.

The benchmark's numbers are only worth quoting if the launches it times give
the reference's results, so each timed configuration is held to the CPU oracle
here at full size:

* the dual-batch launch 2 x [4096 x 8192] @ [8192 x 8192] -> bf16, the output
  type the benchmark times: 9 rows of every 128-row tile of both batches (all
  four tensor-memory lane quarters of both CTAs of every pair), all 8192
  columns, against dequantize + fp32 F.linear -> bf16 (fp4_linear.py:38-40);
* every cell of the shape sweep M in {1, 16, 128, 4096, 16384} x N = K in
  {4096, 8192, 16384} (1 % outliers x 50 in the activations) on sampled rows
  and sampled output columns that cover the first and last tiles and the
  128 / 256-column tile edges;
* the GEMM on operands with scale blocks of 16 (UE8M0 scales, and E4M3 scales =
  NVFP4) at 8192 x 8192 x 8192, the shape their timings are quoted on, on
  sampled rows and columns against the oracles' dequantize + fp32 matmul;
* one 64 Mi-element step sequence of the FP4 wire with error feedback at world
  size 1 (32-bit group indices near their top, the multi-CTA-per-SM grids,
  the tail logic of the decode kernel), bit for bit against the C oracle.

Tolerance of the GEMMs, as everywhere: rel-L2 <= 1e-3 and max-abs <=
2e-2 * ||row||_inf with both sides in the same output type."""

import numpy as np
import pytest
import torch

from oracle import cref, ref_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    from lockstep_b200 import dual_gemm, fp4, mxfp4_gemm
    yield fp4, mxfp4_gemm, dual_gemm
    mxfp4_gemm.gemm_status()


def _check(c, ref, what):
    c, ref = c.float().cpu(), ref.float().cpu()
    rel = ((c - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    row_inf = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)
    worst = ((c - ref).abs() / row_inf).max().item()
    assert rel <= 1e-3 and worst <= 2e-2, f"{what}: rel-L2 {rel:.3e}, max-abs/row-inf {worst:.3e}"


def _tile_rows(M, per_tile_extra, gen):
    """Rows that touch every lane quarter of every 128-row tile (first and last row of
    each quarter) plus random ones; all rows when M is small."""
    if M <= 128:
        return torch.arange(M)
    rows = []
    for mt in range((M + 127) // 128):
        base = mt * 128
        cand = [0, 31, 32, 63, 64, 95, 96, 127]
        cand += torch.randint(0, 128, (per_tile_extra,), generator=gen).tolist()
        rows += [base + r for r in cand if base + r < M]
    return torch.tensor(sorted(set(rows)))


def test_config2_bf16_full_size_vs_oracle(mods):
    fp4, mg, dg = mods
    M, N, K = 4096, 8192, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    xs = torch.randn(2, M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    pw, sfw = fp4.quantize_mxfp4_packed(w)
    c1, c2 = dg.dual_mxfp4(xs[0], xs[1], pw, sfw)             # the call the benchmark times
    mg.gemm_status()
    assert c1.dtype == torch.bfloat16 and c1.shape == (M, N)
    wc, wsc = ref_port.quantize(w.cpu())
    assert torch.equal(fp4.unpack_fp4(pw).cpu(), wc)           # same weight bits on both sides
    wd = ref_port.dequantize(wc, wsc)
    del wc, wsc
    rows = _tile_rows(M, 1, torch.Generator().manual_seed(1))
    assert rows.numel() >= 256
    for b, c in enumerate((c1, c2)):
        xc, xsc = ref_port.quantize(xs[b][rows.cuda()].cpu())
        ref = torch.nn.functional.linear(ref_port.dequantize(xc, xsc), wd).to(torch.bfloat16)
        _check(c[rows.cuda()], ref, f"config 2 batch {b}")


_SWEEP = [(m, nk) for nk in (4096, 8192, 16384) for m in (1, 16, 128, 4096, 16384)]
_weights = {}


def _sweep_weight(fp4, nk):
    if nk not in _weights:
        _weights.clear()                                      # one weight resident at a time
        g = torch.Generator(device="cuda").manual_seed(nk)
        w = (torch.randn(nk, nk, device="cuda", generator=g) * 0.02).bfloat16()
        _weights[nk] = (w, *fp4.quantize_mxfp4_packed(w))
    return _weights[nk]


@pytest.mark.parametrize("M,NK", _SWEEP)
def test_shape_sweep_cell_vs_oracle(mods, M, NK):
    fp4, mg, _ = mods
    w, pw, sfw = _sweep_weight(fp4, NK)
    g = torch.Generator(device="cuda").manual_seed(M + NK)
    a = torch.randn(M, NK, device="cuda", generator=g)
    a = torch.where(torch.rand(M, NK, device="cuda", generator=g) < 0.01, a * 50, a).bfloat16()
    pa, sfa = fp4.quantize_mxfp4_packed(a)
    c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw)
    mg.gemm_status()
    cg = torch.Generator().manual_seed(7)
    rows = _tile_rows(M, 0, cg)
    if rows.numel() > 64:                                     # first, second, last two tiles + a random sample
        keep = rows[(rows < 256) | (rows >= M - 256)]
        rest = rows[(rows >= 256) & (rows < M - 256)]
        rows = torch.cat([keep, rest[torch.randperm(rest.numel(), generator=cg)[:32]]]).sort().values
    edge = [0, 1, 31, 32, 127, 128, 129, 255, 256, 257, 383, 384, 511, 512, NK - 257, NK - 256, NK - 129, NK - 128,
            NK - 33, NK - 32, NK - 1]
    cols = torch.tensor(sorted(set(edge + torch.randint(0, NK, (235,), generator=cg).tolist())))
    ac, asc = ref_port.quantize(a[rows.cuda()].cpu())
    wc, wsc = ref_port.quantize(w[cols.cuda()].cpu())
    ref = ref_port.gemm_fake_quant(ac, asc, wc, wsc)
    _check(c[rows.cuda()][:, cols.cuda()], ref, f"sweep cell {M} x {NK} x {NK}")


@pytest.mark.parametrize("fmt", ["mxfp4-b16", "nvfp4"])
def test_block16_formats_at_the_timed_size_vs_oracle(mods, fmt):
    # 8192 x 8192 x 8192, the shape `bench.py --shape ... --format` and the benchmark's own NVFP4 comparison time:
    # the CTA-pair kernel with 64 shared accumulator columns, every row-tile pair and column tile of it sampled
    fp4, mg, _ = mods
    from lockstep_b200 import nvfp4
    from oracle import nvfp4_ref
    M = N = K = 8192
    g = torch.Generator(device="cuda").manual_seed(16)
    a = torch.randn(M, K, device="cuda", generator=g)
    a = torch.where(torch.rand(M, K, device="cuda", generator=g) < 0.01, a * 50, a).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    cg = torch.Generator().manual_seed(7)
    rows = _tile_rows(M, 0, cg)
    rows = rows[torch.randperm(rows.numel(), generator=cg)[:96]].sort().values
    rows = torch.cat([torch.tensor([0, 127, 128, 255, 256, M - 257, M - 256, M - 1]), rows]).unique()
    edge = [0, 1, 31, 32, 127, 128, 191, 192, 223, 224, 255, 256, 257, 447, 448, 511, 512, N - 257, N - 256, N - 65, N - 64, N - 1]
    cols = torch.tensor(sorted(set(edge + torch.randint(0, N, (234,), generator=cg).tolist())))
    if fmt == "nvfp4":
        pa, _, sfa = nvfp4.quantize_nvfp4(a)
        pw, _, sfw = nvfp4.quantize_nvfp4(w)
        c = nvfp4.nvfp4_gemm_packed(pa, pw, sfa, sfw)
        ac, asc = nvfp4_ref.quantize(a[rows.cuda()].float().cpu().numpy())
        wc, wsc = nvfp4_ref.quantize(w[cols.cuda()].float().cpu().numpy())
        assert np.array_equal(fp4.unpack_fp4(pa[rows.cuda()]).cpu().numpy(), ac)
        ref = torch.nn.functional.linear(torch.from_numpy(nvfp4_ref.dequantize(ac, asc)),
                                         torch.from_numpy(nvfp4_ref.dequantize(wc, wsc))).to(torch.bfloat16)
    else:
        pa, sfa = fp4.quantize_mxfp4_packed(a, block=16)
        pw, sfw = fp4.quantize_mxfp4_packed(w, block=16)
        c = mg.mxfp4_gemm_packed(pa, pw, sfa, sfw, block=16)
        ac, asc = ref_port.quantize(a[rows.cuda()].cpu(), block=16)
        wc, wsc = ref_port.quantize(w[cols.cuda()].cpu(), block=16)
        assert torch.equal(fp4.unpack_fp4(pa[rows.cuda()]).cpu(), ac)
        ref = torch.nn.functional.linear(ref_port.dequantize(ac, asc, 16), ref_port.dequantize(wc, wsc, 16)).to(torch.bfloat16)
    mg.gemm_status()
    _check(c[rows.cuda()][:, cols.cuda()], ref, f"{fmt} 8192^3")


def test_sweep_weights_released():
    _weights.clear()
    torch.cuda.empty_cache()


def test_wire_64mi_one_rank_error_feedback_vs_oracle():
    from lockstep_b200 import wire
    n = 64 << 20
    w = wire.Wire("mxfp4ef", n)
    res_c, ores_c = [np.zeros(n, np.float32)], [np.zeros(n, np.float32)]
    gen = torch.Generator(device="cuda").manual_seed(100)
    for step in range(3):
        z = torch.randn(n, device="cuda", generator=gen)
        chi = torch.zeros(n, device="cuda")
        for _ in range(3):
            chi += torch.randn(n, device="cuda", generator=gen) ** 2
        grad = z / (chi / 3).sqrt() * 1e-3                      # Student-t(3) * 1e-3
        del z, chi
        host = grad.cpu().numpy()
        want, _, _ = cref.wire_step([host], res_c, ores_c, unit=256)
        out = w(grad)
        w.status()
        assert np.array_equal(out.cpu().numpy(), want), f"step {step}: g differs"
        assert np.array_equal(w.res.cpu().numpy()[:n], res_c[0]), f"step {step}: sender residual differs"
        assert np.array_equal(w.ores.cpu().numpy().reshape(-1)[:n], ores_c[0]), f"step {step}: owner residual differs"
        del grad, out, want, host
    w.close()
