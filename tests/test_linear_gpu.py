"""GPU parity of the MXFP4 linear layer: forward against the reference's
fake-quant path (golden output of the real fp4_linear.MXFP4Linear), the
straight-through backward against the reference's gradients, and the MXFP4
backward against its oracle composition (quantize along the contracted axis,
dequantize, fp32 matmul)."""

import numpy as np
import pytest
import torch

from oracle import ref_port

pytestmark = pytest.mark.gpu


def _bf16(u16):
    return torch.from_numpy(u16.view(np.int16).copy()).view(torch.bfloat16)


def _close(got, ref, what, rel_tol=1e-3):
    got, ref = got.float().cpu(), ref.float().cpu()
    rel = ((got - ref).norm() / ref.norm()).item()
    assert rel <= rel_tol, f"{what}: rel-L2 {rel:.3e}"


def test_forward_and_ste_backward_against_reference_golden(golden):
    from lockstep_b200 import fp4_linear
    gd = golden("linear_ste")
    lin = fp4_linear.MXFP4Linear(256, 160).cuda()
    assert fp4_linear.FP4Linear is fp4_linear.MXFP4Linear and fp4_linear.path() == "tcgen05-mxfp4"
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(gd["w"]))
    x = _bf16(gd["x"]).cuda().requires_grad_(True)
    y = lin(x)
    assert y.shape == (4, 24, 160) and y.dtype == torch.bfloat16
    _close(y, _bf16(gd["y"]), "forward")
    worst = ((y.float().cpu() - _bf16(gd["y"]).float()).abs().reshape(-1, 160) /
             _bf16(gd["y"]).float().abs().reshape(-1, 160).amax(1, keepdim=True)).max().item()
    assert worst <= 2e-2
    y.backward(_bf16(gd["gy"]).cuda())
    _close(x.grad, _bf16(gd["gx"]), "dX (ste)", 1e-2)          # bf16 matmuls, different GEMM library
    _close(lin.weight.grad, torch.from_numpy(gd["gw"]), "dW (ste)", 1e-2)
    with pytest.raises(AssertionError):
        fp4_linear.MXFP4Linear(8, 8, bias=True)


def test_autocast_dtype_follows_reference():
    from lockstep_b200 import fp4_linear
    lin = fp4_linear.MXFP4Linear(128, 128).cuda()
    x = torch.randn(4, 128, device="cuda")
    with torch.autocast("cuda", torch.bfloat16):
        assert lin(x).dtype == torch.bfloat16                 # fp4_linear.py:56
    assert lin(x).dtype == torch.float32


def test_mxfp4_backward_against_oracle():
    from lockstep_b200 import fp4_linear
    T, K, N = 256, 384, 512
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = torch.randn(N, K, generator=g) * 0.02
    gy = torch.randn(T, N, generator=g).bfloat16()
    lin = fp4_linear.MXFP4Linear(K, N, backward="mxfp4").cuda()
    with torch.no_grad():
        lin.weight.copy_(w)
    xin = x.cuda().requires_grad_(True)
    lin(xin).backward(gy.cuda())

    def fq(t):                                                 # quantize along the last axis, dequantize
        return ref_port.dequantize(*ref_port.quantize(t))
    gx_ref = fq(gy) @ fq(w.t().contiguous()).t()               # contract over N
    gw_ref = fq(gy.t().contiguous()) @ fq(x.t().contiguous()).t()   # contract over tokens
    _close(xin.grad, gx_ref.bfloat16(), "dX (mxfp4)")
    _close(lin.weight.grad, gw_ref, "dW (mxfp4)")


def test_tiny_decoder_trains():
    import train_bench
    kw = dict(layers=2, width=256, heads=4, context=128, batch=8, vocab=512)
    for kind in ("mxfp4", "ste"):
        t = train_bench.Trainer(kind, **kw)
        _, loss0 = t.time(steps=1, warmup=0)
        _, loss1 = t.time(steps=8, warmup=0)
        t.close()
        assert np.isfinite(loss1) and loss1 < loss0           # the loss goes down on a repeated batch


def test_bucketed_sync_sends_under_backward_and_trains_alike():
    # the flat gradient buffer averaged by one Wire after backward (train.py:124-138) against the
    # bucketed form whose send phases run on a side stream during backward
    import train_bench
    kw = dict(layers=2, width=256, heads=4, context=128, batch=8, vocab=512)
    losses = {}
    for overlap in (False, True):
        t = train_bench.Trainer("mxfp4", overlap=overlap, buckets=3, **kw)
        assert (len(t.parts) == 3) == overlap
        _, first = t.time(steps=1, warmup=0)
        _, last = t.time(steps=10, warmup=0)
        t.close()
        assert np.isfinite(last) and last < first
        losses[overlap] = last
    assert abs(losses[True] - losses[False]) <= 0.05 * abs(losses[False])


@pytest.mark.parametrize("mode", ["ste", "mxfp4"])
def test_fused_mlp_matches_the_unfused_composition(mode):
    # out(gelu(fc(x))) with the activation quantized in the first GEMM's epilogue against two
    # MXFP4Linear modules around F.gelu: outputs and all three gradients within the GEMM tolerance
    from lockstep_b200 import fp4_linear
    T, D = 512, 256
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    gy = torch.randn(T, D, device="cuda", generator=g).bfloat16()
    fused = fp4_linear.MXFP4MLP(D, 4 * D, backward=mode).cuda()
    fc = fp4_linear.MXFP4Linear(D, 4 * D, backward=mode).cuda()
    out = fp4_linear.MXFP4Linear(4 * D, D, backward=mode).cuda()
    with torch.no_grad():
        fc.weight.copy_(fused.fc.weight)
        out.weight.copy_(fused.out.weight)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya = fused(xa)
    ya.backward(gy)
    yb = out(torch.nn.functional.gelu(fc(xb)))
    yb.backward(gy)
    tol = 2e-2 if mode == "mxfp4" else 5e-3        # an MXFP4 backward re-quantizes slightly different values
    _close(ya, yb, "fused mlp forward", 2e-3)
    _close(xa.grad, xb.grad, "fused mlp dX", tol)
    _close(fused.fc.weight.grad, fc.weight.grad, "fused mlp dW fc", tol)
    _close(fused.out.weight.grad, out.weight.grad, "fused mlp dW out", tol)


def test_transposed_quantizer_with_gelu_equals_two_passes():
    from lockstep_b200 import fp4
    g = torch.Generator(device="cuda").manual_seed(8)
    c = (torch.randn(256, 384, device="cuda", generator=g) * 2).bfloat16()
    want_p, want_sf = fp4.quantize_mxfp4_packed_t(torch.nn.functional.gelu(c))
    got_p, got_sf = fp4.quantize_mxfp4_packed_t_gelu(c)
    differ = (got_p != want_p).float().mean().item()          # erf of this library against torch's kernel
    assert differ <= 1e-3, differ


def test_layernorm_quantize_kernel_against_two_passes():
    from lockstep_b200 import fp4
    g = torch.Generator(device="cuda").manual_seed(12)
    for dt, rows, D in ((torch.float32, 300, 1024), (torch.bfloat16, 129, 256), (torch.float32, 64, 4096), (torch.bfloat16, 77, 512),
                        (torch.float32, 1000, 768), (torch.bfloat16, 200, 1536), (torch.float32, 33, 2048), (torch.float32, 50, 1280),
                        (torch.bfloat16, 5000, 1024)):
        x = (torch.randn(rows, D, device="cuda", generator=g) * 3 + 0.5).to(dt)
        gamma = torch.randn(D, device="cuda", generator=g) * 0.2 + 1
        beta = torch.randn(D, device="cuda", generator=g) * 0.1
        y, p, sf, mean, rstd = fp4.layernorm_quantize(x, gamma, beta, 1e-5)
        ref = torch.nn.functional.layer_norm(x.float(), (D,), gamma, beta, 1e-5)
        assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()      # bf16 rounding of the output
        assert torch.allclose(mean, x.float().mean(1), atol=1e-5, rtol=1e-5)
        assert torch.allclose(rstd, (x.float().var(1, unbiased=False) + 1e-5).rsqrt(), rtol=1e-4)
        want_p, want_sf = fp4.quantize_mxfp4_packed(y)            # MXFP4 of exactly the bf16 rows it wrote
        assert torch.equal(p, want_p)
        valid = np.arange(rows)
        pick = lambda t: t.cpu().numpy().reshape(-1, D // 128, 32, 4, 4)[valid // 128, :, valid % 32, (valid % 128) // 32]
        assert np.array_equal(pick(sf), pick(want_sf))


@pytest.mark.parametrize("mode", ["ste", "mxfp4"])
def test_norm_fused_modules_match_the_unfused_composition(mode):
    # linear(layer_norm(x)) and out(gelu(fc(layer_norm(x)))) with the norm fused into the quantizer,
    # against nn.LayerNorm followed by the unfused modules, under bf16 autocast: outputs and gradients
    from lockstep_b200 import fp4_linear
    B, S, D = 4, 128, 256
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn(B, S, D, device="cuda", generator=g)
    gy = torch.randn(B, S, D, device="cuda", generator=g)
    fused_l = fp4_linear.MXFP4NormLinear(D, 3 * D, backward=mode).cuda()
    fused_m = fp4_linear.MXFP4MLP(D, 4 * D, backward=mode, norm=True).cuda()
    norm_l, lin = torch.nn.LayerNorm(D).cuda(), fp4_linear.MXFP4Linear(D, 3 * D, backward=mode).cuda()
    norm_m = torch.nn.LayerNorm(D).cuda()
    fc, out = fp4_linear.MXFP4Linear(D, 4 * D, backward=mode).cuda(), fp4_linear.MXFP4Linear(4 * D, D, backward=mode).cuda()
    with torch.no_grad():
        for n in (fused_l.norm, fused_m.norm, norm_l, norm_m):
            n.weight.copy_(torch.linspace(0.5, 1.5, D)), n.bias.copy_(torch.linspace(-0.1, 0.1, D))
        lin.weight.copy_(fused_l.linear.weight), fc.weight.copy_(fused_m.fc.weight), out.weight.copy_(fused_m.out.weight)
    tol = 2e-2 if mode == "mxfp4" else 5e-3
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", torch.bfloat16):
        ya = fused_l(xa)
        yb = lin(norm_l(xb))
    assert ya.dtype == torch.bfloat16 and ya.shape == (B, S, 3 * D)
    ya.float().backward(torch.cat([gy] * 3, -1))
    yb.float().backward(torch.cat([gy] * 3, -1))
    _close(ya, yb, "norm + linear forward", 2e-3)
    _close(xa.grad, xb.grad, "norm + linear dX", tol)
    _close(fused_l.linear.weight.grad, lin.weight.grad, "norm + linear dW", tol)
    _close(fused_l.norm.weight.grad, norm_l.weight.grad, "norm + linear dgamma", tol)
    _close(fused_l.norm.bias.grad, norm_l.bias.grad, "norm + linear dbeta", tol)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", torch.bfloat16):
        ya = fused_m(xa)
        yb = out(torch.nn.functional.gelu(fc(norm_m(xb))))
    ya.float().backward(gy)
    yb.float().backward(gy)
    _close(ya, yb, "norm + mlp forward", 3e-3)
    _close(xa.grad, xb.grad, "norm + mlp dX", tol)
    _close(fused_m.fc.weight.grad, fc.weight.grad, "norm + mlp dW fc", tol)
    _close(fused_m.out.weight.grad, out.weight.grad, "norm + mlp dW out", tol)
    _close(fused_m.norm.weight.grad, norm_m.weight.grad, "norm + mlp dgamma", tol)


def test_nvfp4_linear_forward_and_straight_through_backward():
    # forward: the oracle's NVFP4 quantization of x and w (lockstep's format rules), dequantized, fp32 matmul,
    # cast; backward: the straight-through matmuls of fp4_linear.py:42-45 on the unquantized tensors
    from lockstep_b200 import fp4_linear
    from oracle import nvfp4_ref
    g = torch.Generator().manual_seed(21)
    lin = fp4_linear.NVFP4Linear(256, 160).cuda()
    w = torch.randn(160, 256, generator=g) * 0.05
    with torch.no_grad():
        lin.weight.copy_(w)
    x = (torch.randn(4, 24, 256, generator=g) * torch.exp2(torch.randint(-3, 4, (4, 24, 1), generator=g).float())).bfloat16()
    xg = x.cuda().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = lin(xg)
    assert y.shape == (4, 24, 160) and y.dtype == torch.bfloat16
    xc, xs = nvfp4_ref.quantize(x.float().reshape(-1, 256).numpy())
    wc, ws = nvfp4_ref.quantize(w.numpy())                              # the layer quantizes its fp32 weight
    ref = torch.nn.functional.linear(torch.from_numpy(nvfp4_ref.dequantize(xc, xs)),
                                     torch.from_numpy(nvfp4_ref.dequantize(wc, ws))).bfloat16()
    _close(y.reshape(-1, 160), ref, "NVFP4 forward")
    gy = torch.randn(4, 24, 160, generator=g).bfloat16()
    y.backward(gy.cuda())
    gx_ref, gw_ref = ref_port.linear_backward_ste(gy.reshape(-1, 160), x.reshape(-1, 256), w)
    _close(xg.grad.reshape(-1, 256), gx_ref, "NVFP4 dX", 1e-2)      # bf16 matmuls, different GEMM library
    _close(lin.weight.grad, gw_ref, "NVFP4 dW", 1e-2)


@pytest.mark.parametrize("rows,D,xdt,gdt", [(1000, 1024, torch.float32, torch.bfloat16), (16384, 1024, torch.float32, torch.bfloat16),
                                            (300, 256, torch.bfloat16, torch.bfloat16), (37, 4096, torch.float32, torch.float32),
                                            (5000, 2048, torch.bfloat16, torch.float32)])
def test_layernorm_backward_kernel_against_torch(rows, D, xdt, gdt):
    # the statistics come from the fused forward kernel; the expected values from torch's own backward in fp64
    from lockstep_b200 import fp4
    g = torch.Generator(device="cuda").manual_seed(rows + D)
    x = (torch.randn(rows, D, device="cuda", generator=g) * 2 + 0.5).to(xdt)
    gy = torch.randn(rows, D, device="cuda", generator=g).to(gdt)
    gamma = torch.randn(D, device="cuda", generator=g)
    beta = torch.randn(D, device="cuda", generator=g)
    _, _, _, mean, rstd = fp4.layernorm_quantize(x, gamma, beta, 1e-5)
    gx, gw, gb = fp4.layernorm_backward(gy, x, mean, rstd, gamma)
    xd = x.double().requires_grad_(True)
    gd, bd = gamma.double().requires_grad_(True), beta.double().requires_grad_(True)
    torch.nn.functional.layer_norm(xd, (D,), gd, bd, 1e-5).backward(gy.double())
    assert gx.dtype == xdt and gw.dtype == torch.float32
    tol = 2e-6 if xdt == torch.float32 else 4e-3                # bf16 gx: one rounding of the result
    _close(gx, xd.grad, "gx", tol)
    _close(gw, gd.grad, "ggamma", 2e-6)
    _close(gb, bd.grad, "gbeta", 2e-6)
    again = fp4.layernorm_backward(gy, x, mean, rstd, gamma)
    assert all(torch.equal(a, b) for a, b in zip(again, (gx, gw, gb)))         # fixed summation order
    gx2, gw2, gb2 = fp4.layernorm_backward(gy, x, mean, rstd, None, want_bias=False)
    assert gw2 is None and gb2 is None
    xd2 = x.double().requires_grad_(True)
    torch.nn.functional.layer_norm(xd2, (D,), None, None, 1e-5).backward(gy.double())
    _close(gx2, xd2.grad, "gx without gamma", tol)
