"""MXFP4 linear layer with the API of lockstep's fp4_linear.py.

Forward: quantize activations and weights along K to MXFP4 and multiply on the
block-scaled tensor cores (the reference does the same through Triton on an
H100 and through dequantize + F.linear elsewhere, fp4_linear.py:33-40; the
results agree with that second path within the GEMM tolerance).

Backward, two modes:
  "ste"    the reference's: straight-through matmuls in the incoming grad's
           dtype, dX = gy @ w, dW = gy.T @ x (fp4_linear.py:42-45)
  "mxfp4"  (extension) both backward GEMMs in MXFP4 too: dX contracts over the
           output features, so gy and w.T are quantized along that axis; dW
           contracts over tokens, so gy.T and x.T are quantized along tokens.
           Each tensor is read once: one kernel emits both orientations, and
           the forward keeps packed x.T and w.T for the backward instead of x.

There is no CPU path: on a device without block-scaled tensor cores the
forward raises.
"""

import functools

import torch
import torch.nn as nn

from . import fp4, mxfp4_gemm


@functools.cache
def kernel():
    """The tcgen05 MXFP4 GEMM on an sm_100 device, else None (fp4_linear.py:16-25)."""
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
        return None
    return mxfp4_gemm.mxfp4_gemm_packed


def path():
    return "tcgen05-mxfp4" if kernel() else "unavailable"


def _need_kernel():
    k = kernel()
    if k is None:
        raise RuntimeError("MXFP4Linear needs an sm_100 GPU (there is no CPU or fake-quant fallback)")
    return k


def _gemm(a, b_t, out_dtype):
    """a [M, K] @ b_t [N, K].T with both operands quantized along K."""
    k = _need_kernel()
    pa, sa = fp4.quantize_mxfp4_packed(a)
    pb, sb = fp4.quantize_mxfp4_packed(b_t)
    return k(pa, pb, sa, sb, out_dtype=out_dtype)


def _quant_t(x):
    """MXFP4 of x.T (blocks run down the columns of x), without a transposed copy
    when the row count allows the fused kernel."""
    if x.shape[0] % 128 == 0:
        return fp4.quantize_mxfp4_packed_t(x)
    return fp4.quantize_mxfp4_packed(x.t().contiguous())


def _quant_both(x):
    """(packed, sf) of x and of x.T; one read of x when both dimensions allow it."""
    if x.shape[0] % 128 == 0 and x.shape[1] % 128 == 0:
        p, s, pt, st = fp4.quantize_mxfp4_both(x)
        return (p, s), (pt, st)
    return fp4.quantize_mxfp4_packed(x), _quant_t(x)


class _MXFP4Matmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, backward_mode="ste"):
        ctx.backward_mode = backward_mode
        if backward_mode == "ste" or not any(ctx.needs_input_grad[:2]):
            ctx.save_for_backward(x, w)
            ctx.backward_mode = "ste"
            return _gemm(x, w, x.dtype)
        # MXFP4 backward: both orientations of x and w come out of the forward's own read
        # of them; what is kept for the backward pass is packed MXFP4, not x itself
        k = _need_kernel()
        (px, sx), (pxt, sxt) = _quant_both(x)                     # x along K; x.T along tokens (for dW)
        (pw, sw), (pwt, swt) = _quant_both(w)                     # w along K; w.T along N (for dX)
        ctx.save_for_backward(pxt, sxt, pwt, swt)
        ctx.dtypes = (x.dtype, w.dtype)
        return k(px, pw, sx, sw, out_dtype=x.dtype)

    @staticmethod
    def backward(ctx, gy):
        if ctx.backward_mode == "ste":
            x, w = ctx.saved_tensors
            return (gy @ w.to(gy.dtype)).to(x.dtype), (gy.t() @ x.to(gy.dtype)).to(w.dtype), None
        k = _need_kernel()
        pxt, sxt, pwt, swt = ctx.saved_tensors
        x_dtype, w_dtype = ctx.dtypes
        (pg, sg), (pgt, sgt) = _quant_both(gy.contiguous())       # gy along N (for dX); gy.T along tokens (for dW)
        gx = k(pg, pwt, sg, swt, out_dtype=x_dtype)               # [T, K], contract over N
        gw = k(pgt, pxt, sgt, sxt, out_dtype=torch.float32)       # [N, K], contract over tokens
        return gx, gw.to(w_dtype), None


class MXFP4Linear(nn.Linear):
    """nn.Linear whose forward GEMM runs in MXFP4 (bias unsupported)."""

    def __init__(self, fan_in, fan_out, bias=False, backward="ste"):
        assert not bias, "MXFP4Linear has no bias"
        assert backward in ("ste", "mxfp4")
        super().__init__(fan_in, fan_out, bias=False)
        self.backward_mode = backward

    def forward(self, x):
        dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        with torch.autocast("cuda", enabled=False):
            y = _MXFP4Matmul.apply(x.reshape(-1, x.shape[-1]).to(dt), self.weight, self.backward_mode)
        return y.view(*x.shape[:-1], -1)


FP4Linear = MXFP4Linear


class _NVFP4Matmul(torch.autograd.Function):
    """x @ w.T with both operands in NVFP4 (blocks of 16 along K under E4M3 scales); straight-through backward as
    fp4_linear.py:42-45."""

    @staticmethod
    def forward(ctx, x, w):
        from . import nvfp4
        _need_kernel()
        ctx.save_for_backward(x, w)
        px, _, sx = nvfp4.quantize_nvfp4(x)
        pw, _, sw = nvfp4.quantize_nvfp4(w)
        return nvfp4.nvfp4_gemm_packed(px, pw, sx, sw, out_dtype=x.dtype)

    @staticmethod
    def backward(ctx, gy):
        x, w = ctx.saved_tensors
        return (gy @ w.to(gy.dtype)).to(x.dtype), (gy.t() @ x.to(gy.dtype)).to(w.dtype)


class NVFP4Linear(nn.Linear):
    """(extension) MXFP4Linear's counterpart in the NVFP4 format that lockstep's format study defines
    (rig_sm75/quant_sim.cuh:90-97) but has no layer for.  fan_in % 128 == 0; no bias."""

    def __init__(self, fan_in, fan_out, bias=False):
        assert not bias, "NVFP4Linear has no bias"
        super().__init__(fan_in, fan_out, bias=False)

    def forward(self, x):
        dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        with torch.autocast("cuda", enabled=False):
            y = _NVFP4Matmul.apply(x.reshape(-1, x.shape[-1]).to(dt), self.weight)
        return y.view(*x.shape[:-1], -1)


def _ln_backward(g_y, x, mean, rstd, gamma, beta):
    """LayerNorm's backward from the statistics the fused forward kept: this library's kernel (it
    reads the incoming gradient in the type the GEMM left it in), torch's for other shapes."""
    rows, D = x.shape
    if D % 256 == 0 and D <= 8192 and x.dtype in (torch.float32, torch.bfloat16):
        gx, gw, gb = fp4.layernorm_backward(g_y, x, mean, rstd, gamma, want_bias=beta is not None)
        return gx, (None if gw is None else gw.to(gamma.dtype)), (None if gb is None else gb.to(beta.dtype))
    return torch.ops.aten.native_layer_norm_backward(g_y.to(x.dtype), x, [D], mean.view(rows, 1), rstd.view(rows, 1),
                                                     gamma, beta, [True, gamma is not None, beta is not None])


class _NormMatmul(torch.autograd.Function):
    """linear(layer_norm(x)) (train.py:50: qkv(ln1(x))) with the normalization and the
    quantization of its output in one kernel: the fp32 normalized tensor, its cast to bf16 and
    the quantizer's read of it disappear; what remains of layer_norm(x) in HBM is the bf16
    copy the backward pass needs."""

    @staticmethod
    def forward(ctx, x, gamma, beta, w, eps, backward_mode):
        k = _need_kernel()
        y, py, sy, mean, rstd = fp4.layernorm_quantize(x, gamma, beta, eps)
        mx = backward_mode == "mxfp4" and any(ctx.needs_input_grad[:4])
        ctx.mx = mx
        if mx:
            pyt, syt = _quant_t(y)
            (pw, sw), (pwt, swt) = _quant_both(w)
            ctx.save_for_backward(x, gamma, beta, mean, rstd, pyt, syt, pwt, swt)
            ctx.w_dtype = w.dtype
        else:
            pw, sw = fp4.quantize_mxfp4_packed(w)
            ctx.save_for_backward(x, gamma, beta, mean, rstd, y, w)
        return k(py, pw, sy, sw, out_dtype=torch.bfloat16)

    @staticmethod
    def backward(ctx, gy):
        if not ctx.mx:
            x, gamma, beta, mean, rstd, y, w = ctx.saved_tensors
            g_y = gy @ w.to(gy.dtype)
            gw = (gy.t() @ y.to(gy.dtype)).to(w.dtype)
        else:
            k = _need_kernel()
            x, gamma, beta, mean, rstd, pyt, syt, pwt, swt = ctx.saved_tensors
            (pg, sg), (pgt, sgt) = _quant_both(gy.contiguous())
            g_y = k(pg, pwt, sg, swt, out_dtype=torch.bfloat16)
            gw = k(pgt, pyt, sgt, syt, out_dtype=torch.float32).to(ctx.w_dtype)
        gx, ggamma, gbeta = _ln_backward(g_y, x, mean, rstd, gamma, beta)
        return gx, ggamma, gbeta, gw, None, None


def _fusable_norm(x, width):
    """The fused LayerNorm + quantize kernel rounds the normalized rows to bf16: it stands in
    for layer_norm + cast exactly when the projection would run in bf16 (autocast)."""
    return (x.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
            and x.dtype in (torch.float32, torch.bfloat16) and width % 256 == 0 and width <= 8192)


class MXFP4NormLinear(nn.Module):
    """(extension) linear(layer_norm(x)) with both in this library: `norm` is an ordinary
    nn.LayerNorm, `linear` an ordinary MXFP4Linear (same parameters as the unfused pair)."""

    def __init__(self, width, out_features, backward="ste", eps=1e-5):
        super().__init__()
        self.norm = nn.LayerNorm(width, eps=eps)
        self.linear = MXFP4Linear(width, out_features, backward=backward)

    def forward(self, x):
        width = x.shape[-1]
        if not _fusable_norm(x, width):
            return self.linear(self.norm(x))
        with torch.autocast("cuda", enabled=False):
            y = _NormMatmul.apply(x.reshape(-1, width).contiguous(), self.norm.weight, self.norm.bias, self.linear.weight,
                                  self.norm.eps, self.linear.backward_mode)
        return y.view(*x.shape[:-1], -1)


class _MXFP4MLP(torch.autograd.Function):
    """out(gelu(fc(x))) of lockstep's block (train.py:53, two _MXFP4Matmul around F.gelu) with
    MXFP4 backward GEMMs and the activation never written to HBM: the quantizer of the second
    GEMM's input applies GELU to the first GEMM's output as it reads it and emits both
    orientations (rows for the forward product, columns for the weight gradient), so the
    elementwise GELU pass and the tensor it would produce disappear.  The backward pass takes
    GELU's derivative from the saved pre-activation.
    (Doing the GELU and the quantization in the first GEMM's epilogue instead --
    mxfp4_gemm_packed_quant -- was measured slower inside a training step: with K = 1024 that
    GEMM is bound by its epilogue already, and erf for 67 M outputs on eight epilogue warps
    per SM costs more than a bandwidth-bound pass with full occupancy.)"""

    @staticmethod
    def forward(ctx, x, w1, w2, gamma=None, beta=None, eps=None):
        k = _need_kernel()
        ctx.normed = eps is not None
        if ctx.normed:                                            # out(gelu(fc(layer_norm(x)))): see _NormMatmul
            xin = x
            x, px, sx, mean, rstd = fp4.layernorm_quantize(xin, gamma, beta, eps)
            pxt, sxt = _quant_t(x)
        else:
            (px, sx), (pxt, sxt) = _quant_both(x)
        (pw1, sw1), (pw1t, sw1t) = _quant_both(w1)
        (pw2, sw2), (pw2t, sw2t) = _quant_both(w2)
        c = k(px, pw1, sx, sw1, out_dtype=x.dtype)                # pre-activation [T, H]
        if c.dtype == torch.bfloat16 and c.shape[0] % 128 == 0 and c.shape[1] % 128 == 0:
            ph, sh, pht, sht = fp4.quantize_mxfp4_both(c, act="gelu")
        else:
            (ph, sh), (pht, sht) = _quant_both(torch.nn.functional.gelu(c))
        y = k(ph, pw2, sh, sw2, out_dtype=x.dtype)
        if ctx.normed:
            ctx.save_for_backward(pxt, sxt, pw1t, sw1t, pw2t, sw2t, pht, sht, c, xin, gamma, beta, mean, rstd)
        else:
            ctx.save_for_backward(pxt, sxt, pw1t, sw1t, pw2t, sw2t, pht, sht, c)
        ctx.dtypes = (x.dtype, w1.dtype, w2.dtype)
        return y

    @staticmethod
    def backward(ctx, gy):
        k = _need_kernel()
        pxt, sxt, pw1t, sw1t, pw2t, sw2t, pht, sht, c = ctx.saved_tensors[:9]
        x_dtype, w1_dtype, w2_dtype = ctx.dtypes
        (pg, sg), (pgt, sgt) = _quant_both(gy.contiguous())
        gh = k(pg, pw2t, sg, sw2t, out_dtype=x_dtype)             # [T, H], contract over the output width
        gw2 = k(pgt, pht, sgt, sht, out_dtype=torch.float32)      # [D, H], contract over tokens
        gc = torch.ops.aten.gelu_backward(gh, c)
        (pgc, sgc), (pgct, sgct) = _quant_both(gc)
        gx = k(pgc, pw1t, sgc, sw1t, out_dtype=x_dtype)           # [T, D], contract over H
        gw1 = k(pgct, pxt, sgct, sxt, out_dtype=torch.float32)    # [H, D], contract over tokens
        if not ctx.normed:
            return gx, gw1.to(w1_dtype), gw2.to(w2_dtype)
        xin, gamma, beta, mean, rstd = ctx.saved_tensors[9:]
        gxin, ggamma, gbeta = _ln_backward(gx, xin, mean, rstd, gamma, beta)
        return gxin, gw1.to(w1_dtype), gw2.to(w2_dtype), ggamma, gbeta, None


class MXFP4MLP(nn.Module):
    """(extension) The feed-forward half of a block, out(gelu(fc(x))).  With backward="mxfp4"
    the activation stays in MXFP4 between the two GEMMs and is never written to HBM (see
    _MXFP4MLP); with backward="ste" the reference's straight-through backward needs the
    activation in bf16 anyway, so the module is the plain composition.  `fc` and `out` are
    ordinary MXFP4Linear modules (same parameters either way)."""

    def __init__(self, width, hidden, backward="ste", norm=False, eps=1e-5):
        super().__init__()
        self.norm = nn.LayerNorm(width, eps=eps) if norm else None     # norm=True: out(gelu(fc(layer_norm(x))))
        self.fc = MXFP4Linear(width, hidden, backward=backward)
        self.out = MXFP4Linear(hidden, width, backward=backward)
        self.backward_mode = backward

    def forward(self, x):
        width = x.shape[-1]
        if self.backward_mode != "mxfp4" or not torch.is_grad_enabled():
            if self.norm is not None and _fusable_norm(x, width):     # only the norm + quantize fusion applies
                with torch.autocast("cuda", enabled=False):
                    h = _NormMatmul.apply(x.reshape(-1, width).contiguous(), self.norm.weight, self.norm.bias,
                                          self.fc.weight, self.norm.eps, self.backward_mode)
                return self.out(torch.nn.functional.gelu(h)).view(*x.shape[:-1], -1)
            h = x if self.norm is None else self.norm(x)
            return self.out(torch.nn.functional.gelu(self.fc(h)))
        if self.norm is not None and _fusable_norm(x, width):
            with torch.autocast("cuda", enabled=False):
                y = _MXFP4MLP.apply(x.reshape(-1, width).contiguous(), self.fc.weight, self.out.weight,
                                    self.norm.weight, self.norm.bias, self.norm.eps)
            return y.view(*x.shape[:-1], -1)
        h = x if self.norm is None else self.norm(x)
        dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else h.dtype
        with torch.autocast("cuda", enabled=False):
            y = _MXFP4MLP.apply(h.reshape(-1, width).to(dt), self.fc.weight, self.out.weight)
        return y.view(*x.shape[:-1], -1)
