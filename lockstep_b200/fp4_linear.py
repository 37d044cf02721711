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
    def forward(ctx, x, w1, w2):
        k = _need_kernel()
        (px, sx), (pxt, sxt) = _quant_both(x)
        (pw1, sw1), (pw1t, sw1t) = _quant_both(w1)
        (pw2, sw2), (pw2t, sw2t) = _quant_both(w2)
        c = k(px, pw1, sx, sw1, out_dtype=x.dtype)                # pre-activation [T, H]
        if c.dtype == torch.bfloat16 and c.shape[0] % 128 == 0 and c.shape[1] % 128 == 0:
            ph, sh, pht, sht = fp4.quantize_mxfp4_both(c, act="gelu")
        else:
            (ph, sh), (pht, sht) = _quant_both(torch.nn.functional.gelu(c))
        y = k(ph, pw2, sh, sw2, out_dtype=x.dtype)
        ctx.save_for_backward(pxt, sxt, pw1t, sw1t, pw2t, sw2t, pht, sht, c)
        ctx.dtypes = (x.dtype, w1.dtype, w2.dtype)
        return y

    @staticmethod
    def backward(ctx, gy):
        k = _need_kernel()
        pxt, sxt, pw1t, sw1t, pw2t, sw2t, pht, sht, c = ctx.saved_tensors
        x_dtype, w1_dtype, w2_dtype = ctx.dtypes
        (pg, sg), (pgt, sgt) = _quant_both(gy.contiguous())
        gh = k(pg, pw2t, sg, sw2t, out_dtype=x_dtype)             # [T, H], contract over the output width
        gw2 = k(pgt, pht, sgt, sht, out_dtype=torch.float32)      # [D, H], contract over tokens
        gc = torch.ops.aten.gelu_backward(gh, c)
        (pgc, sgc), (pgct, sgct) = _quant_both(gc)
        gx = k(pgc, pw1t, sgc, sw1t, out_dtype=x_dtype)           # [T, D], contract over H
        gw1 = k(pgct, pxt, sgct, sxt, out_dtype=torch.float32)    # [H, D], contract over tokens
        return gx, gw1.to(w1_dtype), gw2.to(w2_dtype)


class MXFP4MLP(nn.Module):
    """(extension) The feed-forward half of a block, out(gelu(fc(x))).  With backward="mxfp4"
    the activation stays in MXFP4 between the two GEMMs and is never written to HBM (see
    _MXFP4MLP); with backward="ste" the reference's straight-through backward needs the
    activation in bf16 anyway, so the module is the plain composition.  `fc` and `out` are
    ordinary MXFP4Linear modules (same parameters either way)."""

    def __init__(self, width, hidden, backward="ste"):
        super().__init__()
        self.fc = MXFP4Linear(width, hidden, backward=backward)
        self.out = MXFP4Linear(hidden, width, backward=backward)
        self.backward_mode = backward

    def forward(self, x):
        if self.backward_mode != "mxfp4" or not torch.is_grad_enabled():
            return self.out(torch.nn.functional.gelu(self.fc(x)))
        dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
        with torch.autocast("cuda", enabled=False):
            y = _MXFP4MLP.apply(x.reshape(-1, x.shape[-1]).to(dt), self.fc.weight, self.out.weight)
        return y.view(*x.shape[:-1], -1)
