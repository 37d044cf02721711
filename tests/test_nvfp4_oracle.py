"""The numpy restatement of lockstep's NVFP4 format rules against golden vectors
made by the reference's own header (tests/golden/make_golden_nvfp4.py): the
scalar functions on every E4M3 value, every rounding midpoint and its
neighbours; whole blocks of normal data with outliers; adversarial blocks
(quotients on E2M1 midpoints under scales with a mantissa, maxima on E4M3
midpoints, zero / tiny / huge / NaN / infinite blocks).  Bit for bit."""

from pathlib import Path

import numpy as np
import pytest

from oracle import nvfp4_ref as R

G = Path(__file__).resolve().parent / "golden"


def _f(a):
    return a.view(np.float32)


def test_scalar_functions_match_the_reference():
    z = np.load(G / "nvfp4_scalar.npz")
    got = R.quant_e4m3(_f(z["e4m3_in"]))
    assert np.array_equal(got.view(np.uint32), z["e4m3_out"])
    assert np.array_equal(R.nv_scale(_f(z["amax"])).view(np.uint32), z["scale"])
    assert np.array_equal(R.e2m1_code(_f(z["code_in"])), z["code_out"])
    s = _f(z["scale"])
    assert np.array_equal(R.quant_e4m3(s).view(np.uint32), z["scale"])           # every scale is an E4M3 value
    b = R.e4m3_byte(s)
    dec = np.where(b >> 3 == 0, (b & 7) * 2.0 ** -9, (8 + (b & 7)) * 2.0 ** ((b >> 3).astype(np.int32) - 10)).astype(np.float32)
    assert np.array_equal(dec, s)


@pytest.mark.parametrize("name", ["normal_f32", "normal_bf16", "adversarial"])
def test_blocks_match_the_reference(name):
    z = np.load(G / f"nvfp4_{name}.npz")
    x = _f(z["x"])
    codes, scale = R.quantize(x)
    assert np.array_equal(scale.view(np.uint32), z["scale"])
    assert np.array_equal(codes, z["codes"])
    deq = R.dequantize(codes, scale)
    want = _f(z["deq"])
    live = np.repeat(R.block_amax(x.reshape(*x.shape[:-1], -1, 16)) > 0, 16, axis=-1).reshape(x.shape)
    same = (deq.view(np.uint32) == want.view(np.uint32)) | (deq == want)          # -0.0 code 8 decodes to -0.0
    assert np.all(same | ~live)
    assert np.array_equal(R.pack(codes) & 0xF, codes[..., 0::2]) and np.array_equal(R.pack(codes) >> 4, codes[..., 1::2])


def _rne_e2m1(q):
    """Nearest E2M1 magnitude code with ties to the even code, saturating: what the hardware converter does."""
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    up_on_tie = np.array([0, 1, 0, 1, 0, 1, 0], bool)          # the even neighbour is the upper one at 0.75, 1.75, 3.5
    gt = q[..., None] > mids
    eq = q[..., None] == mids
    return (gt | (eq & up_on_tie)).sum(-1).astype(np.uint8)


def test_converter_shortcut_is_exact_for_every_bf16_value_and_scale():
    # The CUDA quantizer multiplies a bf16 input by (1 / s)(1 - 2^-12) and lets the hardware converter round
    # (nearest-even) instead of dividing and applying the rule's tie-to-smaller.  Every positive finite bf16
    # value against every E4M3 scale: the codes are the rule's.
    a = (np.arange(1, 0x7F80, dtype=np.uint32) << 16).view(np.float32)
    bytes_ = np.arange(1, 0x7F, dtype=np.uint8)
    s = np.where(bytes_ >> 3 == 0, (bytes_ & 7) * 2.0 ** -9, (8 + (bytes_ & 7)) * 2.0 ** ((bytes_ >> 3).astype(np.int32) - 10)).astype(np.float32)
    for sv in s:
        r = np.float32(1.0) / sv
        rc = np.float32(r * np.float32(1 - 2.0 ** -12))
        with np.errstate(over="ignore"):
            fast = _rne_e2m1((a * rc).astype(np.float32))
            want = R.e2m1_code((a / sv).astype(np.float32))
            keep = (a / sv) < 2.0 ** 23                         # beyond, the rule's fp32 distances collapse; the kernel divides there
        assert np.array_equal(fast[keep], want[keep]), float(sv)


def test_converter_bracket_is_exact_where_it_agrees_fp32():
    # fp32 input: two conversions with (1 / s)(1 -+ 2^-21); where they agree the code is the rule's.  Checked on
    # values packed around every midpoint x scale (where they may disagree) and on random values.
    rng = np.random.default_rng(3)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    bytes_ = np.arange(1, 0x7F, dtype=np.uint8)
    s = np.where(bytes_ >> 3 == 0, (bytes_ & 7) * 2.0 ** -9, (8 + (bytes_ & 7)) * 2.0 ** ((bytes_ >> 3).astype(np.int32) - 10)).astype(np.float32)
    agree = total = 0
    for sv in s:
        centre = (mids * sv).astype(np.float32)
        near = (centre[:, None].view(np.uint32).astype(np.int64) + np.arange(-40, 41)).astype(np.uint32).view(np.float32).reshape(-1)
        a = np.concatenate([near, (rng.uniform(0, 7, 2000) * sv).astype(np.float32)])
        r = np.float32(1.0) / sv
        lo = _rne_e2m1((a * np.float32(r * np.float32(1 - 2.0 ** -21))).astype(np.float32))
        hi = _rne_e2m1((a * np.float32(r * np.float32(1 + 2.0 ** -21))).astype(np.float32))
        want = R.e2m1_code((a / sv).astype(np.float32))
        same = lo == hi
        assert np.array_equal(lo[same], want[same]), float(sv)
        agree += int(same.sum())
        total += same.size
    assert agree > 0.5 * total                                  # the shortcut decides most values even in this packed set
