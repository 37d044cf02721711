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
