"""Argument checking at the C ABI on a GPU box: bad shapes, null and misaligned
pointers come back as error codes with a message; nothing is launched."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

EINVAL, EALIGN, ESTATE = -1, -2, -6


@pytest.fixture(scope="module")
def L():
    from lockstep_b200._lib import lib
    return lib()


def _p(t, off=0):
    return ctypes.c_void_p(t.data_ptr() + off)


def test_quantize_argument_errors(L):
    x = torch.zeros(4, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(4 * 64, device="cuda", dtype=torch.uint8)
    assert L.ls_quantize_mxfp4(_p(x), 1, 4, 64, 24, 0, _p(out), None, None, None, None, None) == EINVAL      # block
    assert L.ls_quantize_mxfp4(_p(x), 1, 4, 48, 32, 0, _p(out), None, None, None, None, None) == EINVAL      # K % block
    assert L.ls_quantize_mxfp4(_p(x), 7, 4, 64, 32, 0, _p(out), None, None, None, None, None) == EINVAL      # dtype
    assert L.ls_quantize_mxfp4(_p(x), 1, 4, 64, 32, 0, None, None, None, None, None, None) == EINVAL         # no output
    assert L.ls_quantize_mxfp4(_p(x), 1, 4, 64, 32, 0, None, None, None, None, _p(out), None) == EINVAL      # sf needs K % 128
    assert L.ls_quantize_mxfp4(_p(x, 2), 1, 2, 64, 32, 0, _p(out), None, None, None, None, None) == EALIGN
    assert b"aligned" in L.ls_last_error()
    assert L.ls_quantize_mxfp4(_p(x), 1, 0, 64, 32, 0, None, None, None, None, None, None) == 0              # empty: nothing to do
    y = torch.zeros(128, 128, device="cuda", dtype=torch.bfloat16)
    o = [torch.zeros(128 * 64, device="cuda", dtype=torch.uint8) for _ in range(4)]
    assert L.ls_quantize_mxfp4_both(_p(y), 1, 128, 96, 0, _p(o[0]), _p(o[1]), _p(o[2]), _p(o[3]), None) == EINVAL   # C % 128
    assert L.ls_quantize_mxfp4_both(_p(y), 1, 100, 128, 0, _p(o[0]), _p(o[1]), _p(o[2]), _p(o[3]), None) == EINVAL  # R % 128
    assert L.ls_quantize_mxfp4_both(_p(y), 1, 128, 128, 0, _p(o[0]), None, _p(o[2]), _p(o[3]), None) == EINVAL      # all four outputs
    assert L.ls_quantize_mxfp4_both(_p(y), 1, 128, 128, 0, _p(o[0], 8), _p(o[1]), _p(o[2]), _p(o[3]), None) == EALIGN
    assert L.ls_quantize_mxfp4_both(_p(y), 1, 128, 128, 0, _p(o[0]), _p(o[1]), _p(o[2]), _p(o[3]), None) == 0


def test_gemm_argument_errors(L):
    a = torch.zeros(128 * 64, device="cuda", dtype=torch.uint8)
    c = torch.zeros(128 * 128, device="cuda", dtype=torch.bfloat16)
    args = lambda K, pa=a, pc=c, dt=1: (_p(pa), _p(a), _p(a), _p(a), _p(pc), dt, 128, 128, K, None)
    assert L.ls_mxfp4_gemm(*args(96)) == EINVAL                                   # K % 128
    assert L.ls_mxfp4_gemm(*args(128, dt=5)) == EINVAL
    assert L.ls_mxfp4_gemm(None, _p(a), _p(a), _p(a), _p(c), 1, 128, 128, 128, None) == EINVAL
    assert L.ls_mxfp4_gemm(_p(a, 4), _p(a), _p(a), _p(a), _p(c), 1, 128, 128, 128, None) == EALIGN
    assert L.ls_mxfp4_gemm(*args(128)[:6], 0, 128, 128, None) == 0                # M = 0
    assert L.ls_mxfp4_gemm_quant(_p(a), _p(a), _p(a), _p(a), _p(c), 1, 0, _p(a), _p(a), 128, 100, 128, None) == EINVAL   # N % 128
    assert L.ls_gemm_set_variant(9) == EINVAL and L.ls_gemm_set_variant(4) == EINVAL and L.ls_gemm_set_variant(3) == 0 and L.ls_gemm_set_variant(0) == 0
    assert L.ls_gemm_set_splits(17) == EINVAL and L.ls_gemm_set_splits(0) == 0


def test_block16_and_nvfp4_argument_errors(L):
    a = torch.zeros(128 * 64, device="cuda", dtype=torch.uint8)
    c = torch.zeros(128 * 128, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(4, 128, device="cuda", dtype=torch.bfloat16)
    for fn in (L.ls_mxfp4_gemm_block16, L.ls_nvfp4_gemm):
        assert fn(_p(a), _p(a), _p(a), _p(a), _p(c), 1, 128, 128, 96, None) == EINVAL             # K % 128
        assert fn(_p(a), _p(a), _p(a), _p(a), _p(c), 5, 128, 128, 128, None) == EINVAL            # output type
        assert fn(_p(a), _p(a), None, _p(a), _p(c), 1, 128, 128, 128, None) == EINVAL             # null scales
        assert fn(_p(a), _p(a, 4), _p(a), _p(a), _p(c), 1, 128, 128, 128, None) == EALIGN
        assert fn(_p(a), _p(a), _p(a), _p(a), _p(c), 1, 128, 0, 128, None) == 0                   # N = 0
    for fn in (L.ls_mxfp4_gemm_dual_block16, L.ls_nvfp4_gemm_dual):
        assert fn(_p(a), None, _p(a), _p(a), _p(a), _p(a), _p(c), _p(c), 1, 128, 128, 128, None) == EINVAL
    assert L.ls_sf_bytes_block(130, 256, 16) == 2 * 4 * 512 and L.ls_sf_bytes_block(130, 256, 32) == L.ls_sf_bytes(130, 256)
    assert L.ls_sf_bytes_block(130, 256, 8) == -1 and L.ls_sf_bytes_block(130, 100, 16) == -1
    assert L.ls_scales_to_sf_block(_p(c), 4, 128, 8, _p(a), None, None) == EINVAL                 # block
    assert L.ls_quantize_nvfp4(_p(x), 1, 4, 64, _p(a), None, None, None, None) == EINVAL          # K % 128
    assert L.ls_quantize_nvfp4(_p(x), 9, 4, 128, _p(a), None, None, None, None) == EINVAL         # dtype
    assert L.ls_quantize_nvfp4(_p(x), 1, 4, 128, None, None, None, None, None) == EINVAL          # packed is required
    assert L.ls_quantize_nvfp4(_p(x, 16), 1, 2, 128, _p(a), None, None, None, None) == EALIGN     # 32-byte loads
    assert L.ls_quantize_nvfp4(_p(x), 1, 0, 128, None, None, None, None, None) == 0               # empty
    assert L.ls_dequantize_nvfp4(_p(a), _p(a), 4, 24, _p(c), 1, None) == EINVAL                   # K % 16
    assert L.ls_dequantize_nvfp4(_p(a), None, 4, 128, _p(c), 1, None) == EINVAL


def test_wire_argument_errors(L):
    h = ctypes.c_void_p()
    assert L.ls_wire_create(0, 9, 9 * 256, ctypes.byref(h)) == EINVAL             # at most 8 ranks
    assert L.ls_wire_create(0, 2, 300, ctypes.byref(h)) == EINVAL                 # padding
    assert L.ls_wire_create_int(0, 1, 256, 12, ctypes.byref(h)) == EINVAL         # bits
    assert L.ls_wire_create(0, 2, 512, ctypes.byref(h)) == 0
    g = torch.zeros(512, device="cuda")
    assert L.ls_wire_send(h, _p(g), 512, None, None) == ESTATE                    # peers not mapped yet
    assert L.ls_wire_int_phase(h, 0, _p(g), 512, None, None, None) == ESTATE      # not an integer wire
    assert L.ls_wire_destroy(h) == 0
    assert L.ls_wire_create(0, 1, 512, ctypes.byref(h)) == 0
    assert L.ls_wire_send(h, _p(g), 1024, None, None) == EINVAL                   # numel beyond the wire
    assert L.ls_wire_set_timeout_us(h, 0) == EINVAL and L.ls_wire_set_timeout_us(h, 10**6) == 0
    assert L.ls_wire_set_mode(h, 3, 0, 0) == EINVAL and L.ls_wire_set_mode(h, 0, 9, 0) == EINVAL and L.ls_wire_set_mode(h, 0, 0, 0) == 0
    assert L.ls_wire_destroy(h) == 0
