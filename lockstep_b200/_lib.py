"""ctypes loader of liblockstep_b200.so and small helpers for the host modules.

There is no CPU path: if the shared object is missing, or a tensor is not on a
CUDA device, the call raises.
"""

import ctypes
from pathlib import Path

import torch

PKG = Path(__file__).resolve().parent
SO = PKG / "liblockstep_b200.so"
_lib = None

c_i64, c_int, c_vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

_SIGS = {
    "ls_version": (c_int, []),
    "ls_last_error": (ctypes.c_char_p, []),
    "ls_sf_bytes": (c_i64, [c_i64, c_i64]),
    "ls_sf_bytes_block": (c_i64, [c_i64, c_i64, c_int]),
    "ls_quantize_mxfp4": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "ls_quantize_mxfp4_t": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_vp, c_vp, c_vp, c_vp]),
    "ls_quantize_mxfp4_t_act": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_vp]),
    "ls_quantize_mxfp4_both_act": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "ls_quantize_mxfp4_both": (c_int, [c_vp, c_int, c_i64, c_i64, c_int, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "ls_layernorm_quantize": (c_int, [c_vp, c_int, c_vp, c_vp, ctypes.c_float, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "ls_layernorm_backward_scratch": (c_i64, [c_i64, c_i64]),
    "ls_layernorm_backward": (c_int, [c_vp, c_int, c_vp, c_int, c_vp, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "ls_round_e2m1": (c_int, [c_vp, c_i64, c_int, c_vp, c_vp]),
    "ls_pack_fp4": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "ls_unpack_fp4": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "ls_dequantize_mxfp4": (c_int, [c_vp, c_int, c_vp, c_vp, c_i64, c_i64, c_int, c_vp, c_int, c_vp]),
    "ls_mxfp4_gemm": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "ls_mxfp4_gemm_dual": (c_int, [c_vp] * 8 + [c_int, c_i64, c_i64, c_i64, c_vp]),
    "ls_mxfp4_gemm_block16": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "ls_mxfp4_gemm_dual_block16": (c_int, [c_vp] * 8 + [c_int, c_i64, c_i64, c_i64, c_vp]),
    "ls_quantize_nvfp4": (c_int, [c_vp, c_int, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp]),
    "ls_dequantize_nvfp4": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_int, c_vp]),
    "ls_nvfp4_gemm": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "ls_nvfp4_gemm_dual": (c_int, [c_vp] * 8 + [c_int, c_i64, c_i64, c_i64, c_vp]),
    "ls_mxfp4_gemm_quant": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_int, c_vp, c_vp, c_i64, c_i64, c_i64, c_vp]),
    "ls_gemm_status": (c_int, [c_vp]),
    "ls_gemm_set_variant": (c_int, [c_int]),
    "ls_gemm_set_splits": (c_int, [c_int]),
    "ls_gemm_set_pdl": (c_int, [c_int]),
    "ls_fp4_mma_peak": (c_int, [c_int, ctypes.POINTER(ctypes.c_double), c_vp]),
    "ls_mxfp4_linear_noalloc": (c_int, [c_vp, c_int, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "ls_wire_handle_bytes": (c_i64, []),
    "ls_wire_create": (c_int, [c_int, c_int, c_i64, ctypes.POINTER(c_vp)]),
    "ls_wire_destroy": (c_int, [c_vp]),
    "ls_wire_local_handle": (c_int, [c_vp, c_vp]),
    "ls_wire_map_peers": (c_int, [c_vp, c_vp]),
    "ls_wire_map_local": (c_int, [c_vp, ctypes.POINTER(c_vp)]),
    "ls_wire_send": (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp]),
    "ls_wire_reduce": (c_int, [c_vp, c_vp, c_int, c_vp]),
    "ls_wire_finish": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "ls_wire_allreduce": (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_int, c_vp]),
    "ls_wire_create_int": (c_int, [c_int, c_int, c_i64, c_int, ctypes.POINTER(c_vp)]),
    "ls_wire_int_phase": (c_int, [c_vp, c_int, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "ls_wire_int_allreduce": (c_int, [c_vp, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "ls_wire_status": (c_int, [c_vp, c_vp]),
    "ls_wire_allreduce_group": (c_int, [ctypes.POINTER(c_vp), ctypes.POINTER(c_vp), c_i64, ctypes.POINTER(c_vp),
                                        ctypes.POINTER(c_vp), c_int, c_vp]),
    "ls_wire_set_mode": (c_int, [c_vp, c_int, c_int, c_int]),
    "ls_wire_mode": (c_int, [c_vp]),
    "ls_wire_set_dynamic": (c_int, [c_vp, c_int]),
    "ls_wire_set_timeout_us": (c_int, [c_vp, c_i64]),
    "ls_wire_poll_status": (c_int, [c_vp, c_vp]),
    "ls_wire_reset": (c_int, [c_vp]),
    "ls_wire_debug_slots": (c_int, [c_vp, c_int, c_vp, ctypes.POINTER(c_i64), c_vp]),
    "ls_scales_to_sf": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "ls_scales_to_sf_block": (c_int, [c_vp, c_i64, c_i64, c_int, c_vp, c_vp, c_vp]),
    "ls_scales_to_sf_t": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "ls_e4m3_to_packed": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp]),
    "ls_e4m3_to_packed_t": (c_int, [c_vp, c_i64, c_i64, c_vp, c_vp]),
}

LS_F32, LS_BF16 = 0, 1
_ERR = {-1: "LS_EINVAL", -2: "LS_EALIGN", -3: "LS_ECUDA", -4: "LS_ETIMEOUT", -5: "LS_EARCH", -6: "LS_ESTATE"}


def declared_symbols():
    return list(_SIGS)


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not SO.exists():
            raise RuntimeError(f"{SO} is missing: run `python -m lockstep_b200.build` "
                               "(there is no CPU fallback)")
        L = ctypes.CDLL(str(SO))
        for name, (res, args) in _SIGS.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        msg = lib().ls_last_error().decode(errors="replace")
        raise RuntimeError(f"lockstep_b200: {_ERR.get(rc, rc)}: {msg}")


def need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lockstep_b200 computes on CUDA tensors only; got a "
                               f"{t.device.type} tensor (there is no CPU fallback)")


def aligned(t, n=16):
    """t as a contiguous tensor whose storage pointer is a multiple of n bytes
    (a contiguous slice of a larger tensor may start anywhere; the kernels read
    and write vector words)."""
    if t is None:
        return None
    t = t.contiguous()
    return t.clone() if t.data_ptr() % n else t


def ptr(t):
    return None if t is None else c_vp(t.data_ptr())


def stream():
    return c_vp(torch.cuda.current_stream().cuda_stream)


def dtype_code(dt):
    if dt == torch.float32:
        return LS_F32
    if dt == torch.bfloat16:
        return LS_BF16
    raise TypeError(f"unsupported dtype {dt}")
