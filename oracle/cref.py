"""ctypes binding of the C oracle (mxfp4_ref.c).  Test infrastructure only.

numpy in, numpy out.  The shared object is built with `make -C oracle`
(build() in the repo's entry file does it); loading fails loudly if absent.
"""

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "libmxfp4_ref.so"
_lib = None


def build(force=False):
    if force or not _SO.exists() or _SO.stat().st_mtime < (_DIR / "mxfp4_ref.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR)] + (["-B"] if force else []), check=True,
                       capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_SO))
        _lib.ref_block_exponent.restype = ctypes.c_int
        _lib.ref_block_exponent.argtypes = [ctypes.c_float]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def quantize(x, block=32, rounding="ref", want=("codes", "packed", "scale", "e8m0")):
    """x: float32 array [..., K].  Returns dict of the requested outputs."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    K = x.shape[-1]
    assert K % block == 0
    nb = x.size // block
    out = {}
    if "codes" in want:
        out["codes"] = np.empty(x.shape, np.uint8)
    if "packed" in want:
        out["packed"] = np.empty(x.shape[:-1] + (K // 2,), np.uint8)
    if "scale" in want:
        out["scale"] = np.empty(x.shape[:-1] + (K // block,), np.float32)
    if "e8m0" in want:
        out["e8m0"] = np.empty(x.shape[:-1] + (K // block,), np.uint8)
    lib().ref_quantize_f32(_p(x), ctypes.c_int64(nb), ctypes.c_int(block),
                           ctypes.c_int(1 if rounding == "rne" else 0),
                           _p(out.get("codes")), _p(out.get("packed")),
                           _p(out.get("scale")), _p(out.get("e8m0")))
    return out


def pack(codes):
    codes = np.ascontiguousarray(codes, np.uint8)
    out = np.empty(codes.shape[:-1] + (codes.shape[-1] // 2,), np.uint8)
    lib().ref_pack(_p(codes), _p(out), ctypes.c_int64(out.size))
    return out


def unpack(packed):
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.uint8)
    lib().ref_unpack(_p(packed), _p(out), ctypes.c_int64(packed.size))
    return out


def dequantize(codes, scale, block=32):
    codes = np.ascontiguousarray(codes, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32)
    out = np.empty(codes.shape, np.float32)
    lib().ref_dequantize(_p(codes), _p(scale), ctypes.c_int64(codes.size // block),
                         ctypes.c_int(block), _p(out))
    return out


def block_exponent(amax):
    return lib().ref_block_exponent(ctypes.c_float(float(amax)))


def wire_encode(g, padded, res=None):
    """Sender half.  g float32 [n]; res float32 [padded] updated in place or None."""
    g = np.ascontiguousarray(g, np.float32)
    packed = np.empty(padded // 2, np.uint8)
    e8m0 = np.empty(padded // 32, np.uint8)
    lib().ref_wire_encode(_p(g), ctypes.c_int64(g.size), ctypes.c_int64(padded), _p(res),
                          _p(packed), _p(e8m0))
    return packed, e8m0


def wire_owner(slots, ores=None, reverse=False):
    """slots: list over senders of (packed u8 [shard/2], e8m0 u8 [shard/32])."""
    world = len(slots)
    ps = [np.ascontiguousarray(p) for p, _ in slots]
    es = [np.ascontiguousarray(e) for _, e in slots]
    shard = ps[0].size * 2
    arr_p = (ctypes.c_void_p * world)(*[p.ctypes.data for p in ps])
    arr_e = (ctypes.c_void_p * world)(*[e.ctypes.data for e in es])
    packed = np.empty(shard // 2, np.uint8)
    e8m0 = np.empty(shard // 32, np.uint8)
    lib().ref_wire_owner(arr_p, arr_e, ctypes.c_int(world), ctypes.c_int64(shard), _p(ores),
                         ctypes.c_int(int(reverse)), _p(packed), _p(e8m0))
    return packed, e8m0


def wire_decode(packed, e8m0, n, world):
    g = np.empty(n, np.float32)
    lib().ref_wire_decode(_p(np.ascontiguousarray(packed)), _p(np.ascontiguousarray(e8m0)),
                          ctypes.c_int64(n), ctypes.c_int(world), _p(g))
    return g


def wire_step(gs, res=None, ores=None, reverse=False, unit=64):
    """All ranks of one step in this process.  Returns (out, sent, owned).
    unit: padding granularity per rank (64 in wire.py:86-87; the CUDA kernels
    pad to 256, which moves shard boundaries but no block's arithmetic)."""
    world = len(gs)
    n = gs[0].size
    span = world * unit
    padded = -(-n // span) * span
    shard = padded // world
    sent = [wire_encode(gs[r], padded, None if res is None else res[r]) for r in range(world)]
    owned = []
    for o in range(world):
        slots = [(sent[r][0][o * shard // 2:(o + 1) * shard // 2],
                  sent[r][1][o * shard // 32:(o + 1) * shard // 32]) for r in range(world)]
        owned.append(wire_owner(slots, None if ores is None else ores[o], reverse))
    allp = np.concatenate([p for p, _ in owned])
    alle = np.concatenate([e for _, e in owned])
    return wire_decode(allp, alle, n, world), sent, owned
