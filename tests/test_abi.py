"""The shared library loads without a GPU and exports every symbol that
include/lockstep_b200.h declares; compute entry points fail loudly on a box
with no sm_100 device instead of falling back to the CPU."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "lockstep_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ls_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def so():
    from lockstep_b200 import build
    return ctypes.CDLL(str(build.build()))


def test_header_symbols_exported(so):
    names = _declared()
    assert len(names) >= 8
    for n in names:
        assert hasattr(so, n), f"{n} declared in the header but not exported"


def test_ctypes_table_matches_header():
    from lockstep_b200 import _lib
    assert sorted(_lib.declared_symbols()) == _declared()


def test_version_and_sf_bytes(so):
    assert so.ls_version() >= 100
    so.ls_sf_bytes.restype = ctypes.c_int64
    so.ls_sf_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
    assert so.ls_sf_bytes(128, 128) == 512
    assert so.ls_sf_bytes(129, 256) == 2 * 2 * 512
    assert so.ls_sf_bytes(4096, 8192) == 4096 * 8192 // 32
    assert so.ls_sf_bytes(4, 100) == -1


def test_no_cpu_fallback():
    from lockstep_b200 import fp4
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        fp4.quantize_mxfp4(torch.zeros(2, 32))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        fp4.pack_fp4(torch.zeros(2, 32, dtype=torch.uint8))


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device error path")
def test_compute_entry_points_refuse_without_device(so):
    so.ls_last_error.restype = ctypes.c_char_p
    rc = so.ls_pack_fp4(None, None, ctypes.c_int64(32), None)
    assert rc in (-5, -3)
    assert so.ls_last_error()
