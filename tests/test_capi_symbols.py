"""The C-ABI library builds for sm_100a without a GPU, loads, and exports every symbol the public
header declares (no compute calls here)."""
import ctypes
import re
import shutil
from pathlib import Path

import pytest

from gptoss_b200 import capi

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "gptoss_b200.h"


def _declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(gptoss_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib_path():
    if capi.needs_build():
        if shutil.which("nvcc") is None:
            pytest.skip("library not built and nvcc absent")
        capi.build()
    return capi.LIB_PATH


def test_header_and_binding_agree():
    assert _declared() == sorted(capi.EXPORTS)


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    for name in _declared():
        assert hasattr(lib, name), name


def test_binding_loads_and_reports_version(lib_path):
    lib = capi.load()
    assert lib.gptoss_version().decode().startswith("gptoss_b200")


def test_create_rejects_bad_arguments_without_a_gpu(lib_path):
    lib = capi.load()
    ctx = ctypes.c_void_p()
    dims = capi.MoEDims(30, 64, 32, 4, 1, 7.0)  # hidden not a multiple of 8
    assert lib.gptoss_ctx_create(ctypes.byref(dims), 0, 0, 1, 16, 0, ctypes.byref(ctx)) == capi.ERR_BAD_ARG
    dims = capi.MoEDims(32, 64, 32, 4, 1, 7.0)
    assert lib.gptoss_ctx_create(ctypes.byref(dims), 0, 0, 3, 16, 0, ctypes.byref(ctx)) == capi.ERR_BAD_ARG  # 32 % 3
    assert lib.gptoss_ctx_create(None, 0, 0, 1, 16, 0, ctypes.byref(ctx)) == capi.ERR_BAD_ARG
    assert not ctx.value
