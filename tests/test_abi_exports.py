"""The C-ABI library loads without a GPU, exports every symbol include/xkb200.h declares,
and rejects bad arguments before touching CUDA (no compute call is made here)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from xkernels_b200 import _lib
    from xkernels_b200.build import build

    build()
    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "xkb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xkb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/xkb200.h but not exported"


def test_python_prototypes_cover_the_header():
    from xkernels_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_and_error_string(lib):
    assert b"sm_100a" in lib.xkb_version()
    assert isinstance(lib.xkb_last_error(), bytes)


def test_argument_errors_need_no_gpu(lib):
    # negative sizes, bad dtype codes and missing workspaces are refused with a message
    assert lib.xkb_moe_sum_reduce(None, 7, None, 0, None, 0, 4, 2, 8, ctypes.c_float(1.0), None) == -1
    assert b"dtype" in lib.xkb_last_error()
    assert lib.xkb_moe_align_block_size(None, 16, 4, 0, None, 0, None, None, None, None, None, 0, None) == -1
    assert b"block_size" in lib.xkb_last_error()
    rc = lib.xkb_fused_moe_int4_w4a16(1, 0, 1, 1, 1, 1, None, 0, 1, 4, 32, 60, 2, 2, 32, 1, 0, None, 0, None)
    assert rc == -1 and b"K" in lib.xkb_last_error()
    rc = lib.xkb_fused_moe_int4_w4a16(1, 0, 1, 1, 1, 1, None, 0, 1, 4, 32, 64, 2, 2, 32, 1, 0, None, 0, None)
    assert rc == -3 and b"workspace" in lib.xkb_last_error()
    rc = lib.xkb_fused_moe_mxfp4(1, 0, 1, 1, 1, 1, 1, 1, None, None, None, 0, 1, 4, 48, 32, 2, 2,
                                 ctypes.c_float(10.0), 1, 0, None, 0, None)
    assert rc == -1 and b"32" in lib.xkb_last_error()


def test_workspace_queries(lib):
    small = lib.xkb_fused_moe_int4_w4a16_workspace_bytes(64, 4096, 7168, 48, 8, 0)
    big = lib.xkb_fused_moe_int4_w4a16_workspace_bytes(16384, 4096, 7168, 48, 8, 0)
    assert 64 * 8 * 4096 * 4 <= small < big
    assert lib.xkb_fused_moe_mxfp4_workspace_bytes(48, 4096, 512, 256, 6) >= 48 * 6 * 4096 * 4
    assert lib.xkb_moe_align_workspace_bytes(131072, 48) >= 128 * 49 * 4
