"""ctypes binding of ``libxkb200.so`` — the only route from Python to the kernels.

The library is built in-tree by :mod:`xkernels_b200.build`.  There is no CPU or
eager fallback: if the shared object is missing or fails to load, importing any
op raises, and every op raises on non-CUDA tensors.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libxkb200.so"

XKB_BF16 = 0
XKB_F32 = 1
XKB_F16 = 2
PATH_AUTO, PATH_SIMT, PATH_TC = 0, 1, 2

# name -> (restype, argtypes); mirrors include/xkb200.h one to one.
SIGNATURES = {
    "xkb_version": (c_char_p, []),
    "xkb_last_error": (c_char_p, []),
    "xkb_launch_count": (c_int64, []),
    "xkb_moe_align_workspace_bytes": (c_int64, [c_int64, c_int]),
    "xkb_moe_align_block_size": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int64, c_void_p],
    ),
    "xkb_moe_align_block_size_static": (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "xkb_topk_softmax": (
        c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "xkb_moe_sum_reduce": (
        c_int,
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int64, c_float, c_void_p],
    ),
    "xkb_fused_moe_int4_w4a16_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int, c_int, c_int]),
    "xkb_fused_moe_int4_w4a16": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
         c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p],
    ),
    "xkb_fused_moe_int4_ffn_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int, c_int, c_int]),
    "xkb_fused_moe_int4_ffn": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
         c_int64, c_int64, c_int64, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int64, c_void_p],
    ),
    "xkb_moe_int4_w4a16_rows": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
         c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p],
    ),
    "xkb_moe_int4_w4a16_partial_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int, c_int, c_int]),
    "xkb_moe_int4_w4a16_partial": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int,
         c_int, c_void_p, c_int64, c_void_p],
    ),
    "xkb_set_sm_margin": (c_int, [c_int]),
    "xkb_ep_plan_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int]),
    "xkb_ep_plan": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p],
    ),
    "xkb_gather_rows": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "xkb_moe_gather_sum_reduce": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int64, c_void_p]),
    "xkb_fused_moe_mxfp4_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int, c_int]),
    "xkb_fused_moe_mxfp4": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_float,
         c_int, c_int, c_void_p, c_int64, c_void_p],
    ),
    "xkb_workspace_status": (c_int, [c_void_p, c_void_p]),
    "xkb_selftest_bounded_wait": (c_int, [c_void_p, c_int64, c_void_p]),
    "xkb_gemm_timer_enable": (c_int, [c_int]),
    "xkb_gemm_timer_read": (c_int, [c_void_p, c_int, c_void_p]),
}

_lib = None


class XkbError(RuntimeError):
    """A C-ABI call returned a negative status."""


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m xkernels_b200.build` "
            "(there is no fallback path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().xkb_last_error().decode("utf-8", "replace")
        raise XkbError(f"{what} failed with status {status}: {msg}")


def launch_count() -> int:
    return int(load().xkb_launch_count())


def set_sm_margin(sms: int) -> None:
    """Keep ``sms`` SMs free of the persistent grouped-GEMM kernels (for kernels on other streams)."""
    check(load().xkb_set_sm_margin(int(sms)), "xkb_set_sm_margin")


def gemm_timer_enable(max_calls: int) -> None:
    check(load().xkb_gemm_timer_enable(int(max_calls)), "xkb_gemm_timer_enable")


def gemm_timer_read(capacity: int = 1 << 16) -> list[float]:
    """Durations (ms) of the expert-GEMM launches of the fused calls made since arming."""
    buf = (ctypes.c_float * capacity)()
    n = ctypes.c_int(0)
    check(load().xkb_gemm_timer_read(buf, capacity, ctypes.byref(n)), "xkb_gemm_timer_read")
    return [float(buf[i]) for i in range(n.value)]
