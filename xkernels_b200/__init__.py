"""B200-native (sm_100a) fused-MoE hot path behind the xkernels operator API.

Public callables (same argument names and meaning as the reference backends):

* :func:`moe_align_block_size`
* :func:`fused_moe_int4_w4a16`
* :func:`fused_moe_mxfp4`
* :func:`moe_sum_reduce`
* :func:`topk_softmax` (the router in front of the path)
* :func:`fused_moe_int4_ffn` (two INT4 GEMMs with SwiGLU between them, one call)

``plugin.install()`` registers them as the ``backend="cuda"`` cards of an
installed ``xkernels`` package.
"""

from .ops import (  # noqa: F401
    fused_moe_int4_ffn,
    fused_moe_int4_w4a16,
    fused_moe_mxfp4,
    moe_align_block_size,
    moe_sum_reduce,
    topk_softmax,
)

__all__ = [
    "fused_moe_int4_ffn",
    "fused_moe_int4_w4a16",
    "fused_moe_mxfp4",
    "moe_align_block_size",
    "moe_sum_reduce",
    "topk_softmax",
]
__version__ = "0.1.0"
