"""Host side of the four ops: argument checks, output allocation, one C-ABI call.

The callables keep the parameter names of the reference backends because the
reference's ``verify`` harness calls a card as ``fn(**inputs)``
(src/xkernels/verify.py:213-222 with names from
src/xkernels/registry/input_gen.py:68-72,84-103,138-159).  PyTorch is used for
device memory and the current stream only; all arithmetic happens in
``libxkb200.so``.
"""

from __future__ import annotations

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.XKB_BF16, torch.float32: _lib.XKB_F32}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _require_cuda(name: str, *tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name}: expected torch.Tensor, got {type(t).__name__}")
        if not t.is_cuda:
            raise RuntimeError(
                f"{name}: the sm_100a backend needs CUDA tensors (got device {t.device}); "
                "there is no CPU path"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name}: tensors live on different devices ({dev} vs {t.device})")
    return dev


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


_retired: list[torch.Tensor] = []


def get_workspace(dev: torch.device, nbytes: int, tag: int = 0) -> torch.Tensor:
    """Grow-only per-device scratch buffer shared by calls on one stream.

    Calls that overlap on different streams of one device must pass distinct
    ``tag`` values (or serialise): the buffer holds the routing and the fp32
    partial rows of the call in flight.  When a larger call needs a new buffer the old one is kept
    alive (until :func:`release_workspaces`): a CUDA graph captured earlier, or work still queued
    on another stream, may hold its address.  A caller that wants to own the memory passes
    ``workspace=`` to the fused ops instead.
    """
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)
        size = max(int(nbytes), 1 << 20)
        if buf is not None:
            size = max(size, 2 * buf.numel())        # geometric growth bounds what the retired buffers hold
        buf = torch.empty(size, dtype=torch.uint8, device=dev)
        _workspaces[key] = buf
    return buf


def _caller_workspace(workspace, fits: bool, nbytes_at_capacity: int, dev: torch.device, nbytes: int) -> torch.Tensor:
    """The scratch memory of one fused call.

    ``workspace`` None: this package's per-device buffer.  A CUDA ``uint8`` tensor: used as it is
    (ValueError if it is too small or misaligned).  One of the reference's workspace objects
    (``MoeInt4Workspace`` / ``MoeMxfp4Workspace``, src/xkernels/ops/moe/workspace.py:159-289):
    when its ``matches()`` accepted the call (``fits``), the call's scratch lives in a buffer that is
    created once, sized for the object's capacity, and kept ON the object, so every call through
    that object sees the same addresses - which is what the reference's workspaces are for (CUDA
    graph capture, workspace.py:32-35).  The layout of the kernels here (routing, fp32 slot rows,
    gathered activations) is not the reference's, so its ``scratch`` / ``combine_out`` / ``act``
    tensors are not reinterpreted.  When ``matches()`` refused, the object is ignored and the call
    falls back to the per-device buffer, as the reference falls back to fresh allocations
    (triton/moe_int4_kernel.py:550-558)."""
    if workspace is None:
        return get_workspace(dev, nbytes)
    if isinstance(workspace, torch.Tensor):
        if workspace.dtype != torch.uint8 or not workspace.is_cuda or workspace.device != dev or not workspace.is_contiguous():
            raise ValueError("workspace tensor must be a contiguous uint8 tensor on the inputs' device")
        if workspace.numel() < nbytes or workspace.data_ptr() % 256:
            raise ValueError(f"workspace tensor needs {nbytes} bytes at a 256-byte aligned address "
                             f"(got {workspace.numel()} bytes)")
        return workspace
    if not fits:
        return get_workspace(dev, nbytes)
    buf = getattr(workspace, "_xkb200_scratch", None)
    if buf is None or buf.numel() < nbytes or buf.device != dev:
        buf = torch.empty(max(int(nbytes_at_capacity), int(nbytes)), dtype=torch.uint8, device=dev)
        workspace._xkb200_scratch = buf
    return buf


def check_workspace_status(workspace) -> None:
    """As :func:`check_status`, for a call that was given ``workspace=``."""
    buf = workspace if isinstance(workspace, torch.Tensor) else getattr(workspace, "_xkb200_scratch", None)
    if buf is None:
        return
    with torch.cuda.device(buf.device):
        _lib.check(_lib.load().xkb_workspace_status(buf.data_ptr(), _stream(buf.device)), "xkb_workspace_status")


def check_status(dev=None, tag: int = 0) -> None:
    """Synchronise and raise if a kernel of the last fused call on ``dev`` gave up a bounded
    wait (the tcgen05 kernels never spin without a limit; they record a status word instead)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if dev is None else torch.device(dev)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), tag)
    buf = _workspaces.get(key)
    if buf is None:
        return
    with torch.cuda.device(dev):
        _lib.check(_lib.load().xkb_workspace_status(buf.data_ptr(), _stream(dev)), "xkb_workspace_status")


def release_workspaces() -> None:
    """Drop the per-device buffers (only when no captured graph or queued work still uses them)."""
    _workspaces.clear()
    _retired.clear()


# ---------------------------------------------------------------------------
def moe_align_block_size(topk_ids, block_size, num_experts, truncate=True, workspace=None,
                         expert_map=None):
    """Sort/pad routed token-slots into per-expert blocks on the GPU.

    Same contract as ``moe_align_block_size_ref``
    (src/xkernels/ops/moe/w4a16.py:53-101): returns ``(sorted_token_ids
    [M*top_k + (E+1)*(block-1)], expert_ids, num_tokens_post_padded [1])``, all
    int32, bit-exact with the reference including the unused tails.
    ``truncate=True`` trims ``expert_ids`` to the used blocks and therefore
    reads ``num_tokens_post_padded`` back (one host sync); ``truncate=False`` is
    sync-free.  ``expert_map`` gives the expert-parallel form of
    ``moe_align_block_size_ep`` (w4a16.py:104-155): ``num_experts`` is then the
    local expert count and non-local slots are dropped.
    """
    lib = _lib.load()
    dev = _require_cuda("moe_align_block_size", topk_ids, expert_map)
    block_size, num_experts = int(block_size), int(num_experts)
    if block_size <= 0:
        raise ValueError("block_size must be > 0")
    ids = topk_ids.reshape(-1)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    ids = ids.contiguous()
    numel = ids.numel()
    emap = None
    if expert_map is not None:
        emap = expert_map.to(device=dev, dtype=torch.int32).contiguous()
    max_pad = numel + (num_experts + 1) * (block_size - 1)
    max_blocks = -(-max_pad // block_size)
    # A reference MoeAlignWorkspace (src/xkernels/ops/moe/workspace.py:85-151) that matches the call:
    # the three outputs are written INTO its buffers (address-stable, the reference's contract at
    # triton/align_kernel.py:198-213,245-250) and this kernel's own scratch is kept on the object.
    use_ws = False
    if workspace is not None and hasattr(workspace, "matches") and topk_ids.dim() == 2:
        use_ws = bool(workspace.matches(topk_ids.shape[0], topk_ids.shape[1], num_experts, block_size, device=dev))
    with torch.cuda.device(dev):
        ws_bytes = int(lib.xkb_moe_align_workspace_bytes(numel, num_experts))
        if use_ws:
            sorted_ids, expert_ids, num_post = workspace.sorted_ids, workspace.expert_ids, workspace.num_post
            if max_blocks == 0:
                expert_ids[:1].zero_()
            ws = getattr(workspace, "_xkb200_scratch", None)
            if ws is None or ws.numel() < ws_bytes:
                cap = int(lib.xkb_moe_align_workspace_bytes(max(workspace.sorted_ids.numel(), numel), num_experts))
                ws = torch.empty(max(cap, ws_bytes, 256), dtype=torch.uint8, device=dev)
                workspace._xkb200_scratch = ws
        else:
            sorted_ids = torch.empty(max_pad, dtype=torch.int32, device=dev)
            expert_ids = torch.empty(max(max_blocks, 1), dtype=torch.int32, device=dev)
            num_post = torch.empty(1, dtype=torch.int32, device=dev)
            if max_blocks == 0:
                expert_ids.zero_()
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        _lib.check(
            lib.xkb_moe_align_block_size(
                _ptr(ids), numel, num_experts, block_size, _ptr(emap),
                0 if emap is None else emap.numel(), _ptr(sorted_ids), _ptr(expert_ids),
                _ptr(num_post), 0, _ptr(ws), ws.numel(), _stream(dev)),
            "xkb_moe_align_block_size")
    sorted_ids = sorted_ids[:max_pad]
    if truncate:
        used = int(num_post.item()) // block_size
        expert_ids = expert_ids[: max(used, 1)]
    else:
        expert_ids = expert_ids[: max(max_blocks, 1)] if max_blocks == 0 else expert_ids[:max_blocks]
    return sorted_ids, expert_ids, num_post


# ---------------------------------------------------------------------------
_LOGIT_DT = {torch.bfloat16: _lib.XKB_BF16, torch.float32: _lib.XKB_F32, torch.float16: _lib.XKB_F16}


def topk_softmax(gating_output, topk, renormalize=True):
    """MoE router: fp32 softmax over all experts, top-k in descending probability (ties: ascending
    expert id), optional renormalisation.  Returns ``(topk_weights [M, topk] fp32, topk_ids [M, topk]
    int32)``.

    Reference: ``topk_softmax_ref`` (src/xkernels/ops/moe/topk_softmax.py:33-95).
    """
    lib = _lib.load()
    dev = _require_cuda("topk_softmax", gating_output)
    if gating_output.dim() != 2:
        raise ValueError("gating_output must be [M, E]")
    if gating_output.dtype not in _LOGIT_DT:
        raise TypeError(f"topk_softmax: logits must be bf16, fp16 or fp32, got {gating_output.dtype}")
    M, E = gating_output.shape
    if not (1 <= int(topk) <= E):
        raise ValueError(f"topk must satisfy 1 <= topk <= E (got topk={topk}, E={E})")
    g = gating_output.contiguous()
    with torch.cuda.device(dev):
        w = torch.empty((M, int(topk)), dtype=torch.float32, device=dev)
        ids = torch.empty((M, int(topk)), dtype=torch.int32, device=dev)
        _lib.check(
            lib.xkb_topk_softmax(_ptr(g), _LOGIT_DT[g.dtype], _ptr(w), _ptr(ids), M, E, int(topk),
                                 1 if renormalize else 0, _stream(dev)),
            "xkb_topk_softmax")
    return w, ids


# ---------------------------------------------------------------------------
def moe_sum_reduce(y, w=None, routed_scaling_factor=1.0):
    """``out[m] = routed_scaling_factor * sum_k w[m,k] * y[m,k,:]`` in fp32, ascending k.

    Reference: ``moe_sum_reduce_ref`` (src/xkernels/ops/moe/sum_reduce.py:20-39).
    ``y`` is ``[M, top_k, H]`` bf16/fp32, ``w`` ``[M, top_k]`` fp32/bf16 or None;
    the result has ``y.dtype``.
    """
    lib = _lib.load()
    dev = _require_cuda("moe_sum_reduce", y, w)
    if y.dim() != 3:
        raise ValueError("y must be [M, top_k, H]")
    if y.dtype not in _DT:
        raise TypeError(f"moe_sum_reduce: unsupported y dtype {y.dtype}")
    y = y.contiguous()
    M, top_k, H = y.shape
    if w is not None:
        if w.dtype not in _DT:
            w = w.to(torch.float32)
        if tuple(w.shape) != (M, top_k):
            raise ValueError(f"w must be [M, top_k] = [{M}, {top_k}], got {tuple(w.shape)}")
        w = w.contiguous()
    with torch.cuda.device(dev):
        out = torch.empty((M, H), dtype=y.dtype, device=dev)
        _lib.check(
            lib.xkb_moe_sum_reduce(_ptr(y), _DT[y.dtype], _ptr(w),
                                   _lib.XKB_F32 if w is None else _DT[w.dtype], _ptr(out),
                                   _DT[y.dtype], M, top_k, H, float(routed_scaling_factor),
                                   _stream(dev)),
            "xkb_moe_sum_reduce")
    return out


# ---------------------------------------------------------------------------
_checked_scales: dict[tuple[int, int], int] = {}
_INT4_SCALE_LIMIT = float(2 ** 24)


def _check_int4_scales(scale: torch.Tensor) -> None:
    """The tcgen05 INT4 dequantiser is exact for group scales below 2^24 in magnitude (it multiplies
    by s * 2^103 in bf16); a larger or non-finite scale would come out as inf/NaN, so such a tensor
    is refused.  Checked once per tensor (keyed by storage address, size and version counter): one
    reduction and one host read on the first call with it, so make that call before a stream capture."""
    key = (scale.data_ptr(), scale.numel())
    if _checked_scales.get(key) == scale._version:
        return
    top = float(scale.abs().max()) if scale.numel() else 0.0
    if not (top < _INT4_SCALE_LIMIT):        # also catches NaN
        raise ValueError(f"fused_moe_int4_w4a16: group scales must be finite and below 2^24 in magnitude (max |scale| = {top})")
    if len(_checked_scales) > 256:
        _checked_scales.clear()
    _checked_scales[key] = scale._version


def _routing_args(name, topk_ids, topk_w, expert_map, dev, M):
    if topk_ids.dim() != 2 or topk_ids.shape[0] != M:
        raise ValueError(f"{name}: topk_ids must be [M, top_k]")
    ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
    ids = ids.contiguous()
    tw = topk_w if topk_w.dtype == torch.float32 else topk_w.to(torch.float32)
    tw = tw.contiguous()
    if tuple(tw.shape) != tuple(ids.shape):
        raise ValueError(f"{name}: topk_w shape {tuple(tw.shape)} != topk_ids shape {tuple(ids.shape)}")
    emap = None
    if expert_map is not None:
        emap = expert_map.to(device=dev, dtype=torch.int32).contiguous()
    return ids, tw, emap


def fused_moe_int4_w4a16(A, packed, scale, topk_ids, topk_w, group_size=32, mul_routed_weight=True,
                         fused_combine=None, expert_map=None, workspace=None, *, path="auto"):
    """INT4 W4A16 grouped fused-MoE GEMM ``out[m] = sum_j w[m,j] * (A[m] @ W[e_mj]^T)``.

    Signature of the reference backends (src/xkernels/ops/moe/reference.py:22-33,
    triton/moe_int4_kernel.py:438-449).  ``fused_combine`` is accepted for API
    parity: the combine is always the fixed-order fp32 reduce.  ``workspace``:
    None (this package's per-device buffer), a CUDA uint8 tensor, or the
    reference's ``MoeInt4Workspace`` (see :func:`_caller_workspace`): with the
    latter two every call runs at the same addresses, e.g. under a CUDA graph.
    The tcgen05 kernels never wait without a limit; after a call
    :func:`check_status` (or :func:`check_workspace_status`) tells whether one gave up.
    ``expert_map`` selects the replicated expert-parallel mode (partial output).
    ``path``: ``"auto"`` | ``"simt"`` | ``"tc"``.
    """
    lib = _lib.load()
    dev = _require_cuda("fused_moe_int4_w4a16", A, packed, scale, topk_ids, topk_w, expert_map)
    if A.dtype not in _DT:
        raise TypeError(f"fused_moe_int4_w4a16: A must be bf16 or fp32, got {A.dtype}")
    if packed.dtype != torch.int32 or packed.dim() != 3:
        raise TypeError("fused_moe_int4_w4a16: packed must be int32 [E, N, K//8]")
    A = A.contiguous()
    packed = packed.contiguous()
    M, K = A.shape
    E, N, kp = packed.shape
    group_size = int(group_size)
    if kp * 8 != K:
        raise ValueError(f"packed last dim {kp} != K//8 = {K // 8}")
    if scale.dtype != torch.bfloat16:
        scale = scale.to(torch.bfloat16)
    scale = scale.contiguous()
    if tuple(scale.shape) != (E, N, K // group_size):
        raise ValueError(f"scale must be [E, N, K//group_size] = [{E}, {N}, {K // group_size}]")
    ids, tw, emap = _routing_args("fused_moe_int4_w4a16", topk_ids, topk_w, expert_map, dev, M)
    top_k = ids.shape[1]
    pcode = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tc": _lib.PATH_TC}[path]
    if path != "simt":
        _check_int4_scales(scale)
    with torch.cuda.device(dev):
        out = torch.empty((M, N), dtype=A.dtype, device=dev)
        ws_bytes = int(lib.xkb_fused_moe_int4_w4a16_workspace_bytes(M, N, K, E, top_k, _DT[A.dtype]))
        fits, cap_bytes = False, ws_bytes
        if workspace is not None and hasattr(workspace, "matches"):
            fits = bool(workspace.matches(M, top_k, N, dtype=A.dtype, device=dev))
            if fits:   # capacity of the object = rows of its combine buffer (workspace.py:199-213)
                cap_bytes = int(lib.xkb_fused_moe_int4_w4a16_workspace_bytes(int(workspace.combine_out.shape[0]), N, K, E,
                                                                             top_k, _DT[A.dtype]))
        ws = _caller_workspace(workspace, fits, cap_bytes, dev, ws_bytes)
        _lib.check(
            lib.xkb_fused_moe_int4_w4a16(
                _ptr(A), _DT[A.dtype], _ptr(packed), _ptr(scale), _ptr(ids), _ptr(tw), _ptr(emap),
                0 if emap is None else emap.numel(), _ptr(out), M, N, K, E, top_k, group_size,
                1 if mul_routed_weight else 0, pcode, _ptr(ws), ws.numel(), _stream(dev)),
            "xkb_fused_moe_int4_w4a16")
    return out


def fused_moe_mxfp4(A, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, b13=None, b2=None,
                    swiglu_limit=10.0, group_size=32, mul_routed_weight=True, expert_map=None,
                    workspace=None, *, path="auto"):
    """MXFP4 fused MoE: gate_up GEMM -> clamped SwiGLU -> down GEMM -> weighted combine.

    Signature of the reference backends
    (src/xkernels/ops/moe/mxfp4_reference.py:28-43, triton/moe_mxfp4_kernel.py:487-502).
    ``w13`` ``[E, 2*ispp, hidden//2]`` and ``w2`` ``[E, hidden, ispp//2]`` are uint8
    E2M1 pairs, the scales uint8 e8m0 per 32 elements.  The three bf16 rounding
    points of the reference (gate_up, activation, down) are reproduced.
    ``workspace`` as in :func:`fused_moe_int4_w4a16` (None, a CUDA uint8 tensor or the reference's
    ``MoeMxfp4Workspace``).  After a call :func:`check_status` (or :func:`check_workspace_status`)
    reports a kernel that gave up a bounded wait, a scale byte the prefill-sized tcgen05 instance
    does not convert (191..254), or a routing value out of range.
    """
    lib = _lib.load()
    dev = _require_cuda("fused_moe_mxfp4", A, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, b13, b2,
                        expert_map)
    if int(group_size) != 32:
        raise ValueError("fused_moe_mxfp4: the MX block size is 32")
    if A.dtype not in _DT:
        raise TypeError(f"fused_moe_mxfp4: A must be bf16 or fp32, got {A.dtype}")
    for name, t in (("w13", w13), ("w13_scale", w13_scale), ("w2", w2), ("w2_scale", w2_scale)):
        if t.dtype != torch.uint8:
            raise TypeError(f"fused_moe_mxfp4: {name} must be uint8")
    A = A.contiguous()
    w13, w13_scale, w2, w2_scale = (t.contiguous() for t in (w13, w13_scale, w2, w2_scale))
    M, hidden = A.shape
    E, two_ispp, half_hidden = w13.shape
    ispp = two_ispp // 2
    if half_hidden * 2 != hidden or tuple(w2.shape) != (E, hidden, ispp // 2):
        raise ValueError("fused_moe_mxfp4: w13 must be [E, 2*ispp, hidden//2] and w2 [E, hidden, ispp//2]")
    if tuple(w13_scale.shape) != (E, 2 * ispp, hidden // 32) or tuple(w2_scale.shape) != (E, hidden, ispp // 32):
        raise ValueError("fused_moe_mxfp4: scale shapes must be [E,2*ispp,hidden//32] and [E,hidden,ispp//32]")
    if b13 is not None:
        b13 = b13.to(torch.bfloat16).contiguous()
    if b2 is not None:
        b2 = b2.to(torch.bfloat16).contiguous()
    ids, tw, emap = _routing_args("fused_moe_mxfp4", topk_ids, topk_w, expert_map, dev, M)
    top_k = ids.shape[1]
    limit = 0.0 if swiglu_limit is None else float(swiglu_limit)
    pcode = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tc": _lib.PATH_TC}[path]
    with torch.cuda.device(dev):
        out = torch.empty((M, hidden), dtype=A.dtype, device=dev)
        ws_bytes = int(lib.xkb_fused_moe_mxfp4_workspace_bytes(M, hidden, ispp, E, top_k))
        fits, cap_bytes = False, ws_bytes
        if workspace is not None and hasattr(workspace, "out") and hasattr(workspace, "act"):
            # matches() of MoeMxfp4Workspace wants the align block of ITS kernel; what matters here is
            # that the object was built for this problem: same ispp / hidden / dtype, enough rows
            fits = (workspace.act.shape[1] == ispp and workspace.out.shape[1] == hidden and workspace.out.shape[0] >= M
                    and workspace.act.dtype == A.dtype and workspace.act.device == dev)
            if fits:
                cap_bytes = int(lib.xkb_fused_moe_mxfp4_workspace_bytes(int(workspace.out.shape[0]), hidden, ispp, E, top_k))
        ws = _caller_workspace(workspace, fits, cap_bytes, dev, ws_bytes)
        _lib.check(
            lib.xkb_fused_moe_mxfp4(
                _ptr(A), _DT[A.dtype], _ptr(w13), _ptr(w13_scale), _ptr(w2), _ptr(w2_scale), _ptr(ids),
                _ptr(tw), _ptr(b13), _ptr(b2), _ptr(emap), 0 if emap is None else emap.numel(),
                _ptr(out), M, hidden, ispp, E, top_k, limit, 1 if mul_routed_weight else 0, pcode,
                _ptr(ws), ws.numel(), _stream(dev)),
            "xkb_fused_moe_mxfp4")
    return out


def fused_moe_int4_ffn(A, w13_packed, w13_scale, w2_packed, w2_scale, topk_ids, topk_w, group_size=32,
                       swiglu_limit=None, expert_map=None, workspace=None, *, path="auto"):
    """One expert layer of two INT4 W4A16 GEMMs in one call: gate_up GEMM -> SwiGLU -> down GEMM ->
    weighted top-k combine.

    The reference has the single GEMM only (``fused_moe_int4_w4a16``, src/xkernels/ops/moe/interface.py:19-32;
    its INT4 benchmark measures the two shapes of such a layer, meta/benchmarks/bench_moe_int4_w4a16.py:3-12).
    This op returns what a caller of the reference gets from composing it: the first GEMM over the
    token's slots (bf16 result), ``act = (silu(gate) * up).to(A.dtype)`` with the gate rows first in
    ``w13``, the second GEMM with the routing weights (bf16 result per slot), ``moe_sum_reduce`` over
    the slots.  ``w13_packed [E, 2*inter, hidden//8]``, ``w13_scale [E, 2*inter, hidden//group]``,
    ``w2_packed [E, hidden, inter//8]``, ``w2_scale [E, hidden, inter//group]``.
    ``workspace`` and :func:`check_status` as in :func:`fused_moe_int4_w4a16`.
    """
    lib = _lib.load()
    dev = _require_cuda("fused_moe_int4_ffn", A, w13_packed, w13_scale, w2_packed, w2_scale, topk_ids, topk_w, expert_map)
    if A.dtype not in _DT:
        raise TypeError(f"fused_moe_int4_ffn: A must be bf16 or fp32, got {A.dtype}")
    for name, t in (("w13_packed", w13_packed), ("w2_packed", w2_packed)):
        if t.dtype != torch.int32 or t.dim() != 3:
            raise TypeError(f"fused_moe_int4_ffn: {name} must be int32 [E, rows, K//8]")
    A, w13_packed, w2_packed = A.contiguous(), w13_packed.contiguous(), w2_packed.contiguous()
    M, hidden = A.shape
    E, two_inter, kp = w13_packed.shape
    inter = two_inter // 2
    group_size = int(group_size)
    if kp * 8 != hidden or two_inter % 2 or tuple(w2_packed.shape) != (E, hidden, inter // 8):
        raise ValueError("fused_moe_int4_ffn: w13_packed must be [E, 2*inter, hidden//8] and w2_packed [E, hidden, inter//8]")
    w13_scale = (w13_scale if w13_scale.dtype == torch.bfloat16 else w13_scale.to(torch.bfloat16)).contiguous()
    w2_scale = (w2_scale if w2_scale.dtype == torch.bfloat16 else w2_scale.to(torch.bfloat16)).contiguous()
    if tuple(w13_scale.shape) != (E, 2 * inter, hidden // group_size) or tuple(w2_scale.shape) != (E, hidden, inter // group_size):
        raise ValueError("fused_moe_int4_ffn: scale shapes must be [E, 2*inter, hidden//group] and [E, hidden, inter//group]")
    ids, tw, emap = _routing_args("fused_moe_int4_ffn", topk_ids, topk_w, expert_map, dev, M)
    top_k = ids.shape[1]
    limit = 0.0 if swiglu_limit is None else float(swiglu_limit)
    pcode = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tc": _lib.PATH_TC}[path]
    if path != "simt":
        _check_int4_scales(w13_scale)
        _check_int4_scales(w2_scale)
    with torch.cuda.device(dev):
        out = torch.empty((M, hidden), dtype=A.dtype, device=dev)
        ws_bytes = int(lib.xkb_fused_moe_int4_ffn_workspace_bytes(M, hidden, inter, E, top_k, _DT[A.dtype]))
        ws = _caller_workspace(workspace if isinstance(workspace, torch.Tensor) else None, False, ws_bytes, dev, ws_bytes)
        _lib.check(
            lib.xkb_fused_moe_int4_ffn(
                _ptr(A), _DT[A.dtype], _ptr(w13_packed), _ptr(w13_scale), _ptr(w2_packed), _ptr(w2_scale), _ptr(ids),
                _ptr(tw), _ptr(emap), 0 if emap is None else emap.numel(), _ptr(out), M, hidden, inter, E, top_k,
                group_size, limit, pcode, _ptr(ws), ws.numel(), _stream(dev)),
            "xkb_fused_moe_int4_ffn")
    return out


# ---------------------------------------------------------------------------
# expert-parallel building blocks
# ---------------------------------------------------------------------------
def moe_int4_w4a16_rows(A, packed, scale, topk_ids, topk_w=None, group_size=32, *, path="auto"):
    """Grouped INT4 expert GEMM without the top-k combine: ``[M*top_k, N]`` fp32 rows, row
    ``m*top_k + j`` = ``A[m] @ W[topk_ids[m,j]]^T`` (times ``topk_w[m,j]`` if given)."""
    lib = _lib.load()
    dev = _require_cuda("moe_int4_w4a16_rows", A, packed, scale, topk_ids, topk_w)
    if A.dtype not in _DT:
        raise TypeError(f"moe_int4_w4a16_rows: A must be bf16 or fp32, got {A.dtype}")
    A, packed = A.contiguous(), packed.contiguous()
    scale = scale.to(torch.bfloat16).contiguous()
    M, K = A.shape
    E, N, _ = packed.shape
    ids = topk_ids.to(torch.int32).contiguous()
    top_k = ids.shape[1]
    tw = None if topk_w is None else topk_w.to(torch.float32).contiguous()
    pcode = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tc": _lib.PATH_TC}[path]
    if path != "simt":
        _check_int4_scales(scale)
    with torch.cuda.device(dev):
        rows = torch.empty((M * top_k, N), dtype=torch.float32, device=dev)
        if M == 0:
            return rows
        ws_bytes = int(lib.xkb_fused_moe_int4_w4a16_workspace_bytes(M, N, K, E, top_k, _DT[A.dtype]))
        ws = get_workspace(dev, ws_bytes)
        _lib.check(
            lib.xkb_moe_int4_w4a16_rows(_ptr(A), _DT[A.dtype], _ptr(packed), _ptr(scale), _ptr(ids),
                                        _ptr(tw), _ptr(rows), M, N, K, E, top_k, int(group_size),
                                        0 if tw is None else 1, pcode, _ptr(ws), ws.numel(), _stream(dev)),
            "xkb_moe_int4_w4a16_rows")
    return rows


def moe_int4_w4a16_partial(A, packed, scale, routing, group_size=32, *, out=None, path="auto", workspace_tag=0):
    """Expert side of the all-to-all mode in one C call: ``A [R, K]`` received rows, ``routing
    [R, 2*top_k]`` int32 (local expert ids, -1 = elsewhere, then the routing weights' bit patterns)
    -> ``[R, N]`` fp32, per row the weighted sum over its local experts in ascending slot order (a
    row without a local expert comes out as zeros).  Two calls that overlap on different streams must
    use different ``workspace_tag`` values (see :func:`get_workspace`)."""
    lib = _lib.load()
    dev = _require_cuda("moe_int4_w4a16_partial", A, packed, scale, routing, out)
    if A.dtype not in _DT:
        raise TypeError(f"moe_int4_w4a16_partial: A must be bf16 or fp32, got {A.dtype}")
    if routing.dtype != torch.int32 or routing.dim() != 2 or routing.shape[1] % 2:
        raise TypeError("moe_int4_w4a16_partial: routing must be int32 [R, 2*top_k]")
    A, packed, routing = A.contiguous(), packed.contiguous(), routing.contiguous()
    scale = scale if scale.dtype == torch.bfloat16 else scale.to(torch.bfloat16)
    scale = scale.contiguous()
    R, K = A.shape
    E, N, _ = packed.shape
    top_k = routing.shape[1] // 2
    if routing.shape[0] != R:
        raise ValueError("moe_int4_w4a16_partial: one routing row per received row")
    pcode = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tc": _lib.PATH_TC}[path]
    if path != "simt":
        _check_int4_scales(scale)
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((R, N), dtype=torch.float32, device=dev)
        if out.dtype != torch.float32 or tuple(out.shape) != (R, N) or not out.is_contiguous():
            raise ValueError("moe_int4_w4a16_partial: out must be a contiguous fp32 [R, N] tensor")
        if R == 0:
            return out
        ws_bytes = int(lib.xkb_moe_int4_w4a16_partial_workspace_bytes(R, N, K, E, top_k, _DT[A.dtype]))
        ws = get_workspace(dev, ws_bytes, tag=int(workspace_tag))
        _lib.check(
            lib.xkb_moe_int4_w4a16_partial(_ptr(A), _DT[A.dtype], _ptr(packed), _ptr(scale), _ptr(routing), _ptr(out),
                                           R, N, K, E, top_k, int(group_size), pcode, _ptr(ws), ws.numel(),
                                           _stream(dev)),
            "xkb_moe_int4_w4a16_partial")
    return out


def moe_gather_sum_reduce(rows, row_index, w, out_dtype=torch.bfloat16):
    """``out[m] = sum_k w[m,k] * rows[row_index[m,k]]`` in fp32, ascending k (index < 0 skips)."""
    lib = _lib.load()
    dev = _require_cuda("moe_gather_sum_reduce", rows, row_index, w)
    if rows.dtype != torch.float32:
        raise TypeError("moe_gather_sum_reduce: rows must be fp32")
    rows = rows.contiguous()
    idx = row_index.to(torch.int32).contiguous()
    M, top_k = idx.shape
    H = rows.shape[1]
    w = None if w is None else w.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        out = torch.empty((M, H), dtype=out_dtype, device=dev)
        _lib.check(
            lib.xkb_moe_gather_sum_reduce(_ptr(rows), _ptr(idx), _ptr(w), _ptr(out), _DT[out_dtype], M, top_k,
                                          H, _stream(dev)),
            "xkb_moe_gather_sum_reduce")
    return out


def gather_rows(src, index, count=None, out=None):
    """``out[p] = src[index[p]]`` for ``p < count[0]`` (``count`` a device int32 tensor; all of
    ``index`` if None).  ``out`` (``[>= len(index), row]``) may be a preallocated buffer; rows at and
    beyond the count are left untouched."""
    lib = _lib.load()
    dev = _require_cuda("gather_rows", src, index, count, out)
    src = src.contiguous()
    idx = index if index.dtype == torch.int32 else index.to(torch.int32)
    idx = idx.contiguous()
    row_bytes = src.shape[1] * src.element_size()
    n = idx.numel()
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((n, src.shape[1]), dtype=src.dtype, device=dev)
        if out.dtype != src.dtype or out.shape[1] != src.shape[1] or out.shape[0] < n or not out.is_contiguous():
            raise ValueError("gather_rows: out must be a contiguous [>= len(index), row] tensor of src's dtype")
        _lib.check(lib.xkb_gather_rows(_ptr(src), src.shape[0], row_bytes, _ptr(idx), _ptr(count), n, _ptr(out),
                                       _stream(dev)), "xkb_gather_rows")
    return out


_PLACEMENT = {"contiguous": 0, "round_robin": 1, "snake": 2}


def ep_plan(topk_ids, topk_w, experts_per_rank, world, placement="contiguous", chunks=1, table=None):
    """Device-side dispatch plan of the all-to-all expert-parallel mode (``xkb_ep_plan``): no host
    read.  Returns ``(pair_token, pair_dest, routing, pair_of, counts, info)`` with the per-pair
    arrays sized ``M * top_k`` (the first ``info[0]`` entries are the pairs); see
    ``xkernels_b200/ep.py:plan_dispatch`` for the meaning of each.  ``table`` (``[E, 2]`` int32 on the
    device: destination rank and expert index there, per global expert) overrides ``placement``."""
    lib = _lib.load()
    dev = _require_cuda("ep_plan", topk_ids, topk_w)
    if placement not in _PLACEMENT:
        raise ValueError(f"unknown expert placement {placement!r}")
    ids = topk_ids.to(torch.int32).contiguous()
    w = topk_w.to(torch.float32).contiguous()
    M, top_k = ids.shape
    numel = M * top_k
    if table is not None:
        if table.dtype != torch.int32 or tuple(table.shape) != (int(experts_per_rank) * int(world), 2) or not table.is_cuda:
            raise ValueError("ep_plan: table must be a CUDA int32 tensor of shape [experts_per_rank * world, 2]")
        table = table.contiguous()
    with torch.cuda.device(dev):
        pair_token = torch.empty((numel,), dtype=torch.int32, device=dev)
        pair_dest = torch.empty((numel,), dtype=torch.int32, device=dev)
        routing = torch.empty((numel, 2 * top_k), dtype=torch.int32, device=dev)
        pair_of = torch.empty((M, world), dtype=torch.int32, device=dev)
        counts = torch.empty((chunks, world), dtype=torch.int32, device=dev)
        info = torch.empty((2,), dtype=torch.int32, device=dev)
        ws_bytes = int(lib.xkb_ep_plan_workspace_bytes(M, top_k, world, chunks))
        ws = get_workspace(dev, ws_bytes, tag=1)     # not the fused ops' buffer: that one starts with their status words
        _lib.check(
            lib.xkb_ep_plan(_ptr(ids), _ptr(w), M, top_k, int(experts_per_rank), int(world),
                            _PLACEMENT[placement], _ptr(table), int(chunks), _ptr(pair_token), _ptr(pair_dest),
                            _ptr(routing), _ptr(pair_of), _ptr(counts), _ptr(info), _ptr(ws), ws.numel(),
                            _stream(dev)),
            "xkb_ep_plan")
    return pair_token, pair_dest, routing, pair_of, counts, info
