"""Registers this package as the ``backend="cuda"`` implementation of the fused-MoE ops inside an
installed ``xkernels`` (the reference) — without touching the reference's files.

``install()`` does three things, all through the reference's own seams:

1. ``register(kernel, Backend.CUDA)(fn)`` for ``moe_int4_w4a16``, ``moe_mxfp4``,
   ``moe_align_block_size`` and ``moe_sum_reduce`` (src/xkernels/_dispatch.py:90-95), so that
   ``dispatch(..., backend="auto")`` picks them first on NVIDIA (``_dispatch.py:37-41``);
2. builds an overlay registry directory = the reference's ``registry/`` (ops, shape sweeps, schema,
   cards) with this package's cards added, ``moe_sum_reduce.cuda.card.json`` replaced (the loader
   allows one card per (op, backend), src/xkernels/registry/loader.py:89-94) and the missing
   ``moe_mxfp4`` spec / sweep / reference card supplied, then points the reference's registry root at
   it (src/xkernels/registry/schemas.py:9) and clears the loader cache (loader.py:99-101);
3. registers a seeded input generator for ``moe_mxfp4@1.0.0``
   (src/xkernels/registry/input_gen.py:437-446) built on the reference's own packing helper.

After that the reference's unchanged ``find_impl``, ``verify`` and ``verify_parity`` see the cards.
"""

from __future__ import annotations

import shutil
import tempfile
from pathlib import Path

OVERLAY_SRC = Path(__file__).resolve().parent / "registry"
KERNELS = ("moe_int4_w4a16", "moe_mxfp4", "moe_align_block_size", "moe_sum_reduce", "topk_softmax")
CARD_IDS = ("moe_int4_w4a16.cuda@1.0.0", "moe_align_block_size.cuda@1.0.0", "moe_sum_reduce.cuda@1.1.0",
            "moe_mxfp4.cuda@1.0.0", "topk_softmax.cuda@1.0.0")

_installed_root: Path | None = None


def _align_backend(topk_ids, block_size, num_experts, truncate=True, workspace=None):
    from . import ops

    return ops.moe_align_block_size(topk_ids, block_size, num_experts, truncate=truncate, workspace=workspace)


def _mxfp4_input_gen(point: dict, seed: int, device: str) -> dict:
    """Seeded inputs for ``moe_mxfp4@1.0.0`` in the style of the reference's INT4 generator
    (input_gen.py:138-159): weights from ``make_mxfp4_moe_weights``, ids drawn with replacement,
    uniform un-normalised routing weights."""
    import torch
    from xkernels.ops.moe.mxfp4 import make_mxfp4_moe_weights
    from xkernels.registry.dtypes import to_torch_dtype

    dt = to_torch_dtype(point["dtype"])
    M, hidden, ispp = int(point["M"]), int(point["hidden"]), int(point["ispp"])
    E, top_k = int(point["E"]), int(point["top_k"])
    g = torch.Generator(device=device).manual_seed(int(seed))
    A = torch.randn(M, hidden, generator=g, device=device, dtype=dt)
    w = make_mxfp4_moe_weights(E, hidden, ispp, device=device, seed=seed + 1)
    g2 = torch.Generator(device=device).manual_seed(int(seed) + 2)
    topk_ids = torch.randint(0, E, (M, top_k), generator=g2, device=device, dtype=torch.int32)
    topk_w = torch.rand(M, top_k, generator=g2, device=device, dtype=torch.float32)
    return {"A": A, "w13": w["w13"], "w13_scale": w["w13_scale"], "w2": w["w2"], "w2_scale": w["w2_scale"],
            "topk_ids": topk_ids, "topk_w": topk_w}


def build_overlay(dest: Path, reference_root: Path) -> Path:
    """``dest`` := reference registry + this package's registry files (ours win on name clashes)."""
    dest.mkdir(parents=True, exist_ok=True)
    for sub in ("ops", "impls", "shape_sweeps", "schema"):
        (dest / sub).mkdir(exist_ok=True)
        src = reference_root / sub
        if src.is_dir():
            for f in src.iterdir():
                if f.is_file():
                    shutil.copyfile(f, dest / sub / f.name)
    for sub in ("ops", "impls", "shape_sweeps"):
        for f in (OVERLAY_SRC / sub).glob("*.json"):
            shutil.copyfile(f, dest / sub / f.name)
    return dest


def install(overlay_dir: str | Path | None = None) -> Path:
    """Register the CUDA backends and activate the overlay registry.  Returns the overlay path.
    Raises ImportError if ``xkernels`` is not importable, and whatever ``_lib.load()`` raises if
    ``libxkb200.so`` is missing (there is no fallback to register instead)."""
    global _installed_root
    import xkernels  # the reference
    from xkernels._backends import Backend
    from xkernels._dispatch import register
    from xkernels.registry import input_gen, loader, schemas

    from . import _lib, ops

    _lib.load()
    register("moe_int4_w4a16", Backend.CUDA)(ops.fused_moe_int4_w4a16)
    register("moe_mxfp4", Backend.CUDA)(ops.fused_moe_mxfp4)
    register("moe_align_block_size", Backend.CUDA)(_align_backend)
    register("moe_sum_reduce", Backend.CUDA)(ops.moe_sum_reduce)
    register("topk_softmax", Backend.CUDA)(ops.topk_softmax)

    reference_root = Path(schemas.registry_root())
    if not (reference_root / "ops").is_dir():
        # a wheel install leaves the registry data beside the package instead of three levels up
        beside = Path(xkernels.__file__).resolve().parent.parent / "registry"
        if (beside / "ops").is_dir():
            reference_root = beside
            schemas._SCHEMA_DIR = beside / "schema"
        else:
            raise RuntimeError(f"the reference's registry data was found neither at {reference_root} nor at {beside}")
    if _installed_root is not None and reference_root == _installed_root:
        return _installed_root  # already active
    dest = Path(overlay_dir) if overlay_dir is not None else Path(tempfile.mkdtemp(prefix="xkb200_registry_"))
    build_overlay(dest, reference_root)
    schemas._REGISTRY_ROOT = dest
    loader.reset_cache()
    input_gen.register_input_gen("moe_mxfp4@1.0.0", _mxfp4_input_gen)
    _installed_root = dest
    return dest


def write_back(card_id: str, *, shape: dict, dtype: str, source: str, ms: float | None = None,
               tflops: float | None = None, achieved_bw_pct: float | None = None, knobs: dict | None = None,
               arch: str = "nvidia_sm100", cards_dir: str | Path | None = None) -> dict:
    """Record one measurement on a card of this package through the reference's OWN
    ``record_measurement`` (src/xkernels/registry/writeback.py:30-93: a source and an arch are
    mandatory, an entry for the same (arch, shape, dtype, knobs) point is replaced), then copy the
    updated card file from the overlay registry to ``cards_dir`` (default: this package's
    ``registry/impls``), so that ``perf.measured`` in the repository is written by code."""
    install()
    from xkernels.registry import schemas
    from xkernels.registry.writeback import record_measurement

    res = record_measurement(card_id, arch, shape, dtype, source, knobs=knobs, tflops=tflops,
                             achieved_bw_pct=achieved_bw_pct, ms=ms)
    name = card_id.split("@", 1)[0] + ".card.json"
    dest_dir = Path(cards_dir) if cards_dir is not None else OVERLAY_SRC / "impls"
    dest_dir.mkdir(parents=True, exist_ok=True)
    shutil.copyfile(Path(schemas.registry_root()) / "impls" / name, dest_dir / name)
    return res
