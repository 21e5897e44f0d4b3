"""npz (de)serialisation of golden cases: torch tensors in, torch tensors out.
bf16 tensors are stored as their int16 bit patterns under a ``::bf16`` key suffix;
``None`` values under ``::none``; Python scalars as 0-d arrays under ``::py``."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent


def save_case(name: str, case: dict) -> Path:
    arrays = {}
    for k, v in case.items():
        if v is None:
            arrays[k + "::none"] = np.zeros(0)
        elif isinstance(v, torch.Tensor):
            if v.dtype == torch.bfloat16:
                arrays[k + "::bf16"] = v.contiguous().view(torch.int16).numpy()
            else:
                arrays[k] = v.contiguous().numpy()
        elif isinstance(v, np.ndarray):
            arrays[k] = v
        else:
            arrays[k + "::py"] = np.asarray(v)
    path = GOLDEN_DIR / f"{name}.npz"
    np.savez_compressed(path, **arrays)
    return path


def load_case(name: str) -> dict:
    out = {}
    with np.load(GOLDEN_DIR / f"{name}.npz") as z:
        for k in z.files:
            a = z[k]
            if k.endswith("::none"):
                out[k[:-6]] = None
            elif k.endswith("::bf16"):
                out[k[:-6]] = torch.from_numpy(a.copy()).view(torch.bfloat16)
            elif k.endswith("::py"):
                out[k[:-4]] = a.item()
            else:
                out[k] = torch.from_numpy(a.copy())
    return out
