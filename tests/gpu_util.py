"""Helpers shared by the GPU parity tests."""

import torch

from oracle import moe_oracle as oracle


def to_dev(case: dict, dev) -> dict:
    return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}


def assert_within(actual: torch.Tensor, expected: torch.Tensor, rtol: float, atol: float, what: str = "",
                  allowed: int = 0):
    a, e = actual.detach().cpu(), expected.detach().cpu()
    assert a.shape == e.shape and a.dtype == e.dtype, f"{what}: {a.shape}/{a.dtype} vs {e.shape}/{e.dtype}"
    bad = oracle.count_violations(a, e, rtol, atol)
    if bad > allowed:
        d = (a.double() - e.double()).abs()
        idx = int(d.argmax())
        raise AssertionError(
            f"{what}: {bad}/{a.numel()} elements outside |a-e| <= {atol} + {rtol}|e| (allowed {allowed}); "
            f"max abs diff {d.max().item():.4g} at flat index {idx}: got {a.flatten()[idx].item()}, "
            f"want {e.flatten()[idx].item()}")
