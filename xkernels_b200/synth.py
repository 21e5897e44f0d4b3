"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (tiny INT4, INT4 decode, INT4 prefill + align, MXFP4,
expert-parallel INT4).  No dataset is involved anywhere on this path: the
reference itself measures on random tensors (meta/benchmarks/bench_all.py:226-239).

Everything is drawn from a ``torch.Generator`` on the requested device, so the
CUDA kernels and a CPU checker see identical bits after a ``.cpu()`` copy.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Int4Config:
    name: str
    M: int
    K: int
    N: int
    E: int
    top_k: int
    group_size: int = 32
    expert_bias_std: float = 0.0     # per-expert N(0, std) logit bias (prefill skew)
    zipf_scale: float = 0.0          # 2.0 * rank^-1.1 logit bias (expert-parallel skew)


@dataclass(frozen=True)
class Mxfp4Config:
    name: str
    M: int
    hidden: int
    ispp: int
    E: int
    top_k: int
    scale_lo: int = 118
    scale_hi: int = 130


CONFIGS = {
    "int4_tiny": Int4Config("int4_tiny", M=16, K=512, N=256, E=8, top_k=2),
    "int4_decode": Int4Config("int4_decode", M=64, K=7168, N=4096, E=48, top_k=8),
    "int4_prefill": Int4Config("int4_prefill", M=16384, K=7168, N=4096, E=48, top_k=8,
                               expert_bias_std=0.5),
    "mxfp4_decode": Mxfp4Config("mxfp4_decode", M=48, hidden=4096, ispp=512, E=256, top_k=6),
    "int4_ep": Int4Config("int4_ep", M=4096, K=7168, N=2048, E=256, top_k=8, zipf_scale=2.0),
}


def _gen(device, seed: int) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(int(seed))


def activations(M: int, K: int, *, seed: int, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    return torch.randn(M, K, generator=_gen(device, seed), device=device, dtype=torch.float32).to(dtype)


def routing(M: int, E: int, top_k: int, *, seed: int, device="cpu", expert_bias_std: float = 0.0,
            zipf_scale: float = 0.0):
    """Router logits ~N(0,1) (+ optional per-expert bias) -> softmax -> top-k distinct ids
    (int32) with renormalised fp32 weights."""
    g = _gen(device, seed)
    logits = torch.randn(M, E, generator=g, device=device, dtype=torch.float32)
    if expert_bias_std > 0:
        logits = logits + expert_bias_std * torch.randn(E, generator=g, device=device)
    if zipf_scale > 0:
        rank = torch.arange(1, E + 1, device=device, dtype=torch.float32)
        logits = logits + zipf_scale * rank.pow(-1.1)
    probs = torch.softmax(logits, dim=-1)
    w, ids = torch.topk(probs, top_k, dim=-1)
    w = (w / w.sum(dim=-1, keepdim=True)).to(torch.float32)
    return ids.to(torch.int32).contiguous(), w.contiguous()


def int4_weights(E: int, N: int, K: int, group_size: int = 32, *, seed: int, device="cpu"):
    """``packed [E,N,K//8]`` int32 with uniform 4-bit codes (zero point 8, low nibble =
    lowest k) and ``scale [E,N,K//g]`` bf16 = |N(0,1)| * 0.02.  A uniform random 32-bit
    word is eight independent uniform nibbles, so the words are drawn directly."""
    g = _gen(device, seed)
    packed = torch.randint(-(2 ** 31), 2 ** 31, (E, N, K // 8), generator=g, device=device,
                           dtype=torch.int64).to(torch.int32)
    g2 = _gen(device, seed + 1)
    scale = (torch.randn(E, N, K // group_size, generator=g2, device=device,
                         dtype=torch.float32).abs() * 0.02).to(torch.bfloat16)
    return packed, scale


def pack_int4_codes(codes: torch.Tensor) -> torch.Tensor:
    """``codes [..., K]`` in [0,15] -> ``[..., K//8]`` int32, low nibble = lowest k."""
    *lead, K = codes.shape
    shifts = torch.arange(8, device=codes.device, dtype=torch.int64) * 4
    words = (codes.reshape(*lead, K // 8, 8).to(torch.int64) << shifts).sum(dim=-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def mxfp4_weights(E: int, hidden: int, ispp: int, *, seed: int, device="cpu", scale_lo: int = 118,
                  scale_hi: int = 130, with_bias: bool = False):
    """``w13 [E,2*ispp,hidden//2]``/``w2 [E,hidden,ispp//2]`` uint8 (uniform bytes = uniform
    E2M1 codes) and e8m0 scales uniform in [scale_lo, scale_hi]."""
    g = _gen(device, seed)

    def one(rows: int, cols: int):
        p = torch.randint(0, 256, (E, rows, cols // 2), generator=g, device=device, dtype=torch.uint8)
        s = torch.randint(scale_lo, scale_hi + 1, (E, rows, cols // 32), generator=g, device=device,
                          dtype=torch.uint8)
        return p, s

    w13, w13_scale = one(2 * ispp, hidden)
    w2, w2_scale = one(hidden, ispp)
    out = {"w13": w13, "w13_scale": w13_scale, "w2": w2, "w2_scale": w2_scale, "b13": None, "b2": None}
    if with_bias:
        out["b13"] = (torch.rand(E, 2 * ispp, generator=g, device=device) * 0.2 - 0.1).to(torch.bfloat16)
        out["b2"] = (torch.rand(E, hidden, generator=g, device=device) * 0.2 - 0.1).to(torch.bfloat16)
    return out


def make_int4(cfg: Int4Config, *, seed: int = 1729, device="cpu", M: int | None = None,
              experts: tuple[int, int] | None = None):
    """All tensors of an INT4 configuration.  ``experts=(lo, hi)`` materialises only that
    slice of the expert weights (expert-parallel shards); routing stays global."""
    M = cfg.M if M is None else M
    A = activations(M, cfg.K, seed=seed, device=device)
    lo, hi = (0, cfg.E) if experts is None else experts
    packed, scale = int4_weights(hi - lo, cfg.N, cfg.K, cfg.group_size, seed=seed + 1 + 7 * lo, device=device)
    ids, w = routing(M, cfg.E, cfg.top_k, seed=seed + 3, device=device,
                     expert_bias_std=cfg.expert_bias_std, zipf_scale=cfg.zipf_scale)
    return {"A": A, "packed": packed, "scale": scale, "topk_ids": ids, "topk_w": w,
            "group_size": cfg.group_size}


def make_mxfp4(cfg: Mxfp4Config, *, seed: int = 1729, device="cpu", with_bias: bool = False):
    A = activations(cfg.M, cfg.hidden, seed=seed, device=device)
    wts = mxfp4_weights(cfg.E, cfg.hidden, cfg.ispp, seed=seed + 1, device=device,
                        scale_lo=cfg.scale_lo, scale_hi=cfg.scale_hi, with_bias=with_bias)
    ids, w = routing(cfg.M, cfg.E, cfg.top_k, seed=seed + 3, device=device)
    return {"A": A, **wts, "topk_ids": ids, "topk_w": w}


def int4_algorithmic_bytes(cfg: Int4Config, n_active_experts: int, M: int | None = None) -> int:
    """Bytes one call must move: active experts' packed weights and scales, activations in,
    output out, routing ids + weights."""
    M = cfg.M if M is None else M
    per_expert = cfg.N * (cfg.K // 2 + 2 * cfg.K // cfg.group_size)
    return n_active_experts * per_expert + M * cfg.K * 2 + M * cfg.N * 2 + M * cfg.top_k * 8


def int4_flops(cfg: Int4Config, M: int | None = None) -> int:
    M = cfg.M if M is None else M
    return 2 * M * cfg.top_k * cfg.N * cfg.K


def mxfp4_algorithmic_bytes(cfg: Mxfp4Config, n_active_experts: int) -> int:
    per_expert = (2 * cfg.ispp * (cfg.hidden // 2 + cfg.hidden // 32)
                  + cfg.hidden * (cfg.ispp // 2 + cfg.ispp // 32))
    return n_active_experts * per_expert + 2 * cfg.M * cfg.hidden * 2
