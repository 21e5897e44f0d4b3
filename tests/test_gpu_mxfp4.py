"""fused_moe_mxfp4 on the GPU, through the C-ABI, vs the oracle and the fixtures made by the
reference.  Tolerance: |a-e| <= 1e-2 + 2e-2|e| (task statement; the reference's own GPU test
uses 3e-2, tests/test_moe_mxfp4.py:48).  The kernels round at the reference's three bf16
rounding points, so only fp32 accumulation order differs; on outputs with heavy cancellation a
few elements per 10^4 can land on the other side of a bf16 rounding boundary of an intermediate
and miss the criterion, hence the small allowance stated per test."""

import pytest
import torch

import xkernels_b200 as xkb
from oracle import moe_oracle as oracle
from tests.golden.golden_io import load_case
from tests.gpu_util import assert_within, to_dev
from xkernels_b200 import synth

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2
KEYS = ("A", "w13", "w13_scale", "w2", "w2_scale", "topk_ids", "topk_w", "b13", "b2")


def call(c, dev, **kw):
    d = to_dev({k: c.get(k) for k in KEYS}, dev)
    return xkb.fused_moe_mxfp4(d["A"], d["w13"], d["w13_scale"], d["w2"], d["w2_scale"], d["topk_ids"],
                               d["topk_w"], b13=d["b13"], b2=d["b2"], **kw)


@pytest.mark.parametrize("name", ["mxfp4_small", "mxfp4_small_bias", "mxfp4_mid", "mxfp4_fp32_act",
                                  "mxfp4_scales", "mxfp4_tc_scales"])
@pytest.mark.parametrize("path", ["auto", "simt"])
def test_golden(name, path, cuda_device):
    c = load_case(name)
    out = call(c, cuda_device, swiglu_limit=c["swiglu_limit"], path=path)
    assert_within(out, c["out"], RTOL, ATOL, what=f"{name}/{path}", allowed=max(1, c["out"].numel() // 2000))


@pytest.mark.parametrize("M,hidden,ispp,E,top_k,bias", [
    (1, 64, 32, 4, 2, False), (37, 96, 64, 8, 3, True), (16, 256, 128, 5, 4, False),
    (48, 512, 256, 16, 6, True),
    (48, 512, 512, 16, 6, True),      # multiples of 512: the tcgen05 kernels, 16-token tiles
    (40, 1024, 512, 8, 4, False),     # four 256-K stages in gate_up, two in down
    (640, 512, 512, 4, 2, True),      # more than 48 slots per expert: the 128-token tiles
    (300, 512, 1024, 3, 2, False),    # ragged last blocks in the wide mode
])
def test_against_oracle_with_repeated_ids(M, hidden, ispp, E, top_k, bias, cuda_device):
    g = torch.Generator().manual_seed(M + hidden)
    wts = synth.mxfp4_weights(E, hidden, ispp, seed=M, scale_lo=119, scale_hi=124, with_bias=bias)
    A = torch.randn(M, hidden, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, E, (M, top_k), generator=g, dtype=torch.int32)
    w = torch.rand(M, top_k, generator=g)
    c = {"A": A, **wts, "topk_ids": ids, "topk_w": w}
    want = oracle.moe_mxfp4(A, wts["w13"], wts["w13_scale"], wts["w2"], wts["w2_scale"], ids, w,
                            b13=wts["b13"], b2=wts["b2"])
    got = call(c, cuda_device)
    assert_within(got, want, RTOL, ATOL, what="auto", allowed=max(1, want.numel() // 2000))
    assert torch.equal(got, call(c, cuda_device)), "second run differs: the combine must be deterministic"


def test_expert_parallel_partials_sum_to_dense(cuda_device):
    """Replicated EP mode (tests/test_moe_mxfp4.py:173-219 in the reference): per-rank partials
    with an expert_map sum to the dense result."""
    c = load_case("mxfp4_mid")
    dense = call(c, cuda_device, swiglu_limit=10.0).float().cpu()
    E = c["w13"].shape[0]
    total = torch.zeros_like(dense)
    mags = torch.zeros_like(dense)
    for rank in range(2):
        emap = torch.full((E,), -1, dtype=torch.int32)
        lo, hi = rank * E // 2, (rank + 1) * E // 2
        emap[lo:hi] = torch.arange(hi - lo, dtype=torch.int32)
        d = to_dev({k: c.get(k) for k in KEYS}, cuda_device)
        part = xkb.fused_moe_mxfp4(d["A"], d["w13"][lo:hi].contiguous(), d["w13_scale"][lo:hi].contiguous(),
                                   d["w2"][lo:hi].contiguous(), d["w2_scale"][lo:hi].contiguous(),
                                   d["topk_ids"], d["topk_w"], b13=d["b13"][lo:hi].contiguous(),
                                   b2=d["b2"][lo:hi].contiguous(), expert_map=emap.to(cuda_device))
        want = oracle.moe_mxfp4(c["A"], c["w13"][lo:hi], c["w13_scale"][lo:hi], c["w2"][lo:hi],
                                c["w2_scale"][lo:hi], c["topk_ids"], c["topk_w"], b13=c["b13"][lo:hi],
                                b2=c["b2"][lo:hi], expert_map=emap)
        assert_within(part, want, RTOL, ATOL, what=f"partial {rank}", allowed=max(1, want.numel() // 2000))
        total += part.float().cpu()
        mags += part.float().cpu().abs()
    # each partial is rounded to bf16 on its own, so the sum carries up to half a bf16 ulp of
    # every partial: allow 2^-8 of the partials' magnitudes on top of the op tolerance
    slack = 3e-2 + 3e-2 * dense.abs() + 2.0 ** -8 * mags
    assert bool(((total - dense).abs() <= slack).all()), "sum of partials differs from the dense result"


@pytest.mark.parametrize("path", ["simt", "tc"])
@pytest.mark.parametrize("with_map", [False, True])
def test_slots_without_a_local_expert_are_dropped(path, with_map, cuda_device):
    """Ids of -1 and ids >= E contribute nothing (ops/moe/mxfp4_reference.py:82-83); the combine
    must not add the never-written rows of those slots (workspace poisoned beforehand)."""
    from xkernels_b200 import ops

    cfg = synth.Mxfp4Config("drop", M=24, hidden=512, ispp=512, E=6, top_k=3, scale_lo=119, scale_hi=124)
    c = synth.make_mxfp4(cfg, seed=5)
    g = torch.Generator().manual_seed(4)
    ids = c["topk_ids"].clone()
    kill = torch.rand(cfg.M, cfg.top_k, generator=g)
    ids[kill < 0.2] = -1
    ids[(kill >= 0.2) & (kill < 0.4)] = cfg.E + 1
    ids[0] = -1
    emap = None
    if with_map:
        emap = torch.arange(cfg.E + 4, dtype=torch.int32)
        emap[cfg.E:] = -1
        emap[1] = -1
    want = oracle.moe_mxfp4(c["A"], c["w13"], c["w13_scale"], c["w2"], c["w2_scale"], ids.clamp(min=-1), c["topk_w"],
                            expert_map=None if emap is None else torch.cat([emap, torch.tensor([-1], dtype=torch.int32)]))
    d = to_dev({k: c.get(k) for k in KEYS}, cuda_device)
    ops.get_workspace(cuda_device, 1 << 24).view(torch.float32)[64:].fill_(1.0e4)
    got = xkb.fused_moe_mxfp4(d["A"], d["w13"], d["w13_scale"], d["w2"], d["w2_scale"], ids.to(cuda_device),
                              d["topk_w"], expert_map=None if emap is None else emap.to(cuda_device), path=path)
    ops.check_status(cuda_device)
    assert_within(got, want, RTOL, ATOL, what=f"dropped slots/{path}/map={with_map}", allowed=max(1, want.numel() // 2000))
    assert bool((got[0] == 0).all())


def test_decode_config_full(cuda_device):
    """E=256, hidden=4096, ispp=512, top_k=6, M=48, scales in [118,130]: |out| ~ 4e3 with heavy
    cancellation.  The whole output is compared with the oracle (8 s of CPU); the measured
    fraction of elements outside the criterion is bounded at 0.1 %."""
    cfg = synth.CONFIGS["mxfp4_decode"]
    d = synth.make_mxfp4(cfg, seed=1729, device=cuda_device)
    out = xkb.fused_moe_mxfp4(d["A"], d["w13"], d["w13_scale"], d["w2"], d["w2_scale"], d["topk_ids"],
                              d["topk_w"])
    assert out.shape == (cfg.M, cfg.hidden) and out.dtype == torch.bfloat16
    cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    want = oracle.moe_mxfp4(cpu["A"], cpu["w13"], cpu["w13_scale"], cpu["w2"], cpu["w2_scale"],
                            cpu["topk_ids"], cpu["topk_w"])
    assert_within(out, want, RTOL, ATOL, what="mxfp4 decode", allowed=out.numel() // 1000)
    again = xkb.fused_moe_mxfp4(d["A"], d["w13"], d["w13_scale"], d["w2"], d["w2_scale"], d["topk_ids"],
                                d["topk_w"])
    assert torch.equal(out, again)
