"""topk_softmax (the router in front of the fused-MoE path) on the GPU, through the C-ABI, vs the
fixtures made by the reference and vs the oracle.  The selected ids are compared exactly; the
weights within the spec's per-dtype tolerance (registry/ops/topk_softmax.spec.json in the
reference: fp32 1e-5/1e-6, bf16 and fp16 1e-2/1e-2) -- the softmax here divides by a sum taken
in warp-shuffle order, which can differ from torch's in the last fp32 bit."""

import pytest
import torch

import xkernels_b200 as xkb
from oracle import moe_oracle as oracle
from tests.golden.golden_io import load_case

pytestmark = pytest.mark.gpu

CASES = [f"topk_softmax_sweep{i}" for i in range(6)] + [
    "topk_softmax_ties_bf16", "topk_softmax_ties_fp16", "topk_softmax_all_equal", "topk_softmax_wide_renorm",
    "topk_softmax_wide_raw", "topk_softmax_single"]
TOL = {torch.float32: (1e-5, 1e-6), torch.bfloat16: (1e-2, 1e-2), torch.float16: (1e-2, 1e-2)}


def _check(w, ids, want_w, want_ids, dtype, what):
    assert ids.dtype == torch.int32 and w.dtype == torch.float32
    assert torch.equal(ids.cpu(), want_ids), f"{what}: selected experts differ"
    rtol, atol = TOL[dtype]
    err = (w.cpu() - want_w).abs()
    assert bool((err <= atol + rtol * want_w.abs()).all()), f"{what}: weights differ, max err {float(err.max()):.3g}"


@pytest.mark.parametrize("name", CASES)
def test_golden(name, cuda_device):
    c = load_case(name)
    g = c["gating_output"].to(cuda_device)
    w, ids = xkb.topk_softmax(g, c["topk"], c["renormalize"])
    _check(w, ids, c["topk_weights"], c["topk_ids"], c["gating_output"].dtype, name)
    w2, ids2 = xkb.topk_softmax(g, c["topk"], c["renormalize"])
    assert torch.equal(w, w2) and torch.equal(ids, ids2), "not deterministic"


@pytest.mark.parametrize("M,E,topk,dtype,renorm", [
    (4096, 256, 8, torch.bfloat16, True),      # the router shape of the benchmark configurations
    (333, 48, 8, torch.bfloat16, True),
    (1000, 1024, 16, torch.float32, False),    # the largest expert count
    (17, 33, 33, torch.float16, True),         # every expert selected
])
def test_against_oracle(M, E, topk, dtype, renorm, cuda_device):
    g = torch.Generator().manual_seed(M + E)
    logits = torch.randn(M, E, generator=g).to(dtype)
    want_w, want_ids = oracle.topk_softmax(logits, topk, renorm)
    w, ids = xkb.topk_softmax(logits.to(cuda_device), topk, renorm)
    _check(w, ids, want_w, want_ids, dtype, f"M={M} E={E}")
    if renorm:
        assert bool(((w.sum(1) - 1).abs() < 1e-5).all())


def test_feeds_the_fused_op(cuda_device):
    """Router output goes straight into the fused op: same result as with the oracle's routing."""
    from xkernels_b200 import synth

    cfg = synth.Int4Config("t", M=32, K=256, N=128, E=8, top_k=2)
    d = synth.make_int4(cfg, seed=5, device=cuda_device)
    logits = torch.randn(cfg.M, cfg.E, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    w, ids = xkb.topk_softmax(logits.to(cuda_device), cfg.top_k, True)
    ow, oids = oracle.topk_softmax(logits, cfg.top_k, True)
    out = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], ids, w)
    want = oracle.moe_w4a16(d["A"].cpu(), d["packed"].cpu(), d["scale"].cpu(), oids, ow, 32)
    assert oracle.count_violations(out.cpu(), want, 2e-2, 1e-2) == 0


def test_argument_errors(cuda_device):
    g = torch.zeros(2, 4, device=cuda_device)
    with pytest.raises(ValueError):
        xkb.topk_softmax(g, 5)
    with pytest.raises(ValueError):
        xkb.topk_softmax(g, 0)
    with pytest.raises(RuntimeError):
        xkb.topk_softmax(torch.zeros(2, 4), 2)      # CPU tensors are refused: there is no CPU path
    w, ids = xkb.topk_softmax(torch.zeros(0, 4, device=cuda_device), 2)
    assert w.shape == (0, 2) and ids.shape == (0, 2)
