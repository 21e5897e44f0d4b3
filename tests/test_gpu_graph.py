"""The fused calls are stream-ordered end to end (align without a host read, no allocation inside the
library, status words instead of host-visible errors), so a whole call can be captured in a CUDA
graph and replayed on new inputs -- what the reference's workspace mode exists for
(src/xkernels/ops/moe/workspace.py, tests/test_moe_workspace.py:289-315 there)."""

import pytest
import torch

import xkernels_b200 as xkb
from xkernels_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _capture(fn, warmup=3):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warmup):          # workspaces grow and attributes are set outside the capture
            fn()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    return g, out


def test_int4_call_replays_on_new_inputs(cuda_device):
    cfg = synth.Int4Config("g", M=48, K=1024, N=512, E=8, top_k=4)
    a = synth.make_int4(cfg, seed=1, device=cuda_device)
    b = synth.make_int4(cfg, seed=2, device=cuda_device)
    A, ids, w = a["A"].clone(), a["topk_ids"].clone(), a["topk_w"].clone()
    g, out = _capture(lambda: xkb.fused_moe_int4_w4a16(A, a["packed"], a["scale"], ids, w))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, xkb.fused_moe_int4_w4a16(a["A"], a["packed"], a["scale"], a["topk_ids"], a["topk_w"]))
    # other tokens, other routing (other block counts), same graph
    A.copy_(b["A"]); ids.copy_(b["topk_ids"]); w.copy_(b["topk_w"])
    g.replay()
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
    assert torch.equal(out, xkb.fused_moe_int4_w4a16(b["A"], a["packed"], a["scale"], b["topk_ids"], b["topk_w"]))


def test_router_plus_mxfp4_call_replays(cuda_device):
    cfg = synth.Mxfp4Config("g", M=24, hidden=512, ispp=512, E=8, top_k=2, scale_lo=119, scale_hi=124)
    d = synth.make_mxfp4(cfg, seed=3, device=cuda_device)
    logits = torch.randn(cfg.M, cfg.E, device=cuda_device).to(torch.bfloat16)
    A = d["A"].clone()

    def call():
        w, ids = xkb.topk_softmax(logits, cfg.top_k, True)
        return xkb.fused_moe_mxfp4(A, d["w13"], d["w13_scale"], d["w2"], d["w2_scale"], ids, w)

    g, out = _capture(call)
    logits.copy_(torch.randn(cfg.M, cfg.E, device=cuda_device).to(torch.bfloat16))
    A.copy_(torch.randn_like(A))
    g.replay()
    torch.cuda.synchronize()
    ops.check_status(cuda_device)
    assert torch.equal(out, call())
