"""The reference's workspace contract (src/xkernels/ops/moe/workspace.py:85-289, pinned by its
tests/test_moe_workspace.py:70-138,192-213,289-315) against the sm_100a ops: an object passed as
``workspace=`` must be honoured (outputs / scratch at stable addresses, results unchanged, smaller
batches served from a larger object, a mismatching object ignored), and a whole fused call with a
workspace must replay from a CUDA graph.  The objects here are stand-ins with the reference's field
names and ``matches`` rule; when the reference package is installed under baseline/_ref the same
checks also run with its own classes."""

from dataclasses import dataclass

import pytest
import torch

import xkernels_b200 as xkb
from tests.reference_util import reference_available
from xkernels_b200 import ops, synth

pytestmark = pytest.mark.gpu


@dataclass
class AlignWs:
    sorted_ids: torch.Tensor
    expert_ids: torch.Tensor
    num_post: torch.Tensor
    tokens_cnts: torch.Tensor
    cumsum: torch.Tensor

    @classmethod
    def allocate(cls, M, top_k, E, block, *, device):
        max_pad = M * top_k + (E + 1) * (block - 1)
        i32 = dict(dtype=torch.int32, device=device)
        return cls(torch.empty(max_pad, **i32), torch.empty(-(-max_pad // block), **i32), torch.empty(1, **i32),
                   torch.empty((E + 1, E), **i32), torch.empty(E + 1, **i32))

    def matches(self, M, top_k, E, block, *, device):
        max_pad = M * top_k + (E + 1) * (block - 1)
        return (self.sorted_ids.numel() >= max_pad and self.expert_ids.numel() >= -(-max_pad // block)
                and tuple(self.tokens_cnts.shape) == (E + 1, E) and self.sorted_ids.device == torch.device(device))


@dataclass
class Int4Ws:
    combine_out: torch.Tensor
    scratch: torch.Tensor
    dtype: torch.dtype
    align_workspace: object = None

    @classmethod
    def allocate(cls, max_M, top_k, N, *, dtype, device):
        return cls(torch.empty((max_M, N), dtype=torch.float32, device=device),
                   torch.empty((max_M * top_k, N), dtype=dtype, device=device), dtype)

    def matches(self, M, top_k, N, *, dtype, device):
        return (self.combine_out.shape[1] == N and self.combine_out.shape[0] >= M and self.scratch.shape[0] >= M * top_k
                and self.scratch.dtype == dtype and self.combine_out.device == torch.device(device))


def workspace_classes():
    out = [(AlignWs, Int4Ws)]
    if reference_available(allow_source_tree=False):
        from xkernels.ops.moe.workspace import MoeAlignWorkspace, MoeInt4Workspace
        out.append((MoeAlignWorkspace, MoeInt4Workspace))
    return out


@pytest.mark.parametrize("classes", workspace_classes(), ids=lambda c: c[0].__name__)
def test_align_writes_into_a_matching_workspace_at_stable_addresses(classes, cuda_device):
    Align, _ = classes
    E, block = 8, 64
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, E, (8, 4), generator=g, dtype=torch.int32).to(cuda_device)
    s_a, e_a, n_a = xkb.moe_align_block_size(ids, block, E, truncate=False)
    ws = Align.allocate(8, 4, E, block, device=cuda_device)
    s_w, e_w, n_w = xkb.moe_align_block_size(ids, block, E, truncate=False, workspace=ws)
    assert torch.equal(s_w, s_a) and torch.equal(e_w, e_a) and torch.equal(n_w, n_a)
    assert torch.equal(s_w, ws.sorted_ids) and torch.equal(e_w, ws.expert_ids)     # written into the object's buffers
    s2, _, n2 = xkb.moe_align_block_size(ids, block, E, truncate=False, workspace=ws)
    assert s2.data_ptr() == s_w.data_ptr() == ws.sorted_ids.data_ptr() and n2.data_ptr() == ws.num_post.data_ptr()
    # a third call equals the first: nothing accumulates in the object between calls
    other = torch.randint(0, E, (8, 4), generator=g, dtype=torch.int32).to(cuda_device)
    xkb.moe_align_block_size(other, block, E, truncate=False, workspace=ws)
    s3, e3, n3 = xkb.moe_align_block_size(ids, block, E, truncate=False, workspace=ws)
    assert torch.equal(s3, s_a) and torch.equal(e3, e_a) and torch.equal(n3, n_a)
    # a larger object serves a smaller batch and returns the batch-shaped slices
    ids4 = ids[:4].contiguous()
    big = Align.allocate(16, 4, E, block, device=cuda_device)
    want = xkb.moe_align_block_size(ids4, block, E, truncate=False)
    got = xkb.moe_align_block_size(ids4, block, E, truncate=False, workspace=big)
    assert all(torch.equal(a, b) for a, b in zip(got, want)) and got[0].shape == want[0].shape
    # an object built for another problem is ignored
    wrong = Align.allocate(8, 4, E + 1, block, device=cuda_device)
    got = xkb.moe_align_block_size(ids, block, E, truncate=False, workspace=wrong)
    assert torch.equal(got[0], s_a) and got[0].data_ptr() != wrong.sorted_ids.data_ptr()


@pytest.mark.parametrize("classes", workspace_classes(), ids=lambda c: c[1].__name__)
def test_fused_int4_runs_in_the_callers_workspace(classes, cuda_device):
    _, Int4 = classes
    cfg = synth.Int4Config("ws", M=32, K=512, N=256, E=8, top_k=4)
    d = synth.make_int4(cfg, seed=5, device=cuda_device)
    args = (d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    want = xkb.fused_moe_int4_w4a16(*args)
    ws = Int4.allocate(64, cfg.top_k, cfg.N, dtype=torch.bfloat16, device=cuda_device)       # capacity 64 rows
    got = xkb.fused_moe_int4_w4a16(*args, workspace=ws)
    ops.check_workspace_status(ws)
    assert torch.equal(got, want)
    scratch = ws._xkb200_scratch
    assert scratch.numel() >= 64 * cfg.top_k * cfg.N * 4          # sized for the object's capacity, created once
    half = tuple(t[:16].contiguous() if t.shape[0] == cfg.M else t for t in args)
    got16 = xkb.fused_moe_int4_w4a16(*half, workspace=ws)
    assert ws._xkb200_scratch.data_ptr() == scratch.data_ptr() and torch.equal(got16, want[:16])
    # a batch beyond the object's capacity: matches() refuses, the call still gives the right answer
    big = synth.make_int4(synth.Int4Config("ws", M=96, K=512, N=256, E=8, top_k=4), seed=5, device=cuda_device)
    out = xkb.fused_moe_int4_w4a16(big["A"], big["packed"], big["scale"], big["topk_ids"], big["topk_w"], workspace=ws)
    assert ws._xkb200_scratch.data_ptr() == scratch.data_ptr()
    assert torch.equal(out, xkb.fused_moe_int4_w4a16(big["A"], big["packed"], big["scale"], big["topk_ids"], big["topk_w"]))


def test_fused_ops_take_a_plain_tensor_as_workspace(cuda_device):
    cfg = synth.Int4Config("ws", M=32, K=512, N=256, E=8, top_k=4)
    d = synth.make_int4(cfg, seed=6, device=cuda_device)
    args = (d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    want = xkb.fused_moe_int4_w4a16(*args)
    buf = torch.empty(64 << 20, dtype=torch.uint8, device=cuda_device)
    assert torch.equal(xkb.fused_moe_int4_w4a16(*args, workspace=buf), want)
    ops.check_workspace_status(buf)
    with pytest.raises(ValueError, match="bytes"):
        xkb.fused_moe_int4_w4a16(*args, workspace=buf[:1024])
    m = synth.make_mxfp4(synth.Mxfp4Config("ws", M=16, hidden=512, ispp=512, E=4, top_k=2, scale_lo=119, scale_hi=124),
                         seed=3, device=cuda_device)
    margs = (m["A"], m["w13"], m["w13_scale"], m["w2"], m["w2_scale"], m["topk_ids"], m["topk_w"])
    assert torch.equal(xkb.fused_moe_mxfp4(*margs, workspace=buf), xkb.fused_moe_mxfp4(*margs))


def test_fused_call_with_a_workspace_replays_from_a_cuda_graph(cuda_device):
    """tests/test_moe_workspace.py:289-315 of the reference: capture the whole call with a workspace,
    replay it on new inputs written into the same tensors."""
    cfg = synth.Int4Config("ws", M=16, K=512, N=256, E=8, top_k=2)
    d = synth.make_int4(cfg, seed=7, device=cuda_device)
    ws = Int4Ws.allocate(cfg.M, cfg.top_k, cfg.N, dtype=torch.bfloat16, device=cuda_device)
    A, ids, w = d["A"].clone(), d["topk_ids"].clone(), d["topk_w"].clone()
    fn = lambda: xkb.fused_moe_int4_w4a16(A, d["packed"], d["scale"], ids, w, workspace=ws)   # noqa: E731
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fn()
    d2 = synth.make_int4(cfg, seed=8, device=cuda_device)
    A.copy_(d2["A"]); ids.copy_(d2["topk_ids"]); w.copy_(d2["topk_w"])
    graph.replay()
    torch.cuda.synchronize()
    want = xkb.fused_moe_int4_w4a16(d2["A"], d["packed"], d["scale"], d2["topk_ids"], d2["topk_w"])
    assert torch.equal(out, want)
