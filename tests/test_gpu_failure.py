"""The abort path of the tcgen05 kernels, exercised without faulting or hanging the GPU: a small
self-test kernel of the library waits, with a 20 microsecond budget, on an mbarrier that nothing
arrives on.  The wait must run out, the status word must say so, tensor memory must be released
(the next fused call needs all of it) and the context must stay usable."""

import pytest
import torch

import xkernels_b200 as xkb
from oracle import moe_oracle as oracle
from tests.gpu_util import to_dev
from xkernels_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_leaves_the_gpu_usable(cuda_device):
    lib = _lib.load()
    dev = cuda_device
    cfg = synth.Int4Config("after_abort", M=16, K=512, N=256, E=8, top_k=2)
    c = synth.make_int4(cfg, seed=3)
    d = to_dev(c, dev)
    want = oracle.moe_w4a16(c["A"], c["packed"], c["scale"], c["topk_ids"], c["topk_w"], 32)
    # a normal call first: creates the per-device workspace and leaves status 0
    out = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], path="tc")
    ops.check_status(dev)
    assert oracle.count_violations(out.cpu(), want, 2e-2, 1e-2) == 0

    ws = ops.get_workspace(dev, 1 << 20)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(lib.xkb_selftest_bounded_wait(ws.data_ptr(), ws.numel(), stream), "xkb_selftest_bounded_wait")
    torch.cuda.synchronize(dev)                       # the kernel returned by itself
    with pytest.raises(_lib.XkbError, match=r"bounded wait.*wait site 99"):
        ops.check_status(dev)
    assert lib.xkb_workspace_status(ws.data_ptr(), stream) == -4          # XKB_ERR_DEVICE, still recorded

    # tensor memory was released and the context is intact: the same fused call passes again
    # (it clears the status word, allocates all 512 tensor-memory columns and gives the same bits)
    again = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], path="tc")
    ops.check_status(dev)
    assert torch.equal(out, again)
