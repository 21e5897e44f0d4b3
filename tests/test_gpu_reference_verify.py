"""The acceptance gate of the plug-in: the reference's OWN, unmodified ``verify`` and
``verify_parity`` run on the GPU against the sm_100a cards of this repo (through the overlay
registry that ``plugin.install()`` activates).  Needs the reference package under ``baseline/_ref``
(baseline/install_reference.sh); skipped otherwise."""

import pytest

from tests.reference_util import reference_available

pytestmark = pytest.mark.gpu
HAVE_REF = reference_available(allow_source_tree=False)
needs_ref = pytest.mark.skipif(not HAVE_REF, reason="reference package not installed under baseline/_ref")


@pytest.fixture(scope="module")
def installed(tmp_path_factory):
    from xkernels_b200 import plugin

    return plugin.install(tmp_path_factory.mktemp("overlay"))


@needs_ref
@pytest.mark.parametrize("card", ["moe_align_block_size.cuda@1.0.0", "moe_int4_w4a16.cuda@1.0.0",
                                  "moe_sum_reduce.cuda@1.1.0", "moe_mxfp4.cuda@1.0.0",
                                  "topk_softmax.cuda@1.0.0"])
def test_reference_verify_passes(card, installed, cuda_device):
    from xkernels import verify

    res = verify(card, arch="nvidia_sm100")
    corr = res["correctness"]
    assert res["compiled"] is True, res
    assert corr["passed"] is True, corr
    assert res["determinism_check"] in (True, "passed") or res["determinism_check"].get("passed", True), res


@needs_ref
@pytest.mark.parametrize("op", ["moe_align_block_size@1.0.0", "moe_int4_w4a16@1.0.0", "moe_sum_reduce@1.0.0",
                                "moe_mxfp4@1.0.0", "topk_softmax@1.0.0"])
def test_reference_verify_parity_agrees(op, installed, cuda_device):
    from xkernels import verify_parity

    res = verify_parity(op, archs=["nvidia_sm100"])
    assert res["n_runnable"] >= 2, res
    assert res["agree"] is True, res


@needs_ref
def test_auto_dispatch_picks_the_cuda_backend(installed, cuda_device):
    """``backend="auto"`` on NVIDIA tries CUDA first (src/xkernels/_dispatch.py:37-41)."""
    import torch
    import xkernels

    from xkernels_b200 import _lib, synth

    d = synth.make_int4(synth.CONFIGS["int4_tiny"], seed=3, device=cuda_device)
    before = _lib.launch_count()
    out = xkernels.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], group_size=32)
    assert _lib.launch_count() > before, "auto dispatch did not reach libxkb200.so"
    ref = xkernels.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], group_size=32,
                                        backend="reference")
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=1e-2)
