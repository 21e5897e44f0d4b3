"""moe_align_block_size on the GPU vs the oracle and the reference-made fixtures: bit-exact
on the whole triple including the unused tails (spec: rtol = atol = 0)."""

import numpy as np
import pytest
import torch

import xkernels_b200 as xkb
from oracle import moe_oracle as oracle
from tests.golden.golden_io import load_case

pytestmark = pytest.mark.gpu

GOLDEN = ["align_kat", "align_sweep0", "align_sweep1", "align_sweep2", "align_sweep3", "align_sweep5",
          "align_skew_trunc0", "align_skew_trunc1"]


def run(ids, block, E, truncate, dev, expert_map=None):
    s, e, n = xkb.moe_align_block_size(ids.to(dev), block, E, truncate=truncate,
                                       expert_map=None if expert_map is None else expert_map.to(dev))
    assert s.dtype == e.dtype == n.dtype == torch.int32
    return s.cpu().numpy(), e.cpu().numpy(), n.cpu().numpy()


def check(ids, block, E, truncate, dev):
    got = run(ids, block, E, truncate, dev)
    want = oracle.align_block_size(ids.numpy(), block, E, truncate)
    for g, w, name in zip(got, want, ("sorted_token_ids", "expert_ids", "num_tokens_post_padded")):
        assert g.shape == w.shape, f"{name}: shape {g.shape} vs {w.shape}"
        assert np.array_equal(g, w), f"{name} differs (first at {np.flatnonzero(g != w)[:5]})"


@pytest.mark.parametrize("name", GOLDEN)
def test_golden(name, cuda_device):
    c = load_case(name)
    s, e, n = run(c["topk_ids"], c["block_size"], c["num_experts"], bool(c["truncate"]), cuda_device)
    assert np.array_equal(s, c["sorted_ids"].numpy())
    assert np.array_equal(e, c["expert_ids"].numpy())
    assert np.array_equal(n, c["num_post"].numpy())


@pytest.mark.parametrize("name", ["align_ep_rank0", "align_ep_rank1"])
def test_golden_expert_parallel(name, cuda_device):
    c = load_case(name)
    e_local = int((c["expert_map"] >= 0).sum())
    s, e, n = run(c["topk_ids"], c["block_size"], e_local, True, cuda_device, expert_map=c["expert_map"])
    assert np.array_equal(s, c["sorted_ids"].numpy())
    assert np.array_equal(e, c["expert_ids"].numpy())
    assert np.array_equal(n, c["num_post"].numpy())


@pytest.mark.parametrize("M,top_k,E,block,truncate", [
    (64, 8, 48, 16, True), (64, 8, 48, 16, False), (1, 8, 48, 16, True), (37, 4, 8, 16, True),
    (16, 1, 4, 8, False), (1, 1, 1, 1, True), (1000, 2, 3, 128, False), (1023, 1, 256, 16, True),
    (1025, 8, 257, 64, False), (2048, 4, 1024, 4, True), (48, 6, 256, 16, False),
    (16384, 8, 48, 16, True), (16384, 8, 48, 128, False), (4096, 8, 32, 256, False),
    (8192, 1, 7, 16, True), (8193, 1, 7, 16, True), (40000, 3, 100, 32, False),
])
def test_random_routings(M, top_k, E, block, truncate, cuda_device):
    g = torch.Generator().manual_seed(M * 31 + E)
    ids = torch.randint(0, E, (M, top_k), generator=g, dtype=torch.int32)
    check(ids, block, E, truncate, cuda_device)


def test_skewed_and_empty_experts(cuda_device):
    g = torch.Generator().manual_seed(5)
    # 70 % of the slots on expert 3, experts 10..19 empty
    ids = torch.randint(0, 10, (5000, 8), generator=g, dtype=torch.int32)
    hot = torch.rand(5000, 8, generator=g) < 0.7
    ids[hot] = 3
    for block in (16, 64):
        check(ids, block, 20, True, cuda_device)
        check(ids, block, 20, False, cuda_device)
    # every slot on the last expert
    check(torch.full((3000, 4), 47, dtype=torch.int32), 16, 48, True, cuda_device)


def test_empty_dispatch(cuda_device):
    check(torch.zeros((0, 8), dtype=torch.int32), 16, 48, True, cuda_device)
    check(torch.zeros((0, 8), dtype=torch.int32), 16, 48, False, cuda_device)


def test_invariants_at_prefill_size(cuda_device):
    """M=16384, top_k=8, E=48 with load skew: every slot appears once, blocks are pure,
    runs are stable, totals are multiples of the block (the reference's property tests,
    tests/test_moe_align_block_size.py:39-71)."""
    from xkernels_b200 import synth

    cfg = synth.CONFIGS["int4_prefill"]
    ids, _ = synth.routing(cfg.M, cfg.E, cfg.top_k, seed=3, expert_bias_std=cfg.expert_bias_std)
    B = 16
    s, e, n = run(ids, B, cfg.E, False, cuda_device)
    T = ids.numel()
    n = int(n[0])
    assert n % B == 0
    valid = s[:n][s[:n] < T]
    assert np.array_equal(np.sort(valid), np.arange(T))
    assert (s[n:] == T).all()
    flat = ids.numpy().reshape(-1)
    for b in range(n // B):
        blk = s[b * B:(b + 1) * B]
        real = blk[blk < T]
        assert (flat[real] == e[b]).all()
        assert (np.diff(real) > 0).all()
    assert (e[n // B:] == 0).all()
    check(ids, B, cfg.E, True, cuda_device)
