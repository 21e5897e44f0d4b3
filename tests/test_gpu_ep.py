"""Expert-parallel mode on GPUs: the two local C-ABI building blocks on one GPU, and the full
NCCL all-to-all path as one child process per GPU when at least two GPUs are visible."""

import os
import socket

import pytest
import torch

import xkernels_b200 as xkb
from oracle import moe_oracle as oracle
from tests.gpu_util import assert_within
from xkernels_b200 import ops, synth

pytestmark = pytest.mark.gpu


def test_rows_and_gather_reduce_equal_the_fused_op(cuda_device):
    cfg = synth.Int4Config("t", M=40, K=512, N=256, E=8, top_k=4)
    d = synth.make_int4(cfg, seed=11, device=cuda_device)
    fused = xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])
    rows = ops.moe_int4_w4a16_rows(d["A"], d["packed"], d["scale"], d["topk_ids"])
    assert rows.shape == (cfg.M * cfg.top_k, cfg.N) and rows.dtype == torch.float32
    idx = torch.arange(cfg.M * cfg.top_k, device=cuda_device, dtype=torch.int32).view(cfg.M, cfg.top_k)
    out = ops.moe_gather_sum_reduce(rows, idx, d["topk_w"], torch.bfloat16)
    assert_within(out, fused, 1e-2, 1e-2, what="rows + gather_reduce vs fused")
    # a permuted row buffer with the matching index gives the same bits
    perm = torch.randperm(rows.shape[0], device=cuda_device)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=cuda_device)
    out2 = ops.moe_gather_sum_reduce(rows[perm].contiguous(), inv.view(cfg.M, cfg.top_k).int(), d["topk_w"],
                                     torch.bfloat16)
    assert torch.equal(out, out2)
    # one row per slot with top_k = 1 (the form the expert side of the exchange uses)
    cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    flat_ids = d["topk_ids"].reshape(-1, 1)
    A_rows = d["A"].repeat_interleave(cfg.top_k, dim=0)
    rows1 = ops.moe_int4_w4a16_rows(A_rows, d["packed"], d["scale"], flat_ids)
    want = oracle.moe_w4a16(cpu["A"].repeat_interleave(cfg.top_k, dim=0), cpu["packed"], cpu["scale"],
                            cpu["topk_ids"].reshape(-1, 1), torch.ones(cfg.M * cfg.top_k, 1), 32)
    assert_within(rows1.bfloat16(), want, 2e-2, 1e-2, what="top_k=1 rows")


def test_rows_with_absent_slots_and_per_row_sum(cuda_device):
    """The expert side of the exchange: a received row carries up to top_k local expert ids, -1 where
    the token's slot went to another rank.  Absent slots are dropped by the align stage, the
    weighted rows of the present ones are summed per received row in fp32."""
    cfg = synth.Int4Config("t", M=200, K=512, N=256, E=6, top_k=4)
    d = synth.make_int4(cfg, seed=21, device=cuda_device)
    g = torch.Generator().manual_seed(3)
    absent = (torch.rand(cfg.M, cfg.top_k, generator=g) < 0.45)
    absent[0] = True                                   # a row with no local expert at all
    ids = torch.where(absent.to(cuda_device), torch.full_like(d["topk_ids"], -1), d["topk_ids"])
    rows = ops.moe_int4_w4a16_rows(d["A"], d["packed"], d["scale"], ids, d["topk_w"])
    ops.check_status(cuda_device)
    slot = torch.arange(cfg.M * cfg.top_k, dtype=torch.int32, device=cuda_device).view(cfg.M, cfg.top_k)
    partial = ops.moe_gather_sum_reduce(rows, torch.where(ids >= 0, slot, torch.full_like(slot, -1)), None,
                                        torch.float32)
    assert partial.dtype == torch.float32 and bool((partial[0] == 0).all())
    # oracle: the replicated expert-parallel form with a map that sends absent slots to -1
    cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    ids_cpu = torch.where(absent, torch.full_like(cpu["topk_ids"], cfg.E), cpu["topk_ids"])   # id E = "elsewhere"
    emap = torch.cat([torch.arange(cfg.E, dtype=torch.int32), torch.tensor([-1], dtype=torch.int32)])
    want = oracle.moe_w4a16(cpu["A"], cpu["packed"], cpu["scale"], ids_cpu, cpu["topk_w"], 32, expert_map=emap)
    assert_within(partial.bfloat16(), want, 2e-2, 1e-2, what="partial rows")


@pytest.mark.parametrize("M,E,top_k,world,placement,chunks", [
    (96, 16, 4, 2, "contiguous", 1), (96, 16, 4, 4, "round_robin", 3), (4096, 256, 8, 8, "round_robin", 1),
    (1, 8, 8, 8, "contiguous", 1), (333, 48, 6, 4, "contiguous", 2), (0, 8, 2, 2, "contiguous", 1),
    (500, 64, 8, 8, "snake", 1), (96, 16, 4, 2, "snake", 2),
])
def test_device_plan_equals_host_plan(M, E, top_k, world, placement, chunks, cuda_device):
    """xkb_ep_plan (three launches, no host read) against ep.plan_dispatch (torch ops on the CPU)."""
    from xkernels_b200 import ep

    ids, w = synth.routing(M, E, top_k, seed=M + world, zipf_scale=2.0) if M else (
        torch.zeros((0, top_k), dtype=torch.int32), torch.zeros((0, top_k)))
    want = ep.plan_dispatch(ids, E // world, world, placement, chunks)
    pt, pd, routing, pair_of, counts, info = ops.ep_plan(ids.to(cuda_device), w.to(cuda_device), E // world, world,
                                                          placement, chunks)
    P = want.pair_token.numel()
    assert info.tolist() == [P, 0]
    assert counts.cpu().tolist() == want.send_counts.tolist()
    assert torch.equal(pt[:P].cpu().long(), want.pair_token) and torch.equal(pd[:P].cpu().long(), want.pair_dest)
    assert torch.equal(routing[:P, :top_k].cpu(), want.pair_ids)
    want_w = torch.where(want.pair_ids >= 0, w.float()[want.pair_token], torch.zeros(()))
    assert torch.equal(routing[:P, top_k:].cpu().view(torch.float32), want_w)
    assert torch.equal(pair_of.cpu(), want.pair_of)
    # invalid ids are counted, not acted on
    if M:
        bad = ids.clone()
        bad[0, 0] = E
        bad[-1, -1] = -3
        info2 = ops.ep_plan(bad.to(cuda_device), w.to(cuda_device), E // world, world, placement, chunks)[5]
        assert int(info2[1]) == 2


def test_device_plan_with_replicas_equals_host_plan(cuda_device):
    """The explicit expert table (popular experts served on the token's own rank) through xkb_ep_plan
    against ep.plan_dispatch."""
    from xkernels_b200 import ep

    M, E, top_k, world = 300, 32, 6, 4
    ids, w = synth.routing(M, E, top_k, seed=9, zipf_scale=2.0)
    table = ep.expert_table(E // world, world, "round_robin", rank=2, replicas=[0, 1, 7])
    want = ep.plan_dispatch(ids, E // world, world, "round_robin", 2, table=table)
    pt, pd, routing, pair_of, counts, info = ops.ep_plan(ids.to(cuda_device), w.to(cuda_device), E // world, world,
                                                          "round_robin", 2, table=table.to(cuda_device))
    P = want.pair_token.numel()
    assert info.tolist() == [P, 0] and counts.cpu().tolist() == want.send_counts.tolist()
    assert torch.equal(pt[:P].cpu().long(), want.pair_token) and torch.equal(pd[:P].cpu().long(), want.pair_dest)
    assert torch.equal(routing[:P, :top_k].cpu(), want.pair_ids) and torch.equal(pair_of.cpu(), want.pair_of)
    assert int(want.pair_ids.max()) >= E // world          # replica slots use the indices behind the own experts


def test_device_plan_leaves_home_experts_out(cuda_device):
    """Local-first mode: experts the rank serves itself carry destination -1 in the table and open no
    pair, in xkb_ep_plan as in ep.plan_dispatch."""
    from xkernels_b200 import ep

    M, E, top_k, world, rank = 257, 32, 6, 4, 1
    ids, w = synth.routing(M, E, top_k, seed=11, zipf_scale=2.0)
    table = ep.expert_table(E // world, world, "snake", rank=rank, replicas=[3, 8], home_is_not_dispatched=True)
    assert int((table[:, 0] < 0).sum()) == E // world + 2
    want = ep.plan_dispatch(ids, E // world, world, "snake", 1, table=table)
    pt, pd, routing, pair_of, counts, info = ops.ep_plan(ids.to(cuda_device), w.to(cuda_device), E // world, world,
                                                          "snake", 1, table=table.to(cuda_device))
    P = want.pair_token.numel()
    assert info.tolist() == [P, 0] and counts.cpu().tolist() == want.send_counts.tolist()
    assert counts.cpu()[0, rank] == 0 and bool((pair_of.cpu()[:, rank] == -1).all())
    assert torch.equal(pt[:P].cpu().long(), want.pair_token) and torch.equal(pd[:P].cpu().long(), want.pair_dest)
    assert torch.equal(routing[:P, :top_k].cpu(), want.pair_ids) and torch.equal(pair_of.cpu(), want.pair_of)


def test_gather_rows_with_the_count_on_the_device(cuda_device):
    g = torch.Generator().manual_seed(2)
    src = torch.randn(50, 64, generator=g).to(torch.bfloat16).to(cuda_device)
    idx = torch.randint(0, 50, (40,), generator=g, dtype=torch.int32).to(cuda_device)
    n = torch.tensor([25], dtype=torch.int32, device=cuda_device)
    out = torch.full((40, 64), -7.0, dtype=torch.bfloat16, device=cuda_device)
    ops.gather_rows(src, idx, n, out=out)
    assert torch.equal(out[:25], src[idx[:25].long()]) and bool((out[25:] == -7.0).all())
    assert torch.equal(ops.gather_rows(src, idx), src[idx.long()])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank: int, world: int, port: int, placement: str, chunks: int, n_replicas: int = 0,
               local_first: bool = False):
    import torch.distributed as dist

    from xkernels_b200 import ep

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        cfg = synth.Int4Config("ep", M=96, K=512, N=256, E=16, top_k=4, zipf_scale=2.0)
        packed, scale = synth.int4_weights(cfg.E, cfg.N, cfg.K, 32, seed=5)      # global, CPU, same on all ranks
        e_local = cfg.E // world
        sl = torch.tensor(ep.local_expert_ids(rank, e_local, world, placement))
        A = synth.activations(cfg.M, cfg.K, seed=100 + rank)
        ids, w = synth.routing(cfg.M, cfg.E, cfg.top_k, seed=200 + rank, zipf_scale=cfg.zipf_scale)
        layer = ep.ExpertParallelInt4(packed[sl].to(dev), scale[sl].to(dev), num_global_experts=cfg.E,
                                      placement=placement, chunks=chunks, local_first=local_first)
        if n_replicas:
            hot = layer.rebalance(ids.to(dev), n_replicas)
            assert len(hot) == n_replicas and layer.packed.shape[0] == e_local + n_replicas
        assert layer.local_first == (local_first and chunks == 1)
        out = layer(A.to(dev), ids.to(dev), w.to(dev))
        ops.check_status(dev)
        ops.check_status(dev, tag=2)          # the workspace of the local pass
        want = oracle.moe_w4a16(A, packed, scale, ids, w, 32)
        bad = oracle.count_violations(out.cpu(), want, 2e-2, 1e-2)
        assert bad == 0, f"rank {rank}: {bad} elements differ from the dense oracle"
        again = layer(A.to(dev), ids.to(dev), w.to(dev))
        assert torch.equal(out, again)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("placement,chunks,n_replicas,local_first", [
    ("contiguous", 1, 0, False), ("round_robin", 3, 0, False), ("snake", 1, 0, True), ("round_robin", 1, 3, False),
    ("round_robin", 1, 3, True)])
def test_all_to_all_on_gpus(placement, chunks, n_replicas, local_first):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    world = 4 if n >= 4 else 2
    mp.spawn(_ep_worker, args=(world, _free_port(), placement, chunks, n_replicas, local_first), nprocs=world, join=True)
