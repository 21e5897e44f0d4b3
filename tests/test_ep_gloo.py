"""Expert-parallel dispatch/combine logic on CPU: world_size-2 (and 4) gloo ranks, the local expert
GEMM and per-row sum replaced by the oracle.  Checks the routing plan, the count exchange, both payload all-to-alls
and the final ordering against the dense single-rank oracle on each rank's own tokens."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as oracle
from xkernels_b200 import ep, synth

CFG = synth.Int4Config("ep_cpu", M=24, K=128, N=64, E=8, top_k=3, zipf_scale=2.0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_partial(packed, scale):
    """CPU stand-in for the local compute: per received row the weighted fp32 sum over its experts."""
    def partial_fn(rows_A, ids, w):
        R = rows_A.shape[0]
        out = torch.zeros(R, packed.shape[1], dtype=torch.float32)
        for j in range(ids.shape[1]):                      # ascending slot order, like the kernel path
            for e in torch.unique(ids[:, j]).tolist():
                if e < 0:
                    continue
                sel = (ids[:, j] == e).nonzero(as_tuple=True)[0]
                W = oracle.dequant_w4a16(packed[e], scale[e], 32, out_dtype=rows_A.dtype).float()
                out[sel] += w[sel, j:j + 1] * (rows_A[sel].float() @ W.T)
        return out
    return partial_fn


def _cpu_reduce(rows, row_index, M, dtype):
    out = torch.zeros(M, rows.shape[1], dtype=torch.float32)
    for k in range(row_index.shape[1]):
        idx = row_index[:, k].long()
        ok = idx >= 0
        out[ok] += rows[idx[ok]]
    return out.to(dtype)


def _worker(rank: int, world: int, port: int, fail_rank: int, placement: str = "contiguous", chunks: int = 1,
            n_replicas: int = 0, local_first: bool = True):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        packed, scale = synth.int4_weights(CFG.E, CFG.N, CFG.K, 32, seed=5)      # global experts (same on all ranks)
        e_local = CFG.E // world
        sl = torch.tensor(ep.local_expert_ids(rank, e_local, world, placement))
        A = synth.activations(CFG.M, CFG.K, seed=100 + rank)
        ids, w = synth.routing(CFG.M, CFG.E, CFG.top_k, seed=200 + rank, zipf_scale=CFG.zipf_scale)
        layer = ep.ExpertParallelInt4(packed[sl], scale[sl], num_global_experts=CFG.E, group_size=32,
                                      partial_fn=_oracle_partial(packed[sl], scale[sl]), reduce_fn=_cpu_reduce,
                                      placement=placement, chunks=chunks, local_first=local_first,
                                      max_recv_rows=0 if rank == fail_rank else None)
        assert layer.local_first == (local_first and chunks == 1)
        if fail_rank >= 0:
            # capacity check: EVERY rank raises the same refusal before any payload moves, so none
            # is left waiting in the dispatch all-to-all
            with pytest.raises(ep.ExchangeRefused, match=f"rank {fail_rank} would receive .* capacity 0"):
                layer(A, ids, w)
            # the group is still usable: the next call with the limit lifted goes through
            layer.max_recv_rows = None
            out = layer(A, ids, w)
            want = oracle.moe_w4a16(A, packed, scale, ids, w, 32)
            assert oracle.count_violations(out, want, 2e-2, 1e-2) == 0
            return
        sent_before = None
        if n_replicas:
            layer(A, ids, w)
            sent_before = sum(c for p, c in enumerate(layer.last_send_counts) if p != rank)
            hot = layer.rebalance(ids, n_replicas)
            # every rank picked the same experts and now holds them behind its own
            assert len(hot) == n_replicas and layer.packed.shape[0] == e_local + n_replicas
            for i, g in enumerate(hot):
                assert torch.equal(layer.packed[e_local + i], packed[g]) and torch.equal(layer.scale[e_local + i], scale[g])
            layer.partial_fn = _oracle_partial(layer.packed, layer.scale)
        out = layer(A, ids, w)
        want = oracle.moe_w4a16(A, packed, scale, ids, w, 32)
        assert oracle.count_violations(out, want, 2e-2, 1e-2) == 0, f"rank {rank} differs from the dense oracle"
        if n_replicas:
            # the popular experts' slots stay at home: fewer rows leave this rank than before
            sent_after = sum(c for p, c in enumerate(layer.last_send_counts) if p != rank)
            assert sent_after <= sent_before
            total = torch.tensor([layer.count_recv_slots(), sent_before - sent_after])
            dist.all_reduce(total)
            assert int(total[0]) == world * CFG.M * CFG.top_k and int(total[1]) > 0
            return
        # every token went once to each rank that owns one of its experts, every slot is computed
        # exactly once, and the receive counts add up over the ranks
        plan = ep.plan_dispatch(ids, e_local, world, placement, chunks)
        owners = ep.owner_and_local(ids.long(), e_local, world, placement)[0]
        n_pairs = sum(len(set(row.tolist())) for row in owners)
        assert n_pairs == plan.pair_token.numel() <= CFG.M * CFG.top_k
        # local-first: a token's slots on this rank's own experts never enter the exchange
        n_home = sum(1 for row in owners if rank in row.tolist()) if layer.local_first else 0
        assert sum(layer.last_send_counts) == n_pairs - n_home
        assert not layer.local_first or layer.last_send_counts[rank] == 0
        total = torch.tensor([layer.last_recv_rows, layer.count_recv_slots()])
        dist.all_reduce(total)
        pairs_all = torch.tensor([n_pairs - n_home])
        dist.all_reduce(pairs_all)
        assert int(total[0]) == int(pairs_all) and int(total[1]) == world * CFG.M * CFG.top_k
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,placement,chunks,local_first", [
    (2, "contiguous", 1, True), (4, "contiguous", 1, True), (2, "contiguous", 1, False),
    (2, "round_robin", 3, True), (4, "round_robin", 2, True), (4, "snake", 1, True), (4, "snake", 1, False)])
def test_all_to_all_matches_dense_oracle(world, placement, chunks, local_first):
    mp.spawn(_worker, args=(world, _free_port(), -1, placement, chunks, 0, local_first), nprocs=world, join=True)


@pytest.mark.parametrize("world,placement,chunks,n_replicas", [(2, "contiguous", 1, 2), (4, "round_robin", 2, 3),
                                                               (4, "snake", 1, 3)])
def test_replicated_popular_experts_keep_the_result_and_cut_the_traffic(world, placement, chunks, n_replicas):
    mp.spawn(_worker, args=(world, _free_port(), -1, placement, chunks, n_replicas), nprocs=world, join=True)


def test_expert_table_sends_replicated_experts_home():
    t = ep.expert_table(4, 2, "contiguous", rank=1, replicas=[5, 0])
    assert t.tolist() == [[1, 5], [0, 1], [0, 2], [0, 3], [1, 0], [1, 4], [1, 2], [1, 3]]
    ids = torch.tensor([[0, 5, 2]], dtype=torch.int32)
    plan = ep.plan_dispatch(ids, 4, 2, table=t)                     # as rank 1: experts 0 and 5 are served at home
    assert plan.send_counts.tolist() == [[1, 1]]
    assert plan.pair_dest.tolist() == [0, 1] and plan.pair_ids.tolist() == [[-1, -1, 2], [5, 4, -1]]


def test_plan_dispatch_makes_one_pair_per_token_and_owner():
    ids = torch.tensor([[5, 0, 3], [1, 7, 2]], dtype=torch.int32)
    # contiguous: experts 0-3 on rank 0, 4-7 on rank 1.  token 0 -> ranks {1, 0}, token 1 -> {0, 1}
    plan = ep.plan_dispatch(ids, experts_per_rank=4, world=2)
    assert plan.send_counts.tolist() == [[2, 2]]
    assert plan.pair_token.tolist() == [0, 1, 0, 1]            # grouped by destination, stable in the token
    assert plan.pair_dest.tolist() == [0, 0, 1, 1]
    assert plan.pair_ids.tolist() == [[-1, 0, 3], [1, -1, 2], [1, -1, -1], [-1, 3, -1]]
    assert plan.pair_of.tolist() == [[0, 2], [1, 3]]
    assert plan.n_slots == 6
    with pytest.raises(ValueError):
        ep.plan_dispatch(torch.tensor([[8]], dtype=torch.int32), 4, 2)
    # round robin: expert g on rank g % 2 as local expert g // 2; two token chunks of one token each
    plan = ep.plan_dispatch(ids, experts_per_rank=4, world=2, placement="round_robin", chunks=2)
    assert plan.send_counts.tolist() == [[1, 1], [1, 1]]
    assert plan.pair_token.tolist() == [0, 0, 1, 1]
    assert plan.pair_dest.tolist() == [0, 1, 0, 1]
    assert plan.pair_ids.tolist() == [[-1, 0, -1], [2, -1, 1], [-1, -1, 1], [0, 3, -1]]
    assert ep.local_expert_ids(1, 4, 2, "round_robin") == [1, 3, 5, 7]
    # snake: groups of W experts dealt forwards, backwards, forwards, ...
    assert ep.local_expert_ids(0, 4, 2, "snake") == [0, 3, 4, 7] and ep.local_expert_ids(1, 4, 2, "snake") == [1, 2, 5, 6]
    owner, local = ep.owner_and_local(torch.arange(8), 4, 2, "snake")
    assert owner.tolist() == [0, 1, 1, 0, 0, 1, 1, 0] and local.tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    # a token whose experts all live on one rank crosses the wire once
    plan = ep.plan_dispatch(torch.tensor([[0, 1, 2]], dtype=torch.int32), 4, 2)
    assert plan.send_counts.tolist() == [[1, 0]] and plan.pair_ids.tolist() == [[0, 1, 2]]


@pytest.mark.parametrize("world,fail_rank", [(2, 1), (4, 2)])
def test_receive_capacity_refusal_is_raised_by_every_rank(world, fail_rank):
    """Failure injected on the host: one rank's receive capacity is exceeded.  All ranks learn it
    from the gathered count matrix and raise together; nothing waits on anything."""
    mp.spawn(_worker, args=(world, _free_port(), fail_rank), nprocs=world, join=True)


def _bad_input_worker(rank: int, world: int, port: int, case: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        packed, scale = synth.int4_weights(CFG.E, CFG.N, CFG.K, 32, seed=5)
        e_local = CFG.E // world
        sl = torch.tensor(ep.local_expert_ids(rank, e_local, world, "contiguous"))
        layer = ep.ExpertParallelInt4(packed[sl], scale[sl], num_global_experts=CFG.E, group_size=32,
                                      partial_fn=_oracle_partial(packed[sl], scale[sl]), reduce_fn=_cpu_reduce)
        M = 0 if (case == "empty_rank" and rank == 1) else CFG.M
        A = synth.activations(M, CFG.K, seed=100 + rank)
        if M:
            ids, w = synth.routing(M, CFG.E, CFG.top_k, seed=200 + rank)
        else:
            ids, w = torch.zeros((0, CFG.top_k), dtype=torch.int32), torch.zeros((0, CFG.top_k))
        if case == "invalid_id":
            if rank == 1:
                ids = ids.clone()
                ids[3, 1] = CFG.E          # one bad id on one rank only
            with pytest.raises(ValueError, match=r"rank\(s\) \[1\]"):
                layer(A, ids, w)
        elif case == "negative_count":
            counts = ep.plan_dispatch(ids, e_local, world, "contiguous", 1, host_checks=False).send_counts.clone()
            if rank == 0:
                counts[0, 1] = -5          # a corrupted count matrix on one rank
            with pytest.raises(ep.ExchangeRefused, match="rank 0 reported a negative count"):
                ep.exchange_counts(counts, dist.group.WORLD)
        elif case == "too_many_pairs":
            counts = ep.plan_dispatch(ids, e_local, world, "contiguous", 1, host_checks=False).send_counts.clone()
            if rank == 1:
                counts[0, 0] += 1000       # more pairs than the rank has slots
            with pytest.raises(ep.ExchangeRefused, match="rank 1 reported"):
                ep.exchange_counts(counts, dist.group.WORLD, n_slots=M * CFG.top_k)
        else:                               # empty_rank: a rank without tokens still serves its experts
            out = layer(A, ids, w)
            assert out.shape == (M, CFG.N)
            if M:
                want = oracle.moe_w4a16(A, packed, scale, ids, w, 32)
                assert oracle.count_violations(out, want, 2e-2, 1e-2) == 0
            # what the ranks received is what the ranks sent
            t = torch.tensor([layer.last_recv_rows, sum(layer.last_send_counts)])
            dist.all_reduce(t)
            assert int(t[0]) == int(t[1])
        if case != "empty_rank":
            # the refusal was collective: the group still works afterwards
            ids_ok, w_ok = synth.routing(CFG.M, CFG.E, CFG.top_k, seed=300 + rank)
            A_ok = synth.activations(CFG.M, CFG.K, seed=400 + rank)
            out = layer(A_ok, ids_ok, w_ok)
            want = oracle.moe_w4a16(A_ok, packed, scale, ids_ok, w_ok, 32)
            assert oracle.count_violations(out, want, 2e-2, 1e-2) == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["invalid_id", "negative_count", "too_many_pairs", "empty_rank"])
def test_bad_inputs_on_one_rank_stop_every_rank(case):
    mp.spawn(_bad_input_worker, args=(2, _free_port(), case), nprocs=2, join=True)
