"""Expert-parallel INT4 fused MoE with all-to-all dispatch and combine.

One process per GPU; every rank owns ``E/W`` experts and its own batch of tokens.  A call does

  1. plan: one (token, destination rank) PAIR for every rank that owns at least one of the token's
     top-k experts, grouped by (token chunk, destination), stable inside a group.  A token whose
     experts share a rank crosses the wire once, not once per expert;
  2. all-gather the pair-count matrices (one small collective, one host read); every rank checks
     the whole matrix, so a refusal (invalid expert id, receive capacity exceeded, inconsistent
     counts) is raised by all ranks together before any payload moves;
  3. per chunk: dispatch all-to-all of the pairs' activation rows and of their routing (local expert
     ids padded with -1, routing weights), local grouped GEMM over the received rows and a weighted
     fp32 sum over each pair's experts, all-to-all of ONE fp32 partial row per pair back to the
     token owners;
  4. fixed-order sum of each token's partial rows (ascending rank) on the owner.

With ``chunks > 1`` the exchanges of chunk c+1 are in flight on NCCL's stream while the GEMM of
chunk c runs, so transfer and tensor work overlap.

The reference has no all-to-all (its expert parallelism replicates tokens and lets the caller
all-reduce partials, src/xkernels/ops/moe/interface.py:37-57); what it fixes is the result: the
dense op on each rank's tokens with the global expert set.  fp32 rows travel back so that the
sums see the same operands as the single-GPU op (a bf16 round per partial fails the op tolerance
on some elements, see meta/docs/wiki/04-gotchas.md:452-454 in the reference); only the order of
the fp32 additions differs (experts of one rank first).

Expert placement: ``"contiguous"`` (rank r owns experts ``[r*E/W, (r+1)*E/W)``, the layout of the
reference's ``expert_map`` tests, tests/test_moe_int4_ep.py:84-93) or ``"round_robin"`` (expert g
lives on rank ``g % W`` as local expert ``g // W``), which spreads a popularity-ranked expert set
evenly over the ranks, or ``"snake"`` (like round robin, but every second group of W experts is
dealt in reverse rank order, so that no rank collects the most popular expert of every group).

Replicas: :meth:`ExpertParallelInt4.rebalance` counts the expert popularity over all ranks, copies the
weights of the ``n`` most popular experts to every rank (they are static model state: one broadcast
each) and routes a slot of such an expert to the token's OWN rank.  That takes the hot experts'
slots off the wire and off their owner's GEMM, which is what bounds the step when a router is
skewed (one expert can bring a third of a rank's work).  The result is unchanged: a replica holds
the same bits as the original.

The exchange uses ``torch.distributed`` (NCCL on GPUs, gloo on CPU); data lands in local buffers
before any kernel reads it.  The local compute is pluggable so the routing logic runs on CPU ranks
in tests.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def owner_and_local(expert: torch.Tensor, experts_per_rank: int, world: int, placement: str):
    """Rank that owns each global expert id and the expert's index on that rank."""
    if placement == "contiguous":
        owner = torch.div(expert, experts_per_rank, rounding_mode="floor")
        return owner, expert - owner * experts_per_rank
    if placement == "round_robin":
        return expert % world, torch.div(expert, world, rounding_mode="floor")
    if placement == "snake":
        group = torch.div(expert, world, rounding_mode="floor")
        pos = expert % world
        return torch.where(group % 2 == 0, pos, world - 1 - pos), group
    raise ValueError(f"unknown expert placement {placement!r}")


def local_expert_ids(rank: int, experts_per_rank: int, world: int, placement: str) -> list[int]:
    """Global ids of the experts rank ``rank`` holds, in local-index order."""
    if placement == "contiguous":
        return list(range(rank * experts_per_rank, (rank + 1) * experts_per_rank))
    if placement == "round_robin":
        return [rank + world * i for i in range(experts_per_rank)]
    if placement == "snake":
        return [world * i + (rank if i % 2 == 0 else world - 1 - rank) for i in range(experts_per_rank)]
    raise ValueError(f"unknown expert placement {placement!r}")


@dataclass
class DispatchPlan:
    """Pairs in (chunk, destination) order, stable in the token.  Built without a host read: the
    arrays have one entry per SLOT (``M * top_k``), the first ``n_pairs`` of them are the pairs;
    ``n_pairs`` is None until :meth:`trim` (or the count exchange) has read it."""
    pair_token: torch.Tensor    # [P] int64 source token row of each pair
    pair_dest: torch.Tensor     # [P] int64 destination rank of each pair
    send_counts: torch.Tensor   # [chunks, W] int64 pairs per (chunk, destination)
    pair_ids: torch.Tensor      # [P, top_k] int32 expert index on the destination rank, -1 where the slot goes elsewhere
    pair_of: torch.Tensor       # [M, W] int32 position of pair (token, rank) in the sorted order, -1 if none
    n_slots: int                # M * top_k
    n_bad: torch.Tensor         # 0-d int64: expert ids outside [0, E)
    n_pairs: int | None = None

    def trim(self, n_pairs: int | None = None) -> "DispatchPlan":
        """Cut the per-slot arrays down to the pairs (``n_pairs`` from the host if already known)."""
        P = int(self.send_counts.sum()) if n_pairs is None else int(n_pairs)
        self.pair_token, self.pair_dest, self.pair_ids = self.pair_token[:P], self.pair_dest[:P], self.pair_ids[:P]
        self.n_pairs = P
        return self


def expert_table(experts_per_rank: int, world: int, placement: str, rank: int | None = None,
                 replicas: list[int] | tuple[int, ...] = (), home_is_not_dispatched: bool = False) -> torch.Tensor:
    """``[E, 2]`` int32: (destination rank, expert index there) of every global expert as rank ``rank``
    sees it.  Experts in ``replicas`` (global ids, in replica order) are held by every rank behind its
    own ``experts_per_rank`` experts, so their destination is ``rank`` itself.  With
    ``home_is_not_dispatched`` the experts served by ``rank`` itself get destination -1: the plan then
    opens no pair for them (the layer computes them where the token is, beside the exchange)."""
    E = experts_per_rank * world
    owner, local = owner_and_local(torch.arange(E, dtype=torch.int64), experts_per_rank, world, placement)
    table = torch.stack([owner, local], dim=1).to(torch.int32)
    if replicas:
        if rank is None:
            raise ValueError("expert_table: replicas need the rank that looks them up")
        for i, g in enumerate(replicas):
            table[int(g), 0] = rank
            table[int(g), 1] = experts_per_rank + i
    if home_is_not_dispatched:
        if rank is None:
            raise ValueError("expert_table: home_is_not_dispatched needs the rank")
        table[table[:, 0] == rank, 0] = -1
    return table


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int, placement: str = "contiguous",
                  chunks: int = 1, *, host_checks: bool = True, table: torch.Tensor | None = None) -> DispatchPlan:
    """One pair per (token, rank that owns at least one of its experts), grouped by (chunk, rank).

    With ``host_checks`` (the default) invalid expert ids raise here and the plan comes back
    trimmed, at the price of two host reads; the layer passes False and does both with the one
    read of its count exchange."""
    M, top_k = topk_ids.shape
    dev = topk_ids.device
    E = experts_per_rank * world
    ids = topk_ids.to(torch.int64)
    bad = (ids < 0) | (ids >= E)
    n_bad = bad.sum()
    if host_checks and ids.numel() and int(n_bad) != 0:
        raise ValueError("expert id outside [0, num_global_experts)")
    if table is None:
        dest, local = owner_and_local(ids.clamp(0, max(E - 1, 0)), experts_per_rank, world, placement)   # [M, top_k] each
    else:
        t = table.to(device=dev, dtype=torch.int64)[ids.clamp(0, max(E - 1, 0))]                         # [M, top_k, 2]
        dest, local = t[..., 0], t[..., 1]
    # a slot opens a pair if no earlier slot of its token goes to the same rank
    same = dest.unsqueeze(2) == dest.unsqueeze(1)                                   # [M, j, i]
    earlier = torch.ones(top_k, top_k, dtype=torch.bool, device=dev).tril(-1)       # i < j
    first = ~(same & earlier).any(dim=2) & (dest >= 0)      # a negative destination (table) is not dispatched
    tokens_per_chunk = -(-M // chunks) if M else 1
    chunk = torch.div(torch.arange(M, device=dev), tokens_per_chunk, rounding_mode="floor").unsqueeze(1)
    sentinel = chunks * world                                                        # sorts behind every pair
    key = torch.where(first, chunk * world + dest, torch.full_like(dest, sentinel)).reshape(-1)
    slot = torch.argsort(key, stable=True)             # pairs first, grouped by key, ascending token inside a key
    counts = torch.bincount(key, minlength=sentinel + 1)[:sentinel].view(chunks, world)
    pair_token = torch.div(slot, top_k, rounding_mode="floor")
    pair_dest = dest.reshape(-1)[slot].clamp(min=0)
    is_pair = key[slot] < sentinel
    mine = dest[pair_token] == pair_dest.unsqueeze(1)                               # [numel, top_k]
    pair_ids = torch.where(mine, local[pair_token], torch.full_like(local[pair_token], -1)).to(torch.int32)
    # pair_of[token, rank] = position; non-pairs write to a spare element behind the table
    flat = torch.full((M * world + 1,), -1, dtype=torch.int32, device=dev)
    where = torch.where(is_pair, pair_token * world + pair_dest, torch.full_like(pair_token, M * world))
    flat.scatter_(0, where, torch.arange(slot.numel(), dtype=torch.int32, device=dev))
    pair_of = flat[:M * world].view(M, world)
    plan = DispatchPlan(pair_token=pair_token, pair_dest=pair_dest, send_counts=counts, pair_ids=pair_ids,
                        pair_of=pair_of, n_slots=M * top_k, n_bad=n_bad)
    return plan.trim() if host_checks else plan


class ExchangeRefused(RuntimeError):
    """The count exchange found a reason not to move any payload.  Raised by EVERY rank of the
    group with the same message, so that no rank is left waiting in a collective the others skip."""


class CountExchange:
    """The count all-gather in flight: :func:`exchange_counts_begin` enqueues it and an asynchronous
    copy to pinned host memory; :meth:`finish` waits for that copy only (work enqueued on the
    stream in between keeps running), checks the whole matrix and returns the split sizes."""

    def __init__(self, host, event, world, rank, chunks):
        self.host, self.event, self.world, self.rank, self.chunks = host, event, world, rank, chunks

    def finish(self):
        if self.event is not None:
            self.event.synchronize()
        world, rank, chunks = self.world, self.rank, self.chunks
        host = self.host.view(world, -1).tolist()
        n = chunks * world
        # matrix[src][chunk][dst]
        matrix = [[row[c * world:(c + 1) * world] for c in range(chunks)] for row in host]
        bad_ids = [int(row[n]) for row in host]
        caps = [int(row[n + 1]) for row in host]
        slots = [int(row[n + 2]) for row in host]
        if any(bad_ids):
            who = [r for r, b in enumerate(bad_ids) if b]
            raise ValueError(f"expert id outside [0, num_global_experts) on rank(s) {who}")
        for src in range(world):
            flat = [v for c in range(chunks) for v in matrix[src][c]]
            if min(flat, default=0) < 0:
                raise ExchangeRefused(f"expert-parallel count exchange: rank {src} reported a negative count {matrix[src]}")
            if slots[src] >= 0 and sum(flat) > slots[src]:
                raise ExchangeRefused(f"expert-parallel count exchange: rank {src} reported {sum(flat)} pairs "
                                      f"for {slots[src]} slots")
        for dst in range(world):
            n_in = sum(matrix[src][c][dst] for src in range(world) for c in range(chunks))
            if caps[dst] >= 0 and n_in > caps[dst]:
                raise ExchangeRefused(f"rank {dst} would receive {n_in} rows, capacity {caps[dst]}")
        send_l = matrix[rank]
        recv_l = [[matrix[src][c][rank] for src in range(world)] for c in range(chunks)]
        return send_l, recv_l


def exchange_counts_begin(send_counts: torch.Tensor, group, n_bad: torch.Tensor | None = None,
                          capacity: int | None = None, n_slots: int | None = None) -> CountExchange:
    """All-gather of every rank's [chunks, W] pair-count matrix, its count of invalid expert ids and
    its receive capacity: one collective and one copy to the host, both only enqueued here."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    chunks = send_counts.shape[0]
    dev = send_counts.device
    tail = torch.tensor([0, -1 if capacity is None else int(capacity), -1 if n_slots is None else int(n_slots)],
                        dtype=torch.int64).to(dev, non_blocking=True)
    if n_bad is not None:
        tail = tail + torch.nn.functional.pad(n_bad.reshape(1).to(torch.int64), (0, 2))
    mine = torch.cat([send_counts.to(torch.int64).reshape(-1), tail])          # [chunks * W + 3]
    everyone = torch.empty((world * mine.numel(),), dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(everyone, mine.contiguous(), group=group)
    if dev.type == "cuda":
        host = torch.empty(everyone.shape, dtype=torch.int64, pin_memory=True)
        host.copy_(everyone, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return CountExchange(host, event, world, rank, chunks)
    return CountExchange(everyone, None, world, rank, chunks)


def exchange_counts(send_counts: torch.Tensor, group, n_bad: torch.Tensor | None = None,
                    capacity: int | None = None, n_slots: int | None = None):
    """The count exchange in one call.  Returns ``(send, recv)`` as nested Python lists indexed
    [chunk][peer].

    Every rank sees the whole W x W matrix, so every rank reaches the SAME verdict before any
    payload moves: an invalid expert id anywhere raises ``ValueError`` everywhere; a negative
    count, a rank that claims more pairs than it has slots, or a rank whose receive capacity would
    be exceeded raises :class:`ExchangeRefused` everywhere.  (What a rank receives is by
    construction what the others send it: both are read from the one gathered matrix.)"""
    return exchange_counts_begin(send_counts, group, n_bad, capacity, n_slots).finish()


class ExpertParallelInt4:
    """Callable layer: ``out = layer(A, topk_ids, topk_w)`` with ``topk_ids`` global expert ids.

    ``packed``/``scale`` are this rank's experts in local-index order (``[E/W, N, K//8]`` int32 and
    ``[E/W, N, K//group]`` bf16; see :func:`local_expert_ids`).  ``partial_fn(A_rows, ids, w) ->
    [R, N] fp32`` computes for every received row the weighted sum over its experts
    (``ids [R, top_k]`` local expert indices, -1 = none; ``w [R, top_k]``); by default the C-ABI calls
    ``xkb_moe_int4_w4a16_rows`` + ``xkb_moe_gather_sum_reduce``.  ``reduce_fn(rows, row_index, M,
    dtype)`` is the final sum of each token's partial rows (``row_index [M, W]``, -1 = none); by
    default ``xkb_moe_gather_sum_reduce``.
    """

    def __init__(self, packed, scale, *, num_global_experts: int, group=None, group_size: int = 32,
                 placement: str = "contiguous", chunks: int = 1, partial_fn=None, reduce_fn=None,
                 max_recv_rows: int | None = None, sm_margin: int = 16, local_first: bool = False):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if num_global_experts % self.world != 0:
            raise ValueError("experts must shard evenly over the ranks")
        self.e_local = num_global_experts // self.world
        if packed.shape[0] != self.e_local:
            raise ValueError(f"rank holds {packed.shape[0]} experts, expected {self.e_local}")
        if chunks < 1:
            raise ValueError("chunks must be >= 1")
        owner_and_local(torch.zeros(1, dtype=torch.int64), self.e_local, self.world, placement)  # validates
        self.packed, self.scale, self.group_size = packed, scale, int(group_size)
        self.placement, self.chunks = placement, int(chunks)
        self.N = packed.shape[1]
        self.partial_fn = partial_fn or self._partial_cuda
        self.reduce_fn = reduce_fn or self._reduce_cuda
        self.max_recv_rows = max_recv_rows
        # chunked pipeline on GPUs: SMs the persistent GEMM kernels leave to NCCL's exchange kernels,
        # which would otherwise queue behind them instead of running beside them
        self.sm_margin = int(sm_margin)
        self.last_recv_rows = 0          # pairs (activation rows) received in the last call
        self.last_recv_slots = 0         # expert slots among them (the GEMM work of this rank)
        self.last_send_counts: list[int] = []
        self.own_packed, self.own_scale = packed, scale
        self.replicas: list[int] = []    # global ids of the experts every rank holds a copy of
        self.table = None                # [E, 2] int32 on the weights' device when replicas exist
        # Local-first: the slots whose expert this rank serves itself (its own experts and the
        # replicas) never enter the exchange.  They are computed from the rank's own tokens on a
        # second stream while the count exchange and the dispatch all-to-all are in flight, and
        # their partial rows join the final sum at this rank's position.  Needs one chunk.
        self.local_first = bool(local_first) and self.world > 1 and self.chunks == 1
        self._home_tables = None         # (table as seen from this rank, the same with home experts marked -1)
        self._side = None                # CUDA stream of the local pass

    # ---- replicas of popular experts -------------------------------------------------
    def set_replicas(self, global_ids, packed_rep=None, scale_rep=None) -> None:
        """Install copies of the experts ``global_ids`` (their weights in that order, ``[R, N, K//8]``
        and ``[R, N, K//group]``) behind this rank's own experts; an empty list removes them."""
        global_ids = [int(g) for g in global_ids]
        E = self.e_local * self.world
        if len(set(global_ids)) != len(global_ids) or any(g < 0 or g >= E for g in global_ids):
            raise ValueError("set_replicas: ids must be distinct global expert ids")
        self._home_tables = None
        if not global_ids:
            self.packed, self.scale, self.replicas, self.table = self.own_packed, self.own_scale, [], None
            return
        if packed_rep.shape[0] != len(global_ids) or scale_rep.shape[0] != len(global_ids):
            raise ValueError("set_replicas: one weight slice per replicated expert")
        self.packed = torch.cat([self.own_packed, packed_rep.to(self.own_packed.device)], dim=0).contiguous()
        self.scale = torch.cat([self.own_scale, scale_rep.to(self.own_scale.device)], dim=0).contiguous()
        self.replicas = global_ids
        self.table = expert_table(self.e_local, self.world, self.placement, self.rank, global_ids).to(
            self.own_packed.device)

    def rebalance(self, topk_ids: torch.Tensor, n_replicas: int) -> list[int]:
        """Collective.  Counts how often each global expert is chosen in ``topk_ids`` over all ranks,
        copies the ``n_replicas`` most popular experts to every rank (a broadcast from each owner)
        and from then on routes their slots to the token's own rank.  Returns their global ids."""
        E = self.e_local * self.world
        dev = self.own_packed.device
        hist = torch.bincount(topk_ids.reshape(-1).to(device=dev, dtype=torch.int64).clamp(0, E - 1), minlength=E)
        dist.all_reduce(hist, group=self.group)
        n = max(0, min(int(n_replicas), E))
        # most popular first; ties by ascending id so that every rank picks the same set
        order = torch.argsort(hist.cpu() * E + (E - 1 - torch.arange(E)), descending=True)
        hot = order[:n].tolist()
        if not hot:
            self.set_replicas([])
            return []
        owner, local = owner_and_local(torch.tensor(hot, dtype=torch.int64), self.e_local, self.world, self.placement)
        reps_p, reps_s = [], []
        for g, o, l in zip(hot, owner.tolist(), local.tolist()):
            if o == self.rank:
                pk, sc = self.own_packed[l].clone(), self.own_scale[l].clone()
            else:
                pk, sc = torch.empty_like(self.own_packed[0]), torch.empty_like(self.own_scale[0])
            src = dist.get_global_rank(self.group, o) if self.group is not dist.group.WORLD else o
            dist.broadcast(pk, src=src, group=self.group)
            dist.broadcast(sc, src=src, group=self.group)
            reps_p.append(pk)
            reps_s.append(sc)
        self.set_replicas(hot, torch.stack(reps_p), torch.stack(reps_s))
        return hot

    # ---- default CUDA compute ---------------------------------------------------------
    def _partial_cuda(self, rows_A: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        from . import ops

        R, top_k = ids.shape
        # one fp32 row per (received row, expert slot), already times the routing weight ...
        rows = ops.moe_int4_w4a16_rows(rows_A, self.packed, self.scale, ids, w, group_size=self.group_size)
        # ... summed per received row in ascending slot order (slots that went to other ranks skip)
        slot = torch.arange(R * top_k, dtype=torch.int32, device=ids.device).view(R, top_k)
        row_index = torch.where(ids >= 0, slot, torch.full_like(slot, -1))
        return ops.moe_gather_sum_reduce(rows, row_index, None, torch.float32)

    def _reduce_cuda(self, rows, row_index, M, dtype):
        from . import ops

        return ops.moe_gather_sum_reduce(rows, row_index, None, dtype)

    # ---- one step ----------------------------------------------------------------------
    def __call__(self, A: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        try:
            return self._step(A, topk_ids, topk_w)
        finally:
            # the SM margin is a process-wide setting of the library: never leave it behind, also not
            # when the exchange was refused half-way
            if A.is_cuda and self.sm_margin > 0 and self.chunks > 1:
                from . import _lib

                _lib.set_sm_margin(0)

    def _step(self, A: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        M, K = A.shape
        top_k = topk_ids.shape[1]
        chunks = max(1, min(self.chunks, M))
        local_first = self.local_first and M > 0
        plan_table, home, rows_all, local_done = self.table, None, None, None
        if local_first:
            if self._home_tables is None:
                full = expert_table(self.e_local, self.world, self.placement, self.rank, self.replicas)
                away = expert_table(self.e_local, self.world, self.placement, self.rank, self.replicas,
                                    home_is_not_dispatched=True)
                self._home_tables = (full.to(A.device), away.to(A.device))
            full, plan_table = self._home_tables
            E = self.e_local * self.world
            t = full[topk_ids.to(torch.int64).clamp(0, E - 1)]                       # [M, top_k, 2]; invalid ids are refused below
            home_ids = torch.where(t[..., 0] == self.rank, t[..., 1], torch.full_like(t[..., 1], -1)).to(torch.int32)
            home = (home_ids, topk_w.to(torch.float32))
            # rows of the final sum: [0, M) this rank's own partial per token, then one row per pair
            cap = M * min(top_k, self.world - 1)
            rows_all = torch.empty((M + cap, self.N), dtype=torch.float32, device=A.device)
            fused_home = A.is_cuda and self.partial_fn == self._partial_cuda
            if fused_home:
                routing_home = torch.cat([home_ids, home[1].view(torch.int32)], dim=1).contiguous()
            else:
                rows_all[:M] = self.partial_fn(A, home_ids, home[1])
        if A.is_cuda:
            # the plan on the device (three launches, no host read); the one read of the count exchange
            # also brings the pair count and the invalid-id count.  The send buffer is filled by a
            # gather whose row count is read on the device, enqueued BEFORE the host waits for the
            # counts, so the copy runs while the host is still blocked.
            from . import ops

            pair_token, _dest, routing, pair_of, counts, info = ops.ep_plan(
                topk_ids, topk_w, self.e_local, self.world, self.placement, chunks, table=plan_table)
            pending = exchange_counts_begin(counts, self.group, n_bad=info[1], capacity=self.max_recv_rows,
                                            n_slots=M * top_k)
            send_all = ops.gather_rows(A, pair_token, info[0:1])          # [M * top_k, K]; the first P rows are set
            if local_first and fused_home:
                # The local pass goes to a second stream AFTER everything the exchange waits for has been
                # queued (plan, counts, send-buffer gather), so that those kernels get their SMs first;
                # it then runs beside the host's wait for the counts and the dispatch all-to-all, with
                # sm_margin SMs left to NCCL's kernels.  The remote pass afterwards takes every SM.
                from . import _lib

                if self._side is None:
                    self._side = torch.cuda.Stream(device=A.device)
                self._side.wait_stream(torch.cuda.current_stream(A.device))
                if self.sm_margin > 0:
                    _lib.set_sm_margin(self.sm_margin)
                try:
                    with torch.cuda.stream(self._side):
                        ops.moe_int4_w4a16_partial(A, self.packed, self.scale, routing_home, group_size=self.group_size,
                                                   out=rows_all[:M], workspace_tag=2)
                        local_done = torch.cuda.Event()
                        local_done.record(self._side)
                finally:
                    if self.sm_margin > 0:
                        _lib.set_sm_margin(0)
                A.record_stream(self._side)
                rows_all.record_stream(self._side)
                routing_home.record_stream(self._side)
            send_l, recv_l = pending.finish()
            P = sum(sum(r) for r in send_l)
            pair_token, send_R, send_A = pair_token[:P], routing[:P], send_all[:P]
        else:
            plan = plan_dispatch(topk_ids, self.e_local, self.world, self.placement, chunks, host_checks=False,
                                 table=plan_table)
            send_l, recv_l = exchange_counts(plan.send_counts, self.group, n_bad=plan.n_bad,
                                             capacity=self.max_recv_rows, n_slots=M * top_k)
            P = sum(sum(r) for r in send_l)
            plan.trim(P)
            pair_token, pair_of = plan.pair_token, plan.pair_of
            # routing of a pair in one int32 row: top_k local expert ids, then the top_k weights' bit patterns
            w_pairs = torch.where(plan.pair_ids >= 0, topk_w.to(torch.float32)[pair_token],
                                  torch.zeros((), dtype=torch.float32, device=A.device))
            send_R = torch.cat([plan.pair_ids, w_pairs.view(torch.int32)], dim=1).contiguous()
            send_A = A.index_select(0, pair_token)
        n_recv = sum(sum(r) for r in recv_l)
        self.last_recv_rows = n_recv
        self.last_send_counts = [sum(send_l[c][p] for c in range(chunks)) for p in range(self.world)]

        if local_first:
            back = rows_all[M:M + P]
            # this rank's own partial sits at its position in every token's row of the index, so the
            # sum runs over the ranks in the same order as without the local pass
            pair_of = torch.where(pair_of >= 0, pair_of + M, pair_of)
            pair_of[:, self.rank] = torch.arange(M, dtype=pair_of.dtype, device=pair_of.device)
        else:
            back = torch.empty((P, self.N), dtype=torch.float32, device=A.device)
        use_async = A.is_cuda and chunks > 1

        # dispatch every chunk (in flight back to back on the communication stream) ...
        recv, works, off = [], [], 0
        for c in range(chunks):
            n_send, n_in = sum(send_l[c]), sum(recv_l[c])
            rA = torch.empty((n_in, K), dtype=A.dtype, device=A.device)
            rR = torch.empty((n_in, 2 * top_k), dtype=torch.int32, device=A.device)
            w1 = dist.all_to_all_single(rA, send_A[off:off + n_send], recv_l[c], send_l[c], group=self.group,
                                        async_op=use_async)
            w2 = dist.all_to_all_single(rR, send_R[off:off + n_send], recv_l[c], send_l[c], group=self.group,
                                        async_op=use_async)
            recv.append((rA, rR, off, n_send))
            works.append((w1, w2))
            off += n_send
        # ... then per chunk: wait for its rows, expert GEMM + per-row sum, send the fp32 partials home
        back_works = []
        fused_partial = A.is_cuda and self.partial_fn == self._partial_cuda
        margin = use_async and fused_partial and self.sm_margin > 0
        if margin:
            from . import _lib

            _lib.set_sm_margin(self.sm_margin)
        try:
            for c in range(chunks):
                rA, rR, coff, n_send = recv[c]
                if use_async:
                    works[c][0].wait()
                    works[c][1].wait()
                if fused_partial:
                    # one C call: routing split, align, gather, grouped GEMM, fp32 sum per received row
                    partial = ops.moe_int4_w4a16_partial(rA, self.packed, self.scale, rR, group_size=self.group_size)
                else:
                    r_ids = rR[:, :top_k].contiguous()
                    r_w = rR[:, top_k:].contiguous().view(torch.float32)
                    partial = self.partial_fn(rA, r_ids, r_w)  # [n_in, N] fp32
                wb = dist.all_to_all_single(back[coff:coff + n_send], partial, send_l[c], recv_l[c], group=self.group,
                                            async_op=use_async)
                back_works.append((wb, partial, rR))
        finally:
            if margin:
                _lib.set_sm_margin(0)
        if use_async:
            for wb, _p, _i in back_works:
                wb.wait()
        self._last_routing = [r for _wb, _p, r in back_works]
        if local_first:
            if local_done is not None:
                torch.cuda.current_stream(A.device).wait_event(local_done)
            self._last_routing.append(torch.cat([home[0], home[1].view(torch.int32)], dim=1))
            return self.reduce_fn(rows_all[:M + P], pair_of, M, A.dtype)
        return self.reduce_fn(back, pair_of, M, A.dtype)

    def count_recv_slots(self) -> int:
        """Expert slots among the rows received in the last call (one host read; diagnostics only)."""
        top_k = self._last_routing[0].shape[1] // 2 if self._last_routing else 0
        self.last_recv_slots = int(sum(int((r[:, :top_k] >= 0).sum()) for r in self._last_routing))
        return self.last_recv_slots
