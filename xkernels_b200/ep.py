"""Expert-parallel INT4 fused MoE with all-to-all dispatch and combine.

One process per GPU; every rank owns ``E/W`` experts and its own batch of tokens.  A call does

  1. plan: group this rank's token-slots by (token chunk, destination rank), stable inside a group,
  2. exchange the slot-count matrix (one small all-to-all, one host read; counts are validated
     on the host before any payload moves),
  3. per chunk: dispatch all-to-all of the routed activation rows and their local expert ids,
     local grouped GEMM over the received rows (one slot per row, no combine), all-to-all of the
     fp32 result rows back to the token owners,
  4. fixed-order weighted top-k reduce on the owner.

With ``chunks > 1`` the exchanges of chunk c+1 are in flight on NCCL's stream while the GEMM of
chunk c runs, so transfer and tensor work overlap.

The reference has no all-to-all (its expert parallelism replicates tokens and lets the caller
all-reduce partials, src/xkernels/ops/moe/interface.py:37-57); what it fixes is the result: the
dense op on each rank's tokens with the global expert set.  fp32 rows travel back so that the
reduce sees the same operands as the single-GPU op (a bf16 round per expert fails the op tolerance
on some elements, see meta/docs/wiki/04-gotchas.md:452-454 in the reference).

Expert placement: ``"contiguous"`` (rank r owns experts ``[r*E/W, (r+1)*E/W)``, the layout of the
reference's ``expert_map`` tests, tests/test_moe_int4_ep.py:84-93) or ``"round_robin"`` (expert g
lives on rank ``g % W`` as local expert ``g // W``), which spreads a popularity-ranked expert set
evenly over the ranks.

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
    raise ValueError(f"unknown expert placement {placement!r}")


def local_expert_ids(rank: int, experts_per_rank: int, world: int, placement: str) -> list[int]:
    """Global ids of the experts rank ``rank`` holds, in local-index order."""
    if placement == "contiguous":
        return list(range(rank * experts_per_rank, (rank + 1) * experts_per_rank))
    if placement == "round_robin":
        return [rank + world * i for i in range(experts_per_rank)]
    raise ValueError(f"unknown expert placement {placement!r}")


@dataclass
class DispatchPlan:
    order: torch.Tensor         # [numel] slot ids grouped by (chunk, destination rank), stable inside a group
    send_counts: torch.Tensor   # [chunks, W] int64
    local_expert: torch.Tensor  # [numel] int32, expert index on the destination rank, in `order`
    token: torch.Tensor         # [numel] int64, source token row of each sorted slot


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int, placement: str = "contiguous",
                  chunks: int = 1) -> DispatchPlan:
    """Group the ``M*top_k`` slots by (token chunk, owner rank of their expert)."""
    M, top_k = topk_ids.shape
    flat = topk_ids.reshape(-1).to(torch.int64)
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= experts_per_rank * world):
        raise ValueError("expert id outside [0, num_global_experts)")
    dest, local = owner_and_local(flat, experts_per_rank, world, placement)
    slot = torch.arange(flat.numel(), device=flat.device)
    tokens_per_chunk = -(-M // chunks) if M else 1
    chunk = torch.div(torch.div(slot, top_k, rounding_mode="floor"), tokens_per_chunk, rounding_mode="floor")
    key = chunk * world + dest
    order = torch.argsort(key, stable=True)
    counts = torch.bincount(key, minlength=chunks * world).view(chunks, world)
    return DispatchPlan(order=order, send_counts=counts, local_expert=local[order].to(torch.int32),
                        token=torch.div(order, top_k, rounding_mode="floor"))


def exchange_counts(send_counts: torch.Tensor, group) -> tuple[list[list[int]], list[list[int]]]:
    """All-to-all of the [chunks, W] slot-count matrix.  Returns (send, recv) as nested Python lists
    indexed [chunk][peer] and validates them."""
    world = dist.get_world_size(group)
    chunks = send_counts.shape[0]
    send_t = send_counts.t().contiguous()            # [W, chunks]: row p goes to peer p
    recv_t = torch.empty_like(send_t)
    dist.all_to_all_single(recv_t, send_t, group=group)
    both = torch.stack([send_t, recv_t]).cpu()
    send_l = both[0].t().tolist()
    recv_l = both[1].t().tolist()
    flat = [v for row in send_l + recv_l for v in row]
    if len(send_l) != chunks or any(len(r) != world for r in send_l + recv_l) or (flat and min(flat) < 0):
        raise RuntimeError(f"expert-parallel count exchange returned invalid counts: {send_l} / {recv_l}")
    return send_l, recv_l


class ExpertParallelInt4:
    """Callable layer: ``out = layer(A, topk_ids, topk_w)`` with ``topk_ids`` global expert ids.

    ``packed``/``scale`` are this rank's experts in local-index order (``[E/W, N, K//8]`` int32 and
    ``[E/W, N, K//group]`` bf16; see :func:`local_expert_ids`).  ``rows_fn(A_rows, local_expert_ids)
    -> [R, N] fp32`` computes one un-weighted expert GEMM row per received row; by default it is the
    C-ABI call ``xkb_moe_int4_w4a16_rows`` with ``top_k = 1``.  ``reduce_fn(rows, row_index, w, M,
    dtype)`` is the final gather + weighted sum; by default ``xkb_moe_gather_sum_reduce``.
    """

    def __init__(self, packed, scale, *, num_global_experts: int, group=None, group_size: int = 32,
                 placement: str = "contiguous", chunks: int = 1, rows_fn=None, reduce_fn=None,
                 max_recv_slots: int | None = None):
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
        self.rows_fn = rows_fn or self._rows_cuda
        self.reduce_fn = reduce_fn or self._reduce_cuda
        self.max_recv_slots = max_recv_slots
        self.last_recv_slots = 0
        self.last_send_counts: list[int] = []

    # ---- default CUDA compute ---------------------------------------------------------
    def _rows_cuda(self, rows_A: torch.Tensor, local_expert: torch.Tensor) -> torch.Tensor:
        from . import ops

        return ops.moe_int4_w4a16_rows(rows_A, self.packed, self.scale, local_expert.view(-1, 1),
                                       group_size=self.group_size)

    def _reduce_cuda(self, rows, row_index, w, M, dtype):
        from . import ops

        return ops.moe_gather_sum_reduce(rows, row_index, w, dtype)

    # ---- one step ----------------------------------------------------------------------
    def __call__(self, A: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        M, K = A.shape
        top_k = topk_ids.shape[1]
        chunks = max(1, min(self.chunks, M))
        plan = plan_dispatch(topk_ids, self.e_local, self.world, self.placement, chunks)
        send_l, recv_l = exchange_counts(plan.send_counts, self.group)
        n_recv = sum(sum(r) for r in recv_l)
        if self.max_recv_slots is not None and n_recv > self.max_recv_slots:
            raise RuntimeError(f"rank {self.rank} would receive {n_recv} slots, capacity {self.max_recv_slots}")
        self.last_recv_slots = n_recv
        self.last_send_counts = [sum(send_l[c][p] for c in range(chunks)) for p in range(self.world)]

        numel = plan.order.numel()
        send_A = A.index_select(0, plan.token)
        back = torch.empty((numel, self.N), dtype=torch.float32, device=A.device)
        use_async = A.is_cuda and chunks > 1

        # dispatch every chunk (in flight back to back on the communication stream) ...
        recv, works, off = [], [], 0
        for c in range(chunks):
            n_send, n_in = sum(send_l[c]), sum(recv_l[c])
            rA = torch.empty((n_in, K), dtype=A.dtype, device=A.device)
            rE = torch.empty((n_in,), dtype=torch.int32, device=A.device)
            w1 = dist.all_to_all_single(rA, send_A[off:off + n_send], recv_l[c], send_l[c], group=self.group,
                                        async_op=use_async)
            w2 = dist.all_to_all_single(rE, plan.local_expert[off:off + n_send], recv_l[c], send_l[c],
                                        group=self.group, async_op=use_async)
            recv.append((rA, rE, off, n_send))
            works.append((w1, w2))
            off += n_send
        # ... then per chunk: wait for its rows, expert GEMM, send the fp32 rows home
        back_works = []
        for c in range(chunks):
            rA, rE, coff, n_send = recv[c]
            if use_async:
                works[c][0].wait()
                works[c][1].wait()
            rows = self.rows_fn(rA, rE)  # [n_in, N] fp32, un-weighted
            wb = dist.all_to_all_single(back[coff:coff + n_send], rows, send_l[c], recv_l[c], group=self.group,
                                        async_op=use_async)
            back_works.append((wb, rows))
        if use_async:
            for wb, _rows in back_works:
                wb.wait()

        # slot s sits at sorted position inv[s]
        inv = torch.empty_like(plan.order)
        inv[plan.order] = torch.arange(numel, device=A.device)
        row_index = inv.view(M, top_k).to(torch.int32)
        return self.reduce_fn(back, row_index, topk_w.to(torch.float32), M, A.dtype)
