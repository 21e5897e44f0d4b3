"""Expert-parallel INT4 fused MoE with all-to-all dispatch and combine.

One process per GPU; rank r owns the contiguous expert slice
``[r*E/W, (r+1)*E/W)`` and its own batch of tokens.  A call does

  1. plan: group this rank's token-slots by destination rank (stable),
  2. exchange the per-rank slot counts (one small all-to-all, one host read),
  3. dispatch: all-to-all of the routed activation rows and their local expert ids,
  4. local grouped GEMM over the received rows (one slot per row, no combine),
  5. combine: all-to-all of the fp32 result rows back to the token owners,
  6. fixed-order weighted top-k reduce on the owner.

The reference has no all-to-all (its expert parallelism replicates tokens and
lets the caller all-reduce partials, src/xkernels/ops/moe/interface.py:37-57);
what it fixes is the result: the dense op on each rank's tokens with the global
expert set.  fp32 rows travel back so that the reduce sees the same operands as
the single-GPU op (a bf16 round per expert fails the op tolerance on some
elements, see meta/docs/wiki/04-gotchas.md:452-454 in the reference).

The exchange uses ``torch.distributed`` (NCCL on GPUs, gloo on CPU); data lands in
local buffers before any kernel reads it.  The local compute is pluggable so the
routing logic runs on CPU ranks in tests.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    order: torch.Tensor        # [numel] slot ids grouped by destination rank (stable inside a rank)
    send_counts: torch.Tensor  # [W] int64, slots sent to each rank
    local_expert: torch.Tensor  # [numel] int32, expert id on the destination rank, in `order`
    token: torch.Tensor        # [numel] int64, source token row of each sorted slot


def plan_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int) -> DispatchPlan:
    """Group the ``M*top_k`` slots by the rank that owns their expert."""
    M, top_k = topk_ids.shape
    flat = topk_ids.reshape(-1).to(torch.int64)
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= experts_per_rank * world):
        raise ValueError("expert id outside [0, num_global_experts)")
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)
    local = (flat[order] - dest[order] * experts_per_rank).to(torch.int32)
    token = torch.div(order, top_k, rounding_mode="floor")
    return DispatchPlan(order=order, send_counts=counts, local_expert=local, token=token)


def exchange_counts(send_counts: torch.Tensor, group) -> tuple[list[int], list[int]]:
    """All-to-all of the slot counts; returns (send, recv) as Python lists and validates them."""
    world = dist.get_world_size(group)
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    both = torch.stack([send_counts, recv]).cpu()
    send_l, recv_l = both[0].tolist(), both[1].tolist()
    if len(send_l) != world or min(send_l + recv_l) < 0:
        raise RuntimeError(f"expert-parallel count exchange returned invalid counts: {send_l} / {recv_l}")
    return send_l, recv_l


class ExpertParallelInt4:
    """Callable layer: ``out = layer(A, topk_ids, topk_w)`` with ``topk_ids`` global expert ids.

    ``packed``/``scale`` are this rank's expert slice (``[E/W, N, K//8]`` int32 and
    ``[E/W, N, K//group]`` bf16).  ``rows_fn(A_rows, local_expert_ids) -> [R, N] fp32`` computes
    one un-weighted expert GEMM row per received row; by default it is the C-ABI call
    ``xkb_moe_int4_w4a16_rows`` with ``top_k = 1``.  ``reduce_fn(rows, row_index, w, M, dtype)``
    is the final gather + weighted sum; by default ``xkb_moe_gather_sum_reduce``.
    """

    def __init__(self, packed, scale, *, num_global_experts: int, group=None, group_size: int = 32,
                 rows_fn=None, reduce_fn=None, max_recv_slots: int | None = None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if num_global_experts % self.world != 0:
            raise ValueError("experts must shard evenly over the ranks")
        self.e_local = num_global_experts // self.world
        if packed.shape[0] != self.e_local:
            raise ValueError(f"rank holds {packed.shape[0]} experts, expected {self.e_local}")
        self.packed, self.scale, self.group_size = packed, scale, int(group_size)
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
        plan = plan_dispatch(topk_ids, self.e_local, self.world)
        send_l, recv_l = exchange_counts(plan.send_counts, self.group)
        n_recv = sum(recv_l)
        if self.max_recv_slots is not None and n_recv > self.max_recv_slots:
            raise RuntimeError(f"rank {self.rank} would receive {n_recv} slots, capacity {self.max_recv_slots}")
        self.last_recv_slots, self.last_send_counts = n_recv, send_l

        send_A = A.index_select(0, plan.token)
        recv_A = torch.empty((n_recv, K), dtype=A.dtype, device=A.device)
        recv_e = torch.empty((n_recv,), dtype=torch.int32, device=A.device)
        dist.all_to_all_single(recv_A, send_A, recv_l, send_l, group=self.group)
        dist.all_to_all_single(recv_e, plan.local_expert, recv_l, send_l, group=self.group)

        rows = self.rows_fn(recv_A, recv_e)  # [n_recv, N] fp32, un-weighted
        back = torch.empty((plan.order.numel(), self.N), dtype=torch.float32, device=A.device)
        dist.all_to_all_single(back, rows, send_l, recv_l, group=self.group)

        # slot s sits at sorted position inv[s]
        inv = torch.empty_like(plan.order)
        inv[plan.order] = torch.arange(plan.order.numel(), device=A.device)
        row_index = inv.view(M, top_k).to(torch.int32)
        return self.reduce_fn(back, row_index, topk_w.to(torch.float32), M, A.dtype)
