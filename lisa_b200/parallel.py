"""One-node multi-GPU forms of the path: N-sharded linears with an all-gather of the outputs, and
expert-parallel routed experts with all-to-all dispatch and combine.

The reference has no multi-device code (one Apple GPU); the only hook it offers is DS4's
contiguous expert-ownership rule ``first = rank * (E / world)``
(crates/lisa-mlx/src/shaders/deepseek41/iq.metal:976-982), which the expert-parallel split below
follows.  One process per GPU; ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU
tests) is the plumbing.  The compute callables default to the CUDA operators of ``lisa_b200.ops``;
tests inject CPU stand-ins to exercise the sharding logic without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """Contiguous output-row range of `rank`: ranges are multiples of `multiple` rows (the GGUF
    kernels need rows % 8 == 0), the remainder goes to the last ranks one block at a time."""
    if n % multiple != 0:
        raise ValueError(f"N={n} is not a multiple of {multiple}")
    blocks = n // multiple
    base, extra = divmod(blocks, world)
    begin = rank * base + max(0, rank - (world - extra)) if extra else rank * base
    count = base + (1 if extra and rank >= world - extra else 0)
    return begin * multiple, (begin + count) * multiple


@dataclass
class ShardedQuantizedLinear:
    """Rank-local slice ``W[n0:n1, :]`` of a quantized linear (weights, scales, biases keep the
    reference layout); every rank holds the full activation and computes ``y[:, n0:n1]``."""
    weight: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    n_total: int
    n0: int
    n1: int
    group_size: int = 64
    bits: int = 4

    @classmethod
    def from_full(cls, weight, scales, biases, world: int, rank: int, group_size: int = 64, bits: int = 4):
        n = weight.shape[0]
        n0, n1 = shard_rows(n, world, rank)
        return cls(weight[n0:n1].contiguous(), scales[n0:n1].contiguous(), biases[n0:n1].contiguous(), n, n0, n1,
                   group_size, bits)

    def forward(self, x: torch.Tensor, matmul: Optional[Callable] = None, group=None) -> torch.Tensor:
        """x [M, K] (same on every rank) -> y [M, N] on every rank: local slice, then all-gather."""
        if matmul is None:
            from . import ops
            matmul = ops.quantized_matmul
        local = matmul(x, self.weight, self.scales, self.biases, True, self.group_size, self.bits)
        return all_gather_columns(local, self.n_total, group=group)


def all_gather_columns(local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """Gathers column blocks [M, n_r] of all ranks into [M, N].  For M == 1 the gathered buffer is
    already the output; for M > 1 the [world, M, n_r] gather is laid out rank-major and permuted."""
    world = dist.get_world_size(group)
    m = local.shape[0]
    sizes = [shard_rows(n_total, world, r) for r in range(world)]
    widths = [b - a for a, b in sizes]
    if len(set(widths)) == 1:
        out = torch.empty((world * m, widths[0]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out.view(world, m, widths[0]).permute(1, 0, 2).reshape(m, n_total)
    # uneven shards: pad every slice to the widest one, gather, drop the padding
    wmax = max(widths)
    padded = torch.zeros((m, wmax), dtype=local.dtype, device=local.device)
    padded[:, : local.shape[1]] = local
    out = torch.empty((world * m, wmax), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    out = out.view(world, m, wmax)
    return torch.cat([out[r, :, : widths[r]] for r in range(world)], dim=1)


def expert_range(experts: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous expert ownership, iq.metal:976-982: first = rank * (E / world)."""
    if experts % world != 0:
        raise ValueError(f"{experts} experts do not split over {world} ranks")
    per = experts // world
    return rank * per, (rank + 1) * per


def ep_dispatch_plan(idx: torch.Tensor, experts: int, world: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """For the local tokens' routing `idx` [T, top_k]: the destination rank of every slot, a stable
    order that groups slots by destination rank, and the number of slots per destination."""
    per = experts // world
    flat = idx.reshape(-1).to(torch.int64)
    dest = torch.div(flat, per, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices
    counts = torch.bincount(dest, minlength=world)
    return dest, order, counts


def ep_moe_forward(x: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor, experts: int,
                   local_experts: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                   combine: Optional[Callable] = None, group=None) -> torch.Tensor:
    """Expert-parallel routed experts for the tokens this rank owns.

    x [T, H] bf16 (rank-local tokens), idx int32 [T, top_k], weights f32 [T, top_k] from the
    replicated router.  `local_experts(rows [R, H], local_ids [R]) -> [R, H]` runs the rank's own
    experts (gate/up gather_qmm, SwiGLU, down gather_qmm) on rows sorted however it likes and
    returns them in the order given.  Exchange: slot counts (all-to-all of one int per peer), rows
    and expert ids to the owners (all-to-all), results back (all-to-all), then the weighted fold in
    original slot order on the token's rank (`combine(rows_sorted, weights, inverse, top_k)`,
    default the CUDA ``ops.moe_combine``)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    t, top_k = idx.shape
    hidden = x.shape[1]
    dest, order, send_counts = ep_dispatch_plan(idx, experts, world)
    token_of_slot = torch.div(order, top_k, rounding_mode="floor")
    send_rows = x[token_of_slot].contiguous()
    send_ids = idx.reshape(-1)[order].to(torch.int32).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    s_list, r_list = send_counts.tolist(), recv_counts.tolist()
    recv_rows = torch.empty((sum(r_list), hidden), dtype=x.dtype, device=x.device)
    recv_ids = torch.empty((sum(r_list),), dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_rows, send_rows, r_list, s_list, group=group)
    dist.all_to_all_single(recv_ids, send_ids, r_list, s_list, group=group)
    e0, _ = expert_range(experts, world, rank)
    out_rows = local_experts(recv_rows, recv_ids - e0) if recv_rows.shape[0] else recv_rows
    back = torch.empty_like(send_rows)
    dist.all_to_all_single(back, out_rows.contiguous(), s_list, r_list, group=group)
    # `back` is in dispatch order; inverse[slot] = its row there.  Fold in original slot order.
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device)
    if combine is None:
        from . import ops
        combine = ops.moe_combine
    return combine(back, weights.reshape(t, top_k), inverse.to(torch.int32), top_k)
