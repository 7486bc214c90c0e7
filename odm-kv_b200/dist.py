"""Sharding of the hot path over the GPUs of one node (one process per GPU, torch.distributed).

The path partitions naturally: layers and samples are independent problems, and within a problem the KV
heads are independent for scoring, quantise-and-pack and decode attention.  Only two exchanges exist:
  * with KV heads sharded, the per-layer Lagrangian couples the heads of a (layer, sample): every pass of
    the allocator all-reduces a handful of integer counts (`allocate_bits_kv_sharded`);
  * the per-head attention outputs are gathered (`gather_head_outputs`).
With layers (or samples) sharded instead, compress needs no collective at all.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [lo, hi) share of n units for `rank` of `world` (first n % world ranks get one more)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def plan_units(n_layers: int, n_kv_heads: int, world: int, rank: int, prefer: str = "layers") -> dict:
    """Which (layer, KV head) units a rank owns.  `prefer="layers"` splits layers first (no compress
    collective) and only splits heads when there are fewer layers than ranks; `"heads"` splits KV heads
    (tensor-parallel style: the allocator's count exchange is then needed inside each layer)."""
    if prefer == "heads":
        if n_kv_heads % world and world % n_kv_heads:
            raise ValueError(f"cannot split {n_kv_heads} KV heads over {world} ranks")
        if world <= n_kv_heads:
            h_lo, h_hi = shard_range(n_kv_heads, world, rank)
            return {"layers": (0, n_layers), "heads": (h_lo, h_hi), "head_group": list(range(world))}
        per = world // n_kv_heads
        h = rank // per
        l_lo, l_hi = shard_range(n_layers, per, rank % per)
        return {"layers": (l_lo, l_hi), "heads": (h, h + 1), "head_group": [r for r in range(world) if r % per == rank % per]}
    if world <= n_layers:
        l_lo, l_hi = shard_range(n_layers, world, rank)
        return {"layers": (l_lo, l_hi), "heads": (0, n_kv_heads), "head_group": [rank]}
    per = world // n_layers
    layer = rank // per
    h_lo, h_hi = shard_range(n_kv_heads, per, rank % per)
    return {"layers": (layer, layer + 1), "heads": (h_lo, h_hi), "head_group": [r for r in range(world) if r // per == layer]}


def all_reduce_sum_(t: torch.Tensor, group=None) -> torch.Tensor:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def allocate_bits_kv_sharded(scores_local: torch.Tensor, sink_mask_local: Optional[torch.Tensor], levels: Sequence[int],
                             eps: Sequence[float], target: float, head_lo: int, T: int, group=None, sink_bits: int = 16):
    """Per-layer Lagrangian with the KV heads of each problem spread over the ranks of `group`.
    scores_local [P, H_local, T] are this rank's heads (head_lo = index of its first head); every rank gets
    the bits of its own heads, identical to what a single device would assign to them."""
    from . import ops
    P, Hl, Tl = scores_local.shape
    mask = None if sink_mask_local is None else sink_mask_local.reshape(-1)
    bits, rep = ops.allocate_bits_sharded(scores_local.reshape(P, Hl * Tl), mask, levels, eps, target, idx_base=head_lo * T,
                                          all_reduce=lambda t: all_reduce_sum_(t, group), sink_bits=sink_bits)
    return bits.reshape(P, Hl, Tl), rep


def gather_head_outputs(out_local: torch.Tensor, group=None, dim: int = 1) -> torch.Tensor:
    """All-gather attention outputs [B, Hq_local, d] of head-sharded ranks into [B, Hq, d] (rank order)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return out_local
    parts: List[torch.Tensor] = [torch.empty_like(out_local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=dim)
