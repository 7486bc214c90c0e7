"""Score -> bit-level mapping (mirrors the reference's ``kvquant/allocator.py``).

``optimal_scores_to_bits`` (459-663) and ``calibrate_epsilon`` (352-452) run on the CUDA kernels;
``ratio_scores_to_bits`` (46-148) and ``scores_to_bits`` (11-43) are small rank / bucket maps used
by the decode-buffer flush and are expressed with device tensor operations.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import ops
from .tq_backend import random_rotation

__all__ = ["scores_to_bits", "ratio_scores_to_bits", "optimal_scores_to_bits", "calibrate_epsilon", "effective_bits",
           "DEFAULT_BIT_LEVELS"]

DEFAULT_BIT_LEVELS: tuple[int, ...] = (0, 1, 2, 4, 8)
last_report: list = []   # raw report buffers of the most recent optimal_scores_to_bits call


def effective_bits(b: int, n_outlier: int = 0, d: int = 128, outlier_min_bits: int = 4) -> float:
    """kvquant/allocator.py:333-342."""
    if b == 0 or b >= 16 or n_outlier <= 0:
        return float(b)
    return b + n_outlier * max(0, max(b, outlier_min_bits) - b) / d


def scores_to_bits(scores: torch.Tensor, bit_levels: Sequence[int] = DEFAULT_BIT_LEVELS) -> torch.Tensor:
    """Uniform partition of [0, 1] (kvquant/allocator.py:11-43)."""
    bits_t = torch.tensor(sorted(bit_levels), dtype=torch.int32, device=scores.device)
    if len(bit_levels) == 1:
        return bits_t[0].expand_as(scores).clone()
    n = len(bit_levels)
    thresholds = torch.linspace(0.0, 1.0, n + 1)[1:-1].to(scores.device)
    return bits_t[torch.bucketize(scores.float(), thresholds)]


def ratio_scores_to_bits(scores: torch.Tensor, bit_levels: Sequence[int], ratios: Sequence[float],
                         sink_mask: Optional[torch.Tensor] = None, sink_bits: int = 16, per_head: bool = True) -> torch.Tensor:
    """Rank-tier allocation with given proportions (kvquant/allocator.py:46-148): ascending stable
    rank, tier sizes ``int(round(r * n))`` (Python's rounding), the last tier takes the remainder."""
    assert len(bit_levels) == len(ratios)
    shape = scores.shape
    if per_head and scores.dim() >= 2:
        view = scores.reshape(-1, shape[-1])
        mview = None if sink_mask is None else sink_mask.reshape(-1, shape[-1])
        rows = [ratio_scores_to_bits(view[i], bit_levels, ratios, None if mview is None else mview[i], sink_bits, per_head=False)
                for i in range(view.shape[0])]
        return torch.stack(rows).reshape(shape)
    flat = scores.flatten()
    n = flat.shape[0]
    result = torch.empty(n, dtype=torch.int32, device=scores.device)
    if sink_mask is not None:
        fs = sink_mask.flatten().bool()
        result[fs] = sink_bits
        idx = (~fs).nonzero(as_tuple=True)[0]
    else:
        idx = torch.arange(n, device=scores.device)
    n_active = idx.shape[0]
    if n_active == 0:
        return result.reshape(shape)
    rt = torch.tensor(ratios, dtype=torch.float64)
    rt = (rt / rt.sum()).tolist()
    order = torch.argsort(flat[idx], stable=True)
    bits = torch.empty(n_active, dtype=torch.int32, device=scores.device)
    tiers = sorted(zip([int(b) for b in bit_levels], rt), key=lambda t: t[0])
    cursor = 0
    for i, (b, r) in enumerate(tiers):
        count = n_active - cursor if i == len(tiers) - 1 else min(int(round(r * n_active)), n_active - cursor)
        bits[order[cursor:cursor + count]] = b
        cursor += count
    result[idx] = bits
    return result.reshape(shape)


_epsilon_cache: dict = {}


@torch.no_grad()
def calibrate_epsilon(d: int, bit_levels: Sequence[int], *, n_samples: int = 4096, seed: int = 42, device="cuda",
                      value_group_size: int = 32, n_outlier: int = 0, outlier_min_bits: int = 4,
                      value_quantizer: str = "mse") -> dict[int, float]:
    """Relative MSE of the key and value quantisers per level (kvquant/allocator.py:352-452) for the
    "mse" value quantiser without outlier channels: eps(b) = (relMSE_key + relMSE_value) / 2 on 4096
    seeded fp16 Gaussian vectors, key rotation seed ``seed``, value rotation seed ``seed + 2000``."""
    if n_outlier > 0 or str(value_quantizer).lower() not in ("mse", "turboquant", "turboquant_mse"):
        raise NotImplementedError("only the Lloyd-Max (mse) quantiser without outlier channels is implemented")
    device = torch.device(device)
    if device.type != "cuda":
        raise ops._lib.OdmkvError("calibrate_epsilon runs the CUDA quantiser: pass a CUDA device")
    key = (d, tuple(sorted(bit_levels)), seed, n_samples, str(device))
    if key in _epsilon_cache:
        return _epsilon_cache[key]
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    x = torch.randn(n_samples, d, generator=gen).to(device=device, dtype=torch.float16)
    xf = x.float()
    x_norm_sq = xf.pow(2).sum(-1).mean().item()
    pi_k = random_rotation(d, device, torch.float32, seed=seed)
    pi_v = random_rotation(d, device, torch.float32, seed=seed + 2000)
    out: dict[int, float] = {}
    for b in sorted(set(int(v) for v in bit_levels)):
        if b == 0:
            out[0] = 1.0
            continue
        if b >= 16:
            out[b] = 0.0
            continue
        flat = x.reshape(1, 1, n_samples, d)
        bits = torch.full((1, 1, n_samples), b, dtype=torch.int32, device=device)
        ch = ops.quantize_pack(flat, flat, bits, pi_k, pi_v)
        kr = torch.zeros(1, 1, n_samples, d, dtype=torch.float32, device=device)
        vr = torch.zeros_like(kr)
        ops.dequant_chunk_into(ch, pi_k, pi_v, kr, vr, include_exact=False)
        ek = (xf - kr[0, 0]).pow(2).sum(-1).mean().item() / max(x_norm_sq, 1e-12)
        ev = (xf - vr[0, 0]).pow(2).sum(-1).mean().item() / max(x_norm_sq, 1e-12)
        out[b] = (ek + ev) / 2.0
    _epsilon_cache[key] = out
    return out


def optimal_scores_to_bits(scores: torch.Tensor, bit_levels: Sequence[int], target_avg_bits: float, epsilon: dict,
                           sink_mask: Optional[torch.Tensor] = None, sink_bits: int = 16, eviction_cost: float = 5.0,
                           n_outlier: int = 0, head_dim: int = 128, outlier_min_bits: int = 4,
                           above_target_alpha: float = 1.0) -> torch.Tensor:
    """Lagrangian-optimal allocation of one problem (kvquant/allocator.py:459-663).  ``scores`` of any
    shape is flattened; the result has the same shape, int32.  Outlier channels and above-target
    compression of epsilon are not implemented (the reference's experiments leave both off)."""
    if n_outlier > 0:
        raise NotImplementedError("outlier-channel separation is not implemented")
    levels = sorted(set(int(b) for b in bit_levels))
    eps = [float(epsilon.get(b, 0.0)) for b in levels]
    if eviction_cost != 1.0 and levels[0] == 0:
        eps[0] *= eviction_cost
    if above_target_alpha < 1.0:
        below = [b for b in levels if b <= target_avg_bits and b != 0]
        e_t = epsilon.get(int(target_avg_bits), None)
        if e_t is None and below:
            e_t = epsilon.get(below[-1], 0.0)
        if e_t is not None and e_t > 1e-12:
            for k, b in enumerate(levels):
                if b > target_avg_bits:
                    eps[k] = (1.0 - above_target_alpha) * e_t + above_target_alpha * eps[k]
    shape = scores.shape
    flat = scores.reshape(1, -1)
    mask = None if sink_mask is None else sink_mask.reshape(-1)
    bits, rep = ops.allocate_bits(flat, mask, levels, eps, float(target_avg_bits), sink_bits)
    last_report[:] = [rep]
    return bits.reshape(shape)
