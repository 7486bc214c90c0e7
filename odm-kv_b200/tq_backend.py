"""Rotation, codebooks and the single-level Lloyd-Max quantiser handle.

Mirrors the parts of the reference's ``kvquant/tq_backend.py`` that the "mse" key and value
quantisers use: ``random_rotation`` (25-36), ``_load_or_compute_codebook`` (39-46), ``MSEQuantized``
(49-52), ``_pack_indices`` / ``_unpack_indices`` (103-145) and ``TurboQuantMSE`` (165-203).
"""
from __future__ import annotations

from typing import NamedTuple, Optional

import torch

from . import ops
from ._lib import HEAD_DIM, QLEVEL_BITS
from .codebook import codebook_f32


def random_rotation(dim: int, device, dtype: torch.dtype, seed: Optional[int] = None) -> torch.Tensor:
    """Q * sign(diag R) of a seeded Gaussian matrix (kvquant/tq_backend.py:25-36).

    The matrix is always drawn with torch's CPU generator and then moved: a CUDA generator would
    yield a different rotation for the same seed, and packed caches must not depend on where they
    were built."""
    key = None
    gen = None
    if seed is not None:
        key = (int(dim), int(seed), str(torch.device(device)), dtype)
        if key in _ROTATIONS:
            return _ROTATIONS[key]
        gen = torch.Generator(device="cpu")
        gen.manual_seed(int(seed))
    mat = torch.randn(dim, dim, dtype=torch.float32, generator=gen)
    q, r = torch.linalg.qr(mat)
    diag = torch.diag(r)
    signs = torch.where(diag >= 0, torch.ones_like(diag), -torch.ones_like(diag))
    rot = (q * signs.unsqueeze(0)).contiguous().to(device=device, dtype=dtype)
    if key is not None:
        _ROTATIONS[key] = rot   # seeded rotations are read-only inputs of the kernels: one copy per (seed, device)
    return rot


_ROTATIONS: dict = {}


def _load_or_compute_codebook(bits: int, dim: int, device, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(codebook_f32(bits, dim)).to(device=device, dtype=dtype)


class MSEQuantized(NamedTuple):
    indices: torch.Tensor   # uint8 [N, bytes] in the reference byte layout
    norms: torch.Tensor     # fp32 [N]
    bits: int


def _pack_indices(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """Reference byte layout: 2-bit -> 4 codes per byte, 3/4-bit -> nibbles, 8-bit -> bytes."""
    if bits == 1:
        per, eff = 8, 1
    elif bits == 2:
        per, eff = 4, 2
    elif bits <= 4:
        per, eff = 2, 4
    else:
        return indices.to(torch.uint8)
    dim = indices.shape[-1]
    pad = (-dim) % per
    idx = indices.to(torch.uint8)
    if pad:
        idx = torch.nn.functional.pad(idx, (0, pad), value=0)
    grouped = idx.reshape(*idx.shape[:-1], -1, per)
    shifts = torch.arange(per, device=idx.device, dtype=torch.uint8) * eff
    return (grouped << shifts).sum(dim=-1, dtype=torch.uint8)


def _unpack_indices(packed: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    if bits == 1:
        per, eff = 8, 1
    elif bits == 2:
        per, eff = 4, 2
    elif bits <= 4:
        per, eff = 2, 4
    else:
        return packed.long()
    shifts = torch.arange(per, device=packed.device, dtype=torch.uint8) * eff
    un = (packed.unsqueeze(-1) >> shifts) & ((1 << eff) - 1)
    return un.reshape(*packed.shape[:-1], -1)[..., :dim].long()


class TurboQuantMSE:
    """One-level quantiser handle (norm, rotate, nearest Lloyd-Max centroid, pack) backed by the CUDA
    kernels.  ``quantize`` returns the reference's ``MSEQuantized`` payload; ``roundtrip`` returns the
    fp32 reconstruction (what ``dequantize(quantize(x))`` yields in the reference)."""

    def __init__(self, dim: int, bits: int, *, device, dtype: torch.dtype, seed: int = 42):
        if dim != HEAD_DIM:
            raise ValueError(f"only head_dim {HEAD_DIM} is supported, got {dim}")
        if bits not in QLEVEL_BITS:
            raise ValueError(f"unsupported bit width {bits}; supported: {QLEVEL_BITS}")
        self.dim, self.bits, self.device, self.dtype = dim, bits, torch.device(device), dtype
        self.compute_dtype = torch.float32
        self.pi = random_rotation(dim, self.device, torch.float32, seed=seed)
        self.centroids = _load_or_compute_codebook(bits, dim, self.device, torch.float32)

    def _pack(self, x: torch.Tensor) -> ops.PackedChunk:
        flat = x.reshape(1, 1, -1, self.dim).contiguous()
        bits = torch.full(flat.shape[:3], self.bits, dtype=torch.int32, device=flat.device)
        return ops.quantize_pack(flat, flat, bits, self.pi, self.pi)

    def quantize(self, x: torch.Tensor) -> MSEQuantized:
        ch = self._pack(x)
        _, ik, nk, _, _ = ops.export_bank(ch, self.bits)
        lead = x.shape[:-1]
        return MSEQuantized(indices=ik.reshape(*lead, -1), norms=nk.reshape(lead), bits=self.bits)

    def roundtrip(self, x: torch.Tensor) -> torch.Tensor:
        ch = self._pack(x)
        n = x.reshape(-1, self.dim).shape[0]
        out = torch.zeros(1, 1, n, self.dim, dtype=torch.float32, device=x.device)
        scratch = torch.zeros_like(out)
        ops.dequant_chunk_into(ch, self.pi, self.pi, out, scratch, include_exact=False)
        return out.reshape(*x.shape[:-1], self.dim)
