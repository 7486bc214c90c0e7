"""Lloyd-Max codebooks for one coordinate of a randomly rotated unit vector (host side, offline).

Same algorithm and constants as the reference's ``codebook.py:36-113`` (``compute_codebook``): the
coordinate density is N(0, 1/d) for d >= 100, truncated at +-5 sigma, integrated on a 10 000-point
grid; centroids start on ``linspace(-3 sigma, 3 sigma, k)`` and iterate conditional means until the
largest change drops below 1e-10 (at most 500 sweeps).  The fp32 cast of the result is what the
kernels receive; it is never symmetrised.
"""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np


def coordinate_pdf(x: np.ndarray, d: int) -> np.ndarray:
    if d < 100:
        raise NotImplementedError("only the Gaussian regime (head_dim >= 100) is supported")
    sigma = 1.0 / np.sqrt(d)
    z = (x - 0) / sigma
    return np.exp(-z ** 2 / 2.0) / np.sqrt(2 * np.pi) / sigma


def compute_codebook(k: int, d: int, n_iter: int = 500, tol: float = 1e-10, x_range: float = 5.0) -> np.ndarray:
    sigma = 1.0 / np.sqrt(d)
    lo_x, hi_x = -x_range * sigma, x_range * sigma
    grid = np.linspace(lo_x, hi_x, 10000)
    step = grid[1] - grid[0]
    dens = coordinate_pdf(grid, d)
    cur = np.linspace(-3 * sigma, 3 * sigma, k)
    nxt = cur
    for _ in range(n_iter):
        srt = np.sort(cur)
        edges = np.concatenate([[lo_x], (srt[:-1] + srt[1:]) / 2, [hi_x]])
        nxt = np.zeros(k)
        for i in range(k):
            cell = (grid >= edges[i]) & (grid < edges[i + 1])
            mass = np.sum(dens[cell]) * step
            nxt[i] = np.sum(grid[cell] * dens[cell]) * step / mass if mass > 0 else srt[i]
        if np.max(np.abs(nxt - cur)) < tol:
            break
        cur = nxt
    return np.sort(nxt)


_CACHE: Dict[Tuple[int, int], np.ndarray] = {}


def codebook_f32(bits: int, d: int = 128) -> np.ndarray:
    key = (bits, d)
    if key not in _CACHE:
        _CACHE[key] = compute_codebook(2 ** bits, d).astype(np.float32)
    return _CACHE[key]
