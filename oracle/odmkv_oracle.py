"""TEST INFRASTRUCTURE ONLY -- CPU oracle for the ODM-KV compress-then-decode path.

A numpy (plus one small C file, ``rotquant.c``) restatement of what the reference
computes on its CPU torch path, stage by stage.  Every function cites the reference
site it follows (paths are relative to the reference project root).

Only ``tests/``, the smoke check and the CPU-baseline leg of ``bench.py`` may import
this module.  The product never does: its kernels fail loudly when the CUDA library
is missing.

Parity status: the reference ships no tests or golden vectors, and the module that
defines its nearest-centroid tie rule (``kvquant/tq_triton.py``) is absent from its
tree.  This oracle is pinned against fixtures produced by running the reference
itself on CPU (``tests/golden/make_golden.py``), with a stand-in for the missing
module that follows the comment at ``kvquant/tq_backend.py:191-196``; for coordinates
that sit exactly on a Voronoi midpoint the rule "lower index wins" is a choice, so
parity is unpinned for those (their count is recorded in the fixtures).

Conventions: all inputs are fp32 copies of the fp16/bf16 tensors (the reference run
on fp32-upcast inputs), all arithmetic is fp32 unless stated.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_C_SRC = os.path.join(_HERE, "rotquant.c")
_C_LIB = os.path.join(_HERE, "liboracle_rotquant.so")
_clib = None

f32 = np.float32


# ---------------------------------------------------------------------------
# C helper (rotation + nearest centroid with a fixed FMA chain)
# ---------------------------------------------------------------------------

def build_c(force: bool = False) -> str:
    """Compile rotquant.c with gcc (no contraction besides the explicit fmaf)."""
    if force or not os.path.exists(_C_LIB) or os.path.getmtime(_C_LIB) < os.path.getmtime(_C_SRC):
        subprocess.check_call([
            "gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-mfma", "-o", _C_LIB, _C_SRC, "-lm",
        ])
    return _C_LIB


def _c():
    global _clib
    if _clib is None:
        _clib = ctypes.CDLL(build_c())
        P = ctypes.c_void_p
        _clib.oracle_quantize.argtypes = [P, ctypes.c_int64, ctypes.c_int, P, P, ctypes.c_int, P, P, P]
        _clib.oracle_quantize.restype = None
        _clib.oracle_encode.argtypes = [P, ctypes.c_int64, P, ctypes.c_int, P]
        _clib.oracle_encode.restype = None
        _clib.oracle_dequantize.argtypes = [P, P, ctypes.c_int64, ctypes.c_int, P, P, P]
        _clib.oracle_dequantize.restype = None
    return _clib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


# ---------------------------------------------------------------------------
# Codebook (codebook.py:14-113) and rotation (kvquant/tq_backend.py:25-36)
# ---------------------------------------------------------------------------

def _coord_pdf(x: np.ndarray, d: int) -> np.ndarray:
    """N(0, 1/d) density, written the way scipy evaluates norm.pdf (codebook.py:22-25)."""
    if d < 100:
        raise NotImplementedError("oracle covers head_dim >= 100 (Gaussian branch) only")
    std = 1.0 / np.sqrt(d)
    z = (x - 0) / std
    return np.exp(-z ** 2 / 2.0) / np.sqrt(2 * np.pi) / std


def compute_codebook(k: int, d: int, n_iter: int = 500, tol: float = 1e-10, x_range: float = 5.0) -> np.ndarray:
    """Lloyd-Max centroids for one rotated coordinate (codebook.py:36-113)."""
    std = 1.0 / np.sqrt(d)
    x_min, x_max = -x_range * std, x_range * std
    centroids = np.linspace(-3 * std, 3 * std, k)
    new_centroids = centroids
    for _ in range(n_iter):
        c = np.sort(centroids)
        boundaries = np.concatenate([[x_min], (c[:-1] + c[1:]) / 2, [x_max]])
        x = np.linspace(x_min, x_max, 10000)
        dx = x[1] - x[0]
        px = _coord_pdf(x, d)
        new_centroids = np.zeros(k)
        for i in range(k):
            lo, hi = boundaries[i], boundaries[i + 1]
            mask = (x >= lo) & (x < hi)
            mass = np.sum(px[mask]) * dx
            new_centroids[i] = np.sum(x[mask] * px[mask]) * dx / mass if mass > 0 else c[i]
        if np.max(np.abs(new_centroids - centroids)) < tol:
            break
        centroids = new_centroids
    return np.sort(new_centroids)


_CB_CACHE: Dict[Tuple[int, int], np.ndarray] = {}


def codebook_f32(bits: int, d: int = 128) -> np.ndarray:
    """fp32 centroids as the quantiser holds them (kvquant/tq_backend.py:39-46)."""
    key = (bits, d)
    if key not in _CB_CACHE:
        _CB_CACHE[key] = compute_codebook(2 ** bits, d).astype(np.float32)
    return _CB_CACHE[key]


def random_rotation(dim: int, seed: int) -> np.ndarray:
    """Q * sign(diag R) of a seeded CPU Gaussian matrix (kvquant/tq_backend.py:25-36).

    torch is used because the reference draws from torch's CPU generator and factors
    with torch.linalg.qr; the same matrix is handed to both sides of every comparison.
    """
    import torch

    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    mat = torch.randn(dim, dim, dtype=torch.float32, generator=gen)
    q, r = torch.linalg.qr(mat)
    diag = torch.diag(r)
    signs = torch.where(diag >= 0, torch.ones_like(diag), -torch.ones_like(diag))
    return np.ascontiguousarray((q * signs.unsqueeze(0)).numpy(), dtype=np.float32)


# ---------------------------------------------------------------------------
# Quantiser (kvquant/tq_backend.py:103-145, 185-203)
# ---------------------------------------------------------------------------

def quantize(x: np.ndarray, pi: np.ndarray, cent: np.ndarray, return_y: bool = False):
    """norm, normalise, rotate, nearest centroid (kvquant/tq_backend.py:185-197).

    Returns (idx uint8 [n, d], norms fp32 [n]) and optionally the rotated coordinates.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, d = x.shape
    pi = np.ascontiguousarray(pi, dtype=np.float32)
    cent = np.ascontiguousarray(cent, dtype=np.float32)
    idx = np.empty((n, d), dtype=np.uint8)
    norms = np.empty((n,), dtype=np.float32)
    y = np.empty((n, d), dtype=np.float32) if return_y else None
    _c().oracle_quantize(_ptr(x), n, d, _ptr(pi), _ptr(cent), int(cent.shape[0]), _ptr(idx), _ptr(norms),
                         _ptr(y) if return_y else None)
    return (idx, norms, y) if return_y else (idx, norms)


def encode(y: np.ndarray, cent: np.ndarray) -> np.ndarray:
    """Nearest centroid of given rotated coordinates (the stand-in for kvquant/tq_triton.py)."""
    y = np.ascontiguousarray(y, dtype=np.float32)
    cent = np.ascontiguousarray(cent, dtype=np.float32)
    idx = np.empty(y.shape, dtype=np.uint8)
    _c().oracle_encode(_ptr(y), y.size, _ptr(cent), int(cent.shape[0]), _ptr(idx))
    return idx


def dequantize(idx: np.ndarray, norms: np.ndarray, pi: np.ndarray, cent: np.ndarray) -> np.ndarray:
    """centroid gather, inverse rotation, rescale (kvquant/tq_backend.py:199-203); fp32 result."""
    idx = np.ascontiguousarray(idx, dtype=np.uint8)
    n, d = idx.shape
    norms = np.ascontiguousarray(norms, dtype=np.float32)
    pi = np.ascontiguousarray(pi, dtype=np.float32)
    cent = np.ascontiguousarray(cent, dtype=np.float32)
    out = np.empty((n, d), dtype=np.float32)
    _c().oracle_dequantize(_ptr(idx), _ptr(norms), n, d, _ptr(pi), _ptr(cent), _ptr(out))
    return out


def pack_indices(idx: np.ndarray, bits: int) -> np.ndarray:
    """Reference byte layout (kvquant/tq_backend.py:103-125): 2-bit -> 4 codes per byte,
    3- and 4-bit -> two nibbles per byte, 8-bit -> one byte per code; little-endian in the byte."""
    idx = idx.astype(np.uint8)
    if bits == 2:
        per, eff = 4, 2
    elif bits in (3, 4):
        per, eff = 2, 4
    elif bits == 1:
        per, eff = 8, 1
    else:
        return idx.copy()
    n, d = idx.shape
    r = idx.reshape(n, d // per, per).astype(np.uint32)
    shifts = (np.arange(per, dtype=np.uint32) * eff)
    return (r << shifts).sum(axis=-1).astype(np.uint8)


def unpack_indices(packed: np.ndarray, bits: int, dim: int) -> np.ndarray:
    """Inverse of pack_indices (kvquant/tq_backend.py:128-145)."""
    if bits == 2:
        per, eff = 4, 2
    elif bits in (3, 4):
        per, eff = 2, 4
    elif bits == 1:
        per, eff = 8, 1
    else:
        return packed.astype(np.uint8)
    shifts = (np.arange(per, dtype=np.uint8) * eff)
    un = (packed[..., None] >> shifts) & ((1 << eff) - 1)
    return un.reshape(*packed.shape[:-1], -1)[..., :dim].astype(np.uint8)


# ---------------------------------------------------------------------------
# Scorer (kvquant/scorer.py:285-325, 363-416; kvquant/attention_utils.py:19-115)
# ---------------------------------------------------------------------------

def avg_rope_vectors(cos: np.ndarray, sin: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Mean cos / sin rows over the future positions (kvquant/attention_utils.py:87-104)."""
    return cos.astype(f32).mean(axis=0, dtype=f32), sin.astype(f32).mean(axis=0, dtype=f32)


def apply_avg_rope(mu: np.ndarray, cos_bar: Optional[np.ndarray], sin_bar: Optional[np.ndarray]) -> np.ndarray:
    """mu' = R mu with R = mean_p(diag(cos_p) + diag(sin_p) perm) (kvquant/attention_utils.py:94-108).

    Written in its elementwise form: mu'_i = cos_bar_i mu_i + sin_bar_i rotate_half(mu)_i."""
    if cos_bar is None:
        return mu.astype(f32)
    half = mu.shape[-1] // 2
    rot = np.concatenate([-mu[..., half:], mu[..., :half]], axis=-1)
    return (cos_bar * mu + sin_bar * rot).astype(f32)


def mean_query(hidden: np.ndarray, wq: np.ndarray, bq: Optional[np.ndarray], num_heads: int, head_dim: int,
               n_sink: int = 4) -> np.ndarray:
    """mu = mean over prompt positions after the sinks of q_proj(h) (kvquant/scorer.py:184-195,
    kvquant/attention_utils.py:29-54).  hidden [T, hidden], wq [Hq*d, hidden]; returns [Hq, d]."""
    h = hidden[n_sink:].astype(f32)
    q = h @ wq.astype(f32).T
    if bq is not None:
        q = q + bq.astype(f32)
    q = q.reshape(h.shape[0], num_heads, head_dim)
    return q.mean(axis=0, dtype=f32)


def attention_p(K: np.ndarray, mu: np.ndarray, n_sink: int = 4) -> np.ndarray:
    """GQA-mean softmax of the mean query over the core positions (kvquant/scorer.py:302-315).
    K [H, T, d], mu [Hq, d]; returns p [H, T - n_sink]."""
    H, T, d = K.shape
    Hq = mu.shape[0]
    G = Hq // H
    Kc = K[:, n_sink:].astype(f32)
    logits = np.einsum("hgd,htd->hgt", mu.reshape(H, G, d).astype(f32), Kc).astype(f32) / f32(math.sqrt(d))
    m = logits.max(axis=-1, keepdims=True)
    e = np.exp(logits - m, dtype=f32)
    sm = e / e.sum(axis=-1, keepdims=True, dtype=f32)
    return sm.mean(axis=1, dtype=f32)


def risk_from_p(K: np.ndarray, V: np.ndarray, p: np.ndarray, eps: float) -> np.ndarray:
    """s = (p + eps)^2 (|v|^2 + |k|^2/d |v - o|^2) given p (kvquant/scorer.py:394-403, 406-416)."""
    K = K.astype(f32)
    V = V.astype(f32)
    d = K.shape[-1]
    p = p.astype(f32)
    p_norm = p / np.maximum(p.sum(axis=-1, keepdims=True, dtype=f32), f32(1e-8))
    o = np.einsum("ht,htd->hd", p_norm, V).astype(f32)
    irrep = ((V - o[:, None, :]) ** 2).sum(axis=-1, dtype=f32)
    kn2 = (K ** 2).sum(axis=-1, dtype=f32)
    vn2 = (V ** 2).sum(axis=-1, dtype=f32)
    return ((p + f32(eps)) ** 2 * (vn2 + (kn2 / f32(d)) * irrep)).astype(f32)


def score_prefill(K: np.ndarray, V: np.ndarray, mu: np.ndarray, n_sink: int = 4, eps: float = 1e-2) -> np.ndarray:
    """RiskScorer.score_prefill with normalize_grain "global" (kvquant/scorer.py:385-404, 321-325).

    K, V [H, T, d]; mu [Hq, d] is the (averaged-RoPE'd) mean query.  Returns s [H, T] fp32 with the
    sink slots set to the maximum over the whole core tensor."""
    H, T, _ = K.shape
    if T <= n_sink:
        return np.ones((H, T), dtype=f32)
    p = attention_p(K, mu, n_sink)
    s = risk_from_p(K[:, n_sink:], V[:, n_sink:], p, eps)
    out = np.empty((H, T), dtype=f32)
    out[:, :n_sink] = s.max()
    out[:, n_sink:] = s
    return out


def score_with_attn(K: np.ndarray, V: np.ndarray, p: np.ndarray, eps: float = 1e-2) -> np.ndarray:
    """RiskScorer.score_with_attn (kvquant/scorer.py:406-416)."""
    return risk_from_p(K, V, p, eps)


def chunked_attention_qk(Q: np.ndarray, K: np.ndarray, scale: float, q_offset: int = 0):
    """_chunked_attention_qk (kvquant/attention_utils.py:160-211) in fp32, without the chunking (which only bounds the
    reference's temporaries): Q [Hq, Tq, d], K [H, Tkv, d] -> (sum_attn, max_attn, sum_sq_attn), each [H, Tkv].
    logits = q.k / scale (184), keys with q_pos < k_pos hidden (187-190; here k_pos > q_pos + q_offset), softmax over
    the keys (192), mean over the G query heads of a KV head (195), then sum / max / sum of squares over the queries
    (199-205)."""
    Q = np.asarray(Q, np.float32)
    K = np.asarray(K, np.float32)
    Hq, Tq, _ = Q.shape
    H, Tkv, _ = K.shape
    G = Hq // H
    s_sum = np.zeros((H, Tkv), np.float32)
    s_max = np.zeros((H, Tkv), np.float32)
    s_sq = np.zeros((H, Tkv), np.float32)
    hidden = np.arange(Tkv)[None, :] > (np.arange(Tq)[:, None] + q_offset)           # [Tq, Tkv]
    for h in range(H):
        logits = np.einsum("gqd,kd->gqk", Q[h * G:(h + 1) * G], K[h]).astype(np.float32) / np.float32(scale)
        logits[:, hidden] = -np.inf
        logits -= logits.max(axis=-1, keepdims=True)
        w = np.exp(logits, dtype=np.float32)
        w /= w.sum(axis=-1, keepdims=True, dtype=np.float32)
        m = w.mean(axis=0, dtype=np.float32)                                           # [Tq, Tkv]
        s_sum[h] = m.sum(axis=0, dtype=np.float32)
        s_max[h] = m.max(axis=0)
        s_sq[h] = (m * m).sum(axis=0, dtype=np.float32)
    return s_sum, s_max, s_sq


# ---------------------------------------------------------------------------
# Allocator (kvquant/allocator.py:46-148, 333-342, 352-452, 459-663)
# ---------------------------------------------------------------------------

def calibrate_epsilon(d: int, bit_levels: Sequence[int], seed: int = 42, n_samples: int = 4096) -> Dict[int, float]:
    """Relative MSE of key+value quantisers per level (kvquant/allocator.py:352-452, "mse" values).

    Uses this oracle's quantiser, so values agree with the reference to rounding only."""
    import torch

    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    x = torch.randn(n_samples, d, generator=gen).to(torch.float16).float().numpy()
    x_norm_sq = float((x.astype(f32) ** 2).sum(-1, dtype=f32).mean(dtype=f32))
    out: Dict[int, float] = {}
    for b in sorted(set(int(v) for v in bit_levels)):
        if b == 0:
            out[0] = 1.0
            continue
        if b >= 16:
            out[b] = 0.0
            continue
        cent = codebook_f32(b, d)
        errs = []
        for s in (seed, seed + 2000):
            pi = random_rotation(d, s)
            idx, norms = quantize(x, pi, cent)
            rec = dequantize(idx, norms, pi, cent)
            errs.append(float(((x - rec) ** 2).sum(-1, dtype=f32).mean(dtype=f32)) / max(x_norm_sq, 1e-12))
        out[b] = (errs[0] + errs[1]) / 2.0
    return out


@dataclass
class AllocInfo:
    evaluations: int = 0
    lam: float = 0.0
    gap_before: float = 0.0
    moved: int = 0
    ties_lambda: int = 0
    ties_cut: int = 0


def optimal_scores_to_bits(scores: np.ndarray, bit_levels: Sequence[int], target_avg_bits: float,
                           epsilon: Dict[int, float], sink_mask: Optional[np.ndarray] = None, sink_bits: int = 16,
                           eviction_cost: float = 5.0, info: Optional[AllocInfo] = None) -> np.ndarray:
    """Per-layer Lagrangian allocation with gap closure (kvquant/allocator.py:459-663), OCS off,
    above_target_alpha = 1.  Returns int32 bits of the input shape."""
    levels = sorted(set(int(b) for b in bit_levels))
    shape = scores.shape
    flat = scores.reshape(-1).astype(f32)
    n = flat.shape[0]
    result = np.empty(n, dtype=np.int32)
    if sink_mask is not None:
        fs = sink_mask.reshape(-1).astype(bool)
        result[fs] = sink_bits
        non_sink = ~fs
    else:
        non_sink = np.ones(n, dtype=bool)
    idx = np.nonzero(non_sink)[0]
    n_active = idx.shape[0]
    if n_active == 0:
        return result.reshape(shape)
    target = max(float(levels[0]), min(float(levels[-1]), float(target_avg_bits)))
    if len(levels) == 1:
        result[idx] = levels[0]
        return result.reshape(shape)

    s = flat[idx]
    # sanitise (allocator.py:543-547)
    s = np.maximum(s, f32(0.0))  # note: propagates nan like torch.clamp
    finite = np.isfinite(s)
    if finite.any() and not finite.all():
        s = np.where(finite, s, s[finite].max())
    s = np.nan_to_num(s, nan=0.0, posinf=np.finfo(f32).max, neginf=np.finfo(f32).min).astype(f32)

    K = len(levels)
    eps_raw = [float(epsilon.get(b, 0.0)) for b in levels]
    if eviction_cost != 1.0 and levels[0] == 0:
        eps_raw[0] *= eviction_cost
    eps_t = np.array(eps_raw, dtype=f32)
    bits_t = np.array([float(b) for b in levels], dtype=f32)
    nominal = np.array(levels, dtype=np.int32)
    counter = [0]

    def assign(lam: float):
        counter[0] += 1
        lam32 = f32(lam)
        best = (s * eps_t[0]).astype(f32) + f32(lam32 * bits_t[0])
        chosen = np.zeros(n_active, dtype=np.int64)
        for k in range(1, K):
            cost = (s * eps_t[k]).astype(f32) + f32(lam32 * bits_t[k])
            better = cost < best  # strict: first minimum wins
            chosen[better] = k
            best = np.where(better, cost, best)
        total = f32(bits_t[chosen].astype(np.float64).sum())  # exact integer < 2^24
        avg = float(f32(total) / f32(n_active))
        return chosen, avg

    lo, hi = 0.0, 1.0
    _, avg_hi = assign(hi)
    while avg_hi > target and hi < 1e8:
        hi *= 10.0
        _, avg_hi = assign(hi)
    for _ in range(64):
        mid = (lo + hi) * 0.5
        _, avg = assign(mid)
        if avg > target:
            lo = mid
        else:
            hi = mid
    lam_final = (lo + hi) * 0.5
    chosen, avg = assign(lam_final)

    nom = nominal[chosen].copy()
    gap = (avg - target) * n_active
    moved = 0
    ties_cut = 0
    gap0 = gap
    if abs(gap) > 0.5:
        order = np.argsort(s, kind="stable")
        nom_o = nom[order]
        s_o = s[order]
        if gap > 0:
            for i in range(K - 1):
                delta = float(levels[i + 1] - levels[i])
                at_hi = nom_o == levels[i + 1]
                n_dem = min(int(at_hi.sum()), int(gap / delta + 0.5))
                if n_dem <= 0:
                    continue
                pos = np.nonzero(at_hi)[0]
                sel = pos[:n_dem]
                if n_dem < pos.shape[0] and s_o[pos[n_dem]] == s_o[sel[-1]]:
                    ties_cut += 1
                nom_o[sel] = levels[i]
                moved += n_dem
                gap -= n_dem * delta
                if gap <= 0.5:
                    break
        else:
            gap = -gap
            for i in range(K - 2, -1, -1):
                delta = float(levels[i + 1] - levels[i])
                at_lo = nom_o == levels[i]
                n_pro = min(int(at_lo.sum()), int(gap / delta + 0.5))
                if n_pro <= 0:
                    continue
                pos = np.nonzero(at_lo)[0]
                sel = pos[pos.shape[0] - n_pro:]
                if n_pro < pos.shape[0] and s_o[pos[pos.shape[0] - n_pro - 1]] == s_o[sel[0]]:
                    ties_cut += 1
                nom_o[sel] = levels[i + 1]
                moved += n_pro
                gap -= n_pro * delta
                if gap <= 0.5:
                    break
        nom = np.empty_like(nom_o)
        nom[order] = nom_o
    if info is not None:
        info.evaluations = counter[0]
        info.lam = lam_final
        info.gap_before = gap0
        info.moved = moved
        info.ties_cut = ties_cut
        lam32 = f32(lam_final)
        ties = 0
        for a in range(K - 1):
            ca = (s * eps_t[a]).astype(f32) + f32(lam32 * bits_t[a])
            cb = (s * eps_t[a + 1]).astype(f32) + f32(lam32 * bits_t[a + 1])
            on_hull = (chosen == a) | (chosen == a + 1)
            ties += int((np.abs(ca.astype(np.float64) - cb.astype(np.float64))[on_hull] < 1e-6).sum())
        info.ties_lambda = ties
    result[idx] = nom.astype(np.int32)
    return result.reshape(shape)


def ratio_scores_to_bits(scores: np.ndarray, bit_levels: Sequence[int], ratios: Sequence[float]) -> np.ndarray:
    """Rank-tier allocation of one flat score vector (kvquant/allocator.py:108-148, no sink mask).

    Python round() (banker's rounding) sizes every tier but the last, which takes the remainder."""
    flat = scores.reshape(-1).astype(f32)
    n = flat.shape[0]
    r = np.array(ratios, dtype=np.float64)
    r = r / r.sum()
    order = np.argsort(flat, kind="stable")
    bits = np.empty(n, dtype=np.int32)
    levels = sorted(zip([int(b) for b in bit_levels], r.tolist()), key=lambda t: t[0])
    cursor = 0
    for i, (b, rr) in enumerate(levels):
        count = n - cursor if i == len(levels) - 1 else min(int(round(rr * n)), n - cursor)
        bits[order[cursor:cursor + count]] = b
        cursor += count
    return bits.reshape(scores.shape)


# ---------------------------------------------------------------------------
# Adaptive state: routing into per-level banks (kvquant/tq_adaptive_backend.py:31-541)
# ---------------------------------------------------------------------------

@dataclass
class Bank:
    positions: np.ndarray  # int64 [N, 3] rows (b, h, t) in row-major nonzero order
    k_idx: np.ndarray      # uint8 [N, d] unpacked codes
    k_norm: np.ndarray     # fp32 [N]
    v_idx: np.ndarray
    v_norm: np.ndarray


@dataclass
class State:
    head_dim: int
    levels: Tuple[int, ...]
    seed: int
    batch: int = 0
    heads: int = 0
    seq_len: int = 0
    banks: Dict[int, Bank] = field(default_factory=dict)
    exact_pos: Optional[np.ndarray] = None
    exact_k: Optional[np.ndarray] = None   # values as stored in the cache dtype, held as fp32
    exact_v: Optional[np.ndarray] = None
    masked: Optional[np.ndarray] = None
    pi_k: Optional[np.ndarray] = None
    pi_v: Optional[np.ndarray] = None


def state_prefill(K: np.ndarray, V: np.ndarray, bits: np.ndarray, levels: Sequence[int], seed: int,
                  pi_k: Optional[np.ndarray] = None, pi_v: Optional[np.ndarray] = None) -> State:
    """TurboQuantAdaptiveKVCacheState.prefill (kvquant/tq_adaptive_backend.py:346-374) with "mse"
    key and value quantisers: key rotation seed = seed, value rotation seed = seed + 2000
    (kvquant/tq_adaptive_backend.py:115-133).  K, V [B, H, T, d] fp32 copies of the cache tensors."""
    B, H, T, d = K.shape
    st = State(head_dim=d, levels=tuple(sorted(set(int(x) for x in levels))), seed=seed, batch=B, heads=H, seq_len=T)
    st.pi_k = random_rotation(d, seed) if pi_k is None else pi_k
    st.pi_v = random_rotation(d, seed + 2000) if pi_v is None else pi_v
    for level in st.levels:
        mask = bits == level
        pos = np.argwhere(mask).astype(np.int64)  # row-major (b, h, t), like torch.nonzero
        if level == 0:
            st.masked = pos
            continue
        kk = K[pos[:, 0], pos[:, 1], pos[:, 2]]
        vv = V[pos[:, 0], pos[:, 1], pos[:, 2]]
        if level == 16:
            st.exact_pos, st.exact_k, st.exact_v = pos, kk.astype(f32), vv.astype(f32)
            continue
        cent = codebook_f32(level, d)
        if pos.shape[0] == 0:
            z8 = np.zeros((0, d), np.uint8)
            st.banks[level] = Bank(pos, z8, np.zeros(0, f32), z8.copy(), np.zeros(0, f32))
            continue
        ki, kn = quantize(kk, st.pi_k, cent)
        vi, vn = quantize(vv, st.pi_v, cent)
        st.banks[level] = Bank(pos, ki, kn, vi, vn)
    if st.masked is None:
        st.masked = np.zeros((0, 3), np.int64)
    return st


def materialize(st: State) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Dense fp32 K_hat, V_hat before the cast to the cache dtype, and the keep mask
    (kvquant/tq_adaptive_backend.py:439-452, 205-242, 66-71).  Evicted rows are zero and not kept."""
    B, H, T, d = st.batch, st.heads, st.seq_len, st.head_dim
    Kh = np.zeros((B, H, T, d), f32)
    Vh = np.zeros((B, H, T, d), f32)
    keep = np.zeros((B, H, T), bool)
    if st.exact_pos is not None and st.exact_pos.shape[0]:
        p = st.exact_pos
        Kh[p[:, 0], p[:, 1], p[:, 2]] = st.exact_k
        Vh[p[:, 0], p[:, 1], p[:, 2]] = st.exact_v
        keep[p[:, 0], p[:, 1], p[:, 2]] = True
    for level, bank in st.banks.items():
        if bank.positions.shape[0] == 0:
            continue
        cent = codebook_f32(level, d)
        p = bank.positions
        Kh[p[:, 0], p[:, 1], p[:, 2]] = dequantize(bank.k_idx, bank.k_norm, st.pi_k, cent)
        Vh[p[:, 0], p[:, 1], p[:, 2]] = dequantize(bank.v_idx, bank.v_norm, st.pi_v, cent)
        keep[p[:, 0], p[:, 1], p[:, 2]] = True
    return Kh, Vh, keep


def decode_attention(q: np.ndarray, Kh: np.ndarray, Vh: np.ndarray, keep: np.ndarray,
                     scale: Optional[float] = None) -> np.ndarray:
    """Dense fp32 softmax(q K_hat^T scale) V_hat with evicted positions excluded -- what the
    reference's decode step computes over its dequantised cache with the fake-key mask
    (kvquant/attention_patch.py:30-55).  q [B, Hq, d]; returns [B, Hq, d] fp32."""
    B, H, T, d = Kh.shape
    Hq = q.shape[1]
    G = Hq // H
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = np.zeros((B, Hq, d), f32)
    for b in range(B):
        for h in range(H):
            qq = q[b, h * G:(h + 1) * G].astype(f32)
            logits = (qq @ Kh[b, h].T).astype(f32) * f32(scale)
            logits = np.where(keep[b, h][None, :], logits, -np.inf).astype(f32)
            m = logits.max(axis=-1, keepdims=True)
            e = np.exp(logits - m, dtype=f32)
            p = e / e.sum(axis=-1, keepdims=True, dtype=f32)
            out[b, h * G:(h + 1) * G] = (p @ Vh[b, h]).astype(f32)
    return out


# ---------------------------------------------------------------------------
# Synthetic inputs (the "config 0" generator: outlier key channels + attention sinks)
# ---------------------------------------------------------------------------

def synth_inputs(H: int, T: int, G: int, d: int = 128, window: int = 64, seed: int = 0, B: int = 1):
    """Seeded fp16 K, V, window queries and a decode query with four x10 key channels and four
    attention-sink tokens worth about +8 logits.  Drawn with torch's CPU generator in a fixed order.
    Returns fp16 numpy arrays: K, V [B, H, T, d], Qw [B, H*G, window, d], qd [B, H*G, d]."""
    import torch

    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    K = torch.randn(B, H, T, d, generator=g)
    V = torch.randn(B, H, T, d, generator=g)
    Qw = torch.randn(B, H * G, window, d, generator=g)
    e = torch.randn(d, generator=g)
    e = e / e.norm()
    qd = torch.randn(B, H * G, d, generator=g)
    K[..., 0:4] *= 10.0
    Qw = Qw + 3.0 * e
    qd = qd + 3.0 * e
    K[:, :, 0:4, :] += (8.0 * math.sqrt(d) / 3.0) * e
    return (K.half().numpy(), V.half().numpy(), Qw.half().numpy(), qd.half().numpy())
