"""Tensor-level wrappers over the C ABI: torch owns the memory and the stream, the kernels do the work.

Every function takes CUDA tensors and enqueues on ``torch.cuda.current_stream()``.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import (CLASS_BITS, CODE_BYTES, HEAD_DIM, NUM_CLASSES, NUM_QLEVELS, QLEVEL_BITS, REF_CODE_BYTES, AllocReport,
                   Chunk, OdmkvError, check, dtype_code, lib, ptr, require_cuda, stream_ptr)
from .codebook import codebook_f32


def _rot(pi: torch.Tensor, device) -> torch.Tensor:
    """Rotation matrices reach the kernels as row-major fp32 (torch.linalg.qr may hand back a
    column-major tensor, whose data pointer would otherwise be read as the transpose)."""
    if pi.shape != (HEAD_DIM, HEAD_DIM):
        raise ValueError(f"rotation must be [{HEAD_DIM}, {HEAD_DIM}], got {tuple(pi.shape)}")
    return pi.to(device=device, dtype=torch.float32).contiguous()


def _ws(nbytes: int, device) -> torch.Tensor:
    # torch's caching allocator returns 512-byte aligned blocks
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


_CB_TABLES: dict = {}


def codebook_table(device, dim: int = HEAD_DIM) -> torch.Tensor:
    """[4, 256] fp32: row li holds the 2^bits(li) ascending Lloyd-Max centroids of level li."""
    key = (str(device), dim)
    if key not in _CB_TABLES:
        tab = np.zeros((NUM_QLEVELS, 256), np.float32)
        for li, b in enumerate(QLEVEL_BITS):
            tab[li, : 2 ** b] = codebook_f32(b, dim)
        _CB_TABLES[key] = torch.from_numpy(tab).to(device)
    return _CB_TABLES[key]


# ---------------------------------------------------------------------------------------------
# scorer
# ---------------------------------------------------------------------------------------------

def score_prefill(K: torch.Tensor, V: torch.Tensor, mu: torch.Tensor, n_sink: int = 4, eps: float = 1e-2,
                  check_status: bool = False, return_status: bool = False):
    """K, V [B, H, T, 128] (fp16/bf16/fp32), mu [B, H*G, 128] fp32 -> scores [B, H, T] fp32.
    ``check_status`` synchronises and raises if a sweep reported an expired wait on one of its bulk copies;
    ``return_status`` returns ``(scores, status)`` instead, ``status`` a one-element int32 device tensor (0 = clean)
    that the caller can read at a point where it synchronises anyway."""
    require_cuda(K, "keys")
    if K.shape != V.shape or K.dim() != 4 or K.shape[-1] != HEAD_DIM:
        raise ValueError(f"expected keys/values [B, H, T, {HEAD_DIM}], got {tuple(K.shape)} / {tuple(V.shape)}")
    B, H, T, _ = K.shape
    if mu.dim() != 3 or mu.shape[0] != B or mu.shape[1] % H != 0 or mu.shape[2] != HEAD_DIM:
        raise ValueError(f"expected mean query [B, H*G, {HEAD_DIM}], got {tuple(mu.shape)}")
    G = mu.shape[1] // H
    K, V = K.contiguous(), V.contiguous()
    if K.data_ptr() % 16:   # the sweeps stream rows with bulk copies, which need 16-byte aligned sources
        K = K.clone()
    if V.data_ptr() % 16:
        V = V.clone()
    mu = mu.to(device=K.device, dtype=torch.float32).contiguous()
    scores = torch.empty(B, H, T, dtype=torch.float32, device=K.device)
    nbytes = lib().odmkv_score_workspace_bytes(B, H, G, T)
    ws = _ws(nbytes, K.device)
    check(lib().odmkv_score_prefill(ptr(K), ptr(V), dtype_code(K.dtype), ptr(mu), B, H, G, T, int(n_sink), float(eps),
                                    ptr(scores), ptr(ws), ws.numel(), stream_ptr(K.device)), "odmkv_score_prefill")
    status = None
    if T > n_sink:
        off = lib().odmkv_score_status_offset(B, H, G, T, int(n_sink))
        status = ws[off:off + 4].view(torch.int32)
        if check_status and int(status.item()) != 0:
            raise OdmkvError("odmkv_score_prefill: a bounded wait on a bulk copy expired; the scores are invalid")
    return (scores, status) if return_status else scores


def score_with_attn(K: torch.Tensor, V: torch.Tensor, p: torch.Tensor, eps: float = 1e-2) -> torch.Tensor:
    """K, V [R, T, 128], p [R, T] -> [R, T] fp32 (risk formula with given attention weights)."""
    require_cuda(K, "keys")
    R, T, _ = K.shape
    K, V = K.contiguous(), V.contiguous()
    p = p.to(torch.float32).contiguous()
    out = torch.empty(R, T, dtype=torch.float32, device=K.device)
    check(lib().odmkv_score_with_attn(ptr(K), ptr(V), dtype_code(K.dtype), ptr(p), R, T, float(eps), ptr(out),
                                      stream_ptr(K.device)), "odmkv_score_with_attn")
    return out


def window_attn_stats(Q: torch.Tensor, K: torch.Tensor, scale: Optional[float] = None, q_offset: int = 0,
                      check_status: bool = True):
    """Q [B, H*G, Tq, 128], K [B, H, Tkv, 128] (fp16 / bf16) -> (sum_attn, max_attn, sum_sq_attn), each [B, H, Tkv] fp32:
    per key the sum / maximum / sum of squares over the queries of the head-averaged causal softmax weight (key j is
    hidden from query r when j > r + q_offset).  ``check_status`` synchronises and raises if a bounded wait expired."""
    require_cuda(Q, "queries")
    if Q.dim() != 4 or K.dim() != 4 or Q.shape[-1] != HEAD_DIM or K.shape[-1] != HEAD_DIM or Q.shape[0] != K.shape[0]:
        raise ValueError(f"expected queries [B, Hq, Tq, {HEAD_DIM}] and keys [B, H, Tkv, {HEAD_DIM}], got {tuple(Q.shape)} / {tuple(K.shape)}")
    if Q.dtype not in (torch.float16, torch.bfloat16) or K.dtype != Q.dtype:
        raise NotImplementedError("window_attn_stats takes fp16 or bf16 queries and keys of one dtype")
    B, Hq, Tq, _ = Q.shape
    H, Tkv = K.shape[1], K.shape[2]
    if Hq % H:
        raise ValueError(f"query heads {Hq} not a multiple of KV heads {H}")
    G = Hq // H
    Q, K = Q.contiguous(), K.contiguous()
    if Q.data_ptr() % 16:
        Q = Q.clone()
    if K.data_ptr() % 16:
        K = K.clone()
    dev = Q.device
    outs = [torch.empty(B, H, Tkv, dtype=torch.float32, device=dev) for _ in range(3)]
    L = lib()
    ws = _ws(L.odmkv_window_stats_workspace_bytes(B, H, G, Tq), dev)
    scale = float(HEAD_DIM ** 0.5) if scale is None else float(scale)
    check(L.odmkv_window_attn_stats(ptr(Q), ptr(K), dtype_code(Q.dtype), B, H, G, Tq, Tkv, int(q_offset), scale, ptr(outs[0]),
                                    ptr(outs[1]), ptr(outs[2]), ptr(ws), ws.numel(), stream_ptr(dev)), "odmkv_window_attn_stats")
    if check_status:
        off = L.odmkv_window_stats_status_offset(B, H, G, Tq)
        if int(ws[off:off + 4].view(torch.int32).item()) != 0:
            raise OdmkvError("odmkv_window_attn_stats: a bounded wait on the tensor cores expired; the statistics are invalid")
    return tuple(outs)


def quantize_status() -> int:
    """0 while no bounded wait of the tensor-core quantise kernel has expired on the current device since the library
    was loaded, 1 afterwards (the codes of that call are invalid).  Synchronises the device."""
    rc = int(lib().odmkv_quantize_status())
    if rc < 0:
        raise OdmkvError("odmkv_quantize_status: the status word could not be read")
    return rc


# ---------------------------------------------------------------------------------------------
# allocator
# ---------------------------------------------------------------------------------------------

def _level_arrays(levels: Sequence[int], eps: Sequence[float]):
    K = len(levels)
    lv = (ctypes.c_int * K)(*[int(v) for v in levels])
    ev = (ctypes.c_double * K)(*[float(v) for v in eps])
    return lv, ev, K


def read_reports(rep: torch.Tensor) -> List[dict]:
    """Decode the device report buffer (synchronises)."""
    raw = rep.cpu().numpy().tobytes()
    size = ctypes.sizeof(AllocReport)
    out = []
    for i in range(len(raw) // size):
        r = AllocReport.from_buffer_copy(raw[i * size:(i + 1) * size])
        out.append(dict(lam=r.lam, gap_before=r.gap_before, counts=list(r.counts), n_active=r.n_active,
                        evaluations=r.evaluations, moved=r.moved, ties_lambda=r.ties_lambda, ties_cut=r.ties_cut,
                        done=bool(r.done)))
    return out


def allocate_bits(scores: torch.Tensor, sink_mask: Optional[torch.Tensor], levels: Sequence[int], eps: Sequence[float],
                  target: float, sink_bits: int = 16) -> Tuple[torch.Tensor, torch.Tensor]:
    """scores [P, n] fp32; sink_mask [n] bool/uint8 or None; eps already holds the eviction cost.
    Returns (bits int32 [P, n], report buffer uint8 [P * sizeof(report)])."""
    require_cuda(scores, "scores")
    P, n = scores.shape
    scores = scores.to(torch.float32).contiguous()
    mask = None if sink_mask is None else sink_mask.to(device=scores.device, dtype=torch.uint8).contiguous()
    bits = torch.empty(P, n, dtype=torch.int32, device=scores.device)
    rep = torch.zeros(P * ctypes.sizeof(AllocReport), dtype=torch.uint8, device=scores.device)
    ws = _ws(lib().odmkv_alloc_workspace_bytes(P, n), scores.device)
    lv, ev, K = _level_arrays(levels, eps)
    check(lib().odmkv_allocate_bits(ptr(scores), ptr(mask), P, n, lv, ev, K, float(target), int(sink_bits), ptr(bits),
                                    ptr(rep), ptr(ws), ws.numel(), stream_ptr(scores.device)), "odmkv_allocate_bits")
    return bits, rep


def allocate_bits_sharded(scores: torch.Tensor, sink_mask: Optional[torch.Tensor], levels: Sequence[int],
                          eps: Sequence[float], target: float, idx_base: int, all_reduce, sink_bits: int = 16
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same problem with the scores of each problem split over ranks (KV heads sharded): ``scores`` is this
    rank's [P, n_local] slice starting at global index ``idx_base``; ``all_reduce(t)`` must sum the int64
    tensor ``t`` in place over the ranks that share the problems (e.g. torch.distributed.all_reduce)."""
    require_cuda(scores, "scores")
    P, n = scores.shape
    scores = scores.to(torch.float32).contiguous()
    mask = None if sink_mask is None else sink_mask.to(device=scores.device, dtype=torch.uint8).contiguous()
    bits = torch.empty(P, n, dtype=torch.int32, device=scores.device)
    rep = torch.zeros(P * ctypes.sizeof(AllocReport), dtype=torch.uint8, device=scores.device)
    ws = _ws(lib().odmkv_alloc_workspace_bytes(P, n), scores.device)
    xlen = lib().odmkv_alloc_exchange_len()
    exch = torch.zeros(P, xlen, dtype=torch.int64, device=scores.device)
    lv, ev, K = _level_arrays(levels, eps)
    st = stream_ptr(scores.device)
    check(lib().odmkv_alloc_begin(ptr(scores), ptr(mask), P, n, int(idx_base), lv, ev, K, float(target), int(sink_bits),
                                  ptr(ws), ws.numel(), ptr(exch), st), "odmkv_alloc_begin")
    # the first 1 + 64 + 1 rounds are always assignment passes, which only fill the 16-entry head of
    # the accumulator; later rounds may already be gap-closure passes that fill the histogram
    eval_rounds = 66 if K > 1 else 1
    for r in range(lib().odmkv_alloc_num_rounds(K)):
        check(lib().odmkv_alloc_eval(ptr(ws), ptr(exch), st), "odmkv_alloc_eval")
        if r < eval_rounds:
            head = exch[:, :16].contiguous()
            all_reduce(head)
            exch[:, :16] = head
        else:
            all_reduce(exch)
        check(lib().odmkv_alloc_update(ptr(ws), ptr(exch), st), "odmkv_alloc_update")
    check(lib().odmkv_alloc_finish(ptr(ws), ptr(bits), ptr(rep), st), "odmkv_alloc_finish")
    return bits, rep


# ---------------------------------------------------------------------------------------------
# packed chunks
# ---------------------------------------------------------------------------------------------

@dataclass
class PackedChunk:
    """Packed form of one [B, H, T] block of tokens: per-class banks plus the segment table."""

    B: int
    H: int
    T: int
    t_offset: int
    dtype: torch.dtype
    device: torch.device
    seg_start: torch.Tensor            # int32 [6, B*H]
    seg_count: torch.Tensor            # int32 [6, B*H]
    totals: List[int]                  # padded slots per class
    k_codes: List[torch.Tensor] = field(default_factory=list)
    v_codes: List[torch.Tensor] = field(default_factory=list)
    k_norm: List[torch.Tensor] = field(default_factory=list)
    v_norm: List[torch.Tensor] = field(default_factory=list)
    pos: List[torch.Tensor] = field(default_factory=list)
    exact_k: Optional[torch.Tensor] = None
    exact_v: Optional[torch.Tensor] = None
    exact_pos: Optional[torch.Tensor] = None
    evicted_pos: Optional[torch.Tensor] = None
    _seg_count_host: Optional[np.ndarray] = None
    _c_struct: Optional[Chunk] = None     # chunks are immutable once built: the C view and the totals are cached
    _stored: Optional[int] = None

    def __deepcopy__(self, memo):
        # the cached C view holds raw pointers into this chunk's tensors: a copy gets its own on first use
        import copy
        new = self.__class__.__new__(self.__class__)
        memo[id(self)] = new
        for k, v in self.__dict__.items():
            setattr(new, k, None if k == "_c_struct" else copy.deepcopy(v, memo))
        return new

    def c_struct(self) -> Chunk:
        if self._c_struct is not None:
            return self._c_struct
        c = Chunk()
        for li in range(NUM_QLEVELS):
            c.k_codes[li] = self.k_codes[li].data_ptr()
            c.v_codes[li] = self.v_codes[li].data_ptr()
            c.k_norm[li] = self.k_norm[li].data_ptr()
            c.v_norm[li] = self.v_norm[li].data_ptr()
            c.pos[li] = self.pos[li].data_ptr()
        c.exact_k = self.exact_k.data_ptr()
        c.exact_v = self.exact_v.data_ptr()
        c.exact_pos = self.exact_pos.data_ptr()
        c.evicted_pos = self.evicted_pos.data_ptr()
        c.seg_start = self.seg_start.data_ptr()
        c.seg_count = self.seg_count.data_ptr()
        for k in range(NUM_CLASSES):
            c.cap[k] = int(self.totals[k])
        c.B, c.H, c.T, c.t_offset = self.B, self.H, self.T, self.t_offset
        self._c_struct = c
        return c

    def seg_count_host(self) -> np.ndarray:
        if self._seg_count_host is None:
            self._seg_count_host = self.seg_count.cpu().numpy()
        return self._seg_count_host

    def packed_bytes(self) -> int:
        """Bytes a decode step reads from this chunk (codes, norms, exact rows; real tokens only)."""
        cnt = self.seg_count_host().sum(axis=1)
        total = 0
        for li in range(NUM_QLEVELS):
            total += int(cnt[li + 1]) * 2 * (CODE_BYTES[li] + 4)
        total += int(cnt[5]) * 2 * HEAD_DIM * self.exact_k.element_size()
        return total

    def stored_tokens(self) -> int:
        if self._stored is None:
            self._stored = int(self.seg_count_host()[1:].sum())
        return self._stored


def quantize_pack(K: torch.Tensor, V: torch.Tensor, bits: torch.Tensor, pi_k: torch.Tensor, pi_v: torch.Tensor,
                  t_offset: int = 0) -> PackedChunk:
    """Route, quantise and pack [B, H, T, 128] keys/values according to bits [B, H, T] (int32 in
    {0, 2, 3, 4, 8, 16}).  One host read-back (the per-class totals) sizes the banks."""
    require_cuda(K, "keys")
    if K.shape != V.shape:
        raise ValueError(f"Mismatched key/value shapes: {tuple(K.shape)} vs {tuple(V.shape)}")
    if K.dim() != 4:
        raise ValueError(f"Expected keys/values with shape [B, H, T, D], got {tuple(K.shape)}")
    if tuple(bits.shape) != tuple(K.shape[:3]):
        raise ValueError(f"Expected bits shape {tuple(K.shape[:3])}, got {tuple(bits.shape)}")
    if K.shape[-1] != HEAD_DIM:
        raise ValueError(f"Expected head_dim {HEAD_DIM}, got {K.shape[-1]}")
    B, H, T, _ = K.shape
    dev = K.device
    K, V = K.contiguous(), V.contiguous()
    bits = bits.to(device=dev, dtype=torch.int32).contiguous()
    pi_k, pi_v = _rot(pi_k, dev), _rot(pi_v, dev)
    st = stream_ptr(dev)
    L = lib()
    plan = _ws(L.odmkv_pack_plan_workspace_bytes(B, H, T), dev)
    seg_start = torch.empty(NUM_CLASSES, B * H, dtype=torch.int32, device=dev)
    seg_count = torch.empty(NUM_CLASSES, B * H, dtype=torch.int32, device=dev)
    totals_d = torch.empty(8, dtype=torch.int32, device=dev)
    check(L.odmkv_pack_plan(ptr(bits), B, H, T, ptr(seg_start), ptr(seg_count), ptr(totals_d), ptr(plan), plan.numel(), st),
          "odmkv_pack_plan")
    totals = totals_d.cpu().tolist()
    if totals[6] != 0:
        raise ValueError(f"bits holds {totals[6]} values outside {CLASS_BITS}")
    ch = PackedChunk(B=B, H=H, T=T, t_offset=int(t_offset), dtype=K.dtype, device=dev, seg_start=seg_start,
                     seg_count=seg_count, totals=totals[:NUM_CLASSES])
    for li in range(NUM_QLEVELS):
        n = max(totals[li + 1], 1)
        ch.k_codes.append(torch.empty(n, CODE_BYTES[li], dtype=torch.uint8, device=dev))
        ch.v_codes.append(torch.empty(n, CODE_BYTES[li], dtype=torch.uint8, device=dev))
        ch.k_norm.append(torch.empty(n, dtype=torch.float32, device=dev))
        ch.v_norm.append(torch.empty(n, dtype=torch.float32, device=dev))
        ch.pos.append(torch.empty(n, dtype=torch.int32, device=dev))
    n16 = max(totals[5], 1)
    ch.exact_k = torch.empty(n16, HEAD_DIM, dtype=K.dtype, device=dev)
    ch.exact_v = torch.empty(n16, HEAD_DIM, dtype=K.dtype, device=dev)
    ch.exact_pos = torch.empty(n16, dtype=torch.int32, device=dev)
    ch.evicted_pos = torch.empty(max(totals[0], 1), dtype=torch.int32, device=dev)
    cs = ch.c_struct()
    scratch = _ws(L.odmkv_quantize_workspace_bytes(cs.cap), dev)   # linear value codes before re-tiling
    check(L.odmkv_quantize_pack(ptr(K), ptr(V), dtype_code(K.dtype), ptr(bits), ptr(pi_k), ptr(pi_v),
                                ptr(codebook_table(dev)), ctypes.byref(cs), ptr(plan), ptr(scratch), scratch.numel(), st),
          "odmkv_quantize_pack")
    return ch


def compact_chunks(chunks: Sequence[PackedChunk]) -> PackedChunk:
    """Merge chunks (time order) into one: inside every (b, h) segment of every class the tokens keep their order,
    chunk after chunk.  Host work: the summed segment table (from the chunks' cached counts)."""
    if not chunks:
        raise ValueError("compact_chunks needs at least one chunk")
    first = chunks[0]
    B, H, dev = first.B, first.H, first.device
    counts = np.stack([c.seg_count_host() for c in chunks]).astype(np.int64)          # [n, 6, BH]
    new_count = counts.sum(axis=0)
    padded = (new_count + _lib.SEG_ALIGN - 1) // _lib.SEG_ALIGN * _lib.SEG_ALIGN
    new_start = np.concatenate([np.zeros((NUM_CLASSES, 1), np.int64), np.cumsum(padded, axis=1)[:, :-1]], axis=1)
    totals = padded.sum(axis=1).tolist()
    dst_off = np.concatenate([np.zeros((1, NUM_CLASSES, B * H), np.int64), np.cumsum(counts, axis=0)[:-1]], axis=0)
    t_lo = min(c.t_offset for c in chunks)
    t_hi = max(c.t_offset + c.T for c in chunks)
    out = PackedChunk(B=B, H=H, T=t_hi - t_lo, t_offset=t_lo, dtype=first.dtype, device=dev,
                      seg_start=torch.from_numpy(new_start.astype(np.int32)).to(dev),
                      seg_count=torch.from_numpy(new_count.astype(np.int32)).to(dev), totals=[int(t) for t in totals])
    out._seg_count_host = new_count.astype(np.int32)
    for li in range(NUM_QLEVELS):
        n = max(totals[li + 1], 1)
        out.k_codes.append(torch.zeros(n, CODE_BYTES[li], dtype=torch.uint8, device=dev))
        out.v_codes.append(torch.zeros(n, CODE_BYTES[li], dtype=torch.uint8, device=dev))
        out.k_norm.append(torch.zeros(n, dtype=torch.float32, device=dev))
        out.v_norm.append(torch.zeros(n, dtype=torch.float32, device=dev))
        out.pos.append(torch.full((n,), -1, dtype=torch.int32, device=dev))
    n16 = max(totals[5], 1)
    out.exact_k = torch.zeros(n16, HEAD_DIM, dtype=first.dtype, device=dev)
    out.exact_v = torch.zeros(n16, HEAD_DIM, dtype=first.dtype, device=dev)
    out.exact_pos = torch.full((n16,), -1, dtype=torch.int32, device=dev)
    out.evicted_pos = torch.full((max(totals[0], 1),), -1, dtype=torch.int32, device=dev)
    arr = (Chunk * len(chunks))(*[c.c_struct() for c in chunks])
    cs = out.c_struct()
    off_d = torch.from_numpy(dst_off.astype(np.int32)).to(dev)
    L = lib()
    ws = _ws(L.odmkv_quantize_workspace_bytes(cs.cap), dev)
    check(L.odmkv_compact_chunks(arr, len(chunks), ctypes.byref(cs), ptr(off_d), dtype_code(first.dtype), ptr(ws), ws.numel(),
                                 stream_ptr(dev)), "odmkv_compact_chunks")
    return out


def encode_pack(y: torch.Tensor, bits: int) -> torch.Tensor:
    """Nearest centroid + pack of rotated coordinates y [n, 128] fp32 -> uint8 [n, code_bytes]."""
    require_cuda(y, "y")
    li = QLEVEL_BITS.index(bits)
    y = y.to(torch.float32).contiguous()
    out = torch.empty(y.shape[0], CODE_BYTES[li], dtype=torch.uint8, device=y.device)
    cb = codebook_table(y.device)[li].contiguous()
    check(lib().odmkv_encode_pack(ptr(y), y.shape[0], bits, ptr(cb), ptr(out), stream_ptr(y.device)), "odmkv_encode_pack")
    return out


def dequant_chunk_into(ch: PackedChunk, pi_k: torch.Tensor, pi_v: torch.Tensor, K_out: torch.Tensor, V_out: torch.Tensor,
                       include_exact: bool) -> None:
    """Scatter the dequantised tokens of a chunk into dense [B, H, T_dense, 128] tensors."""
    pi_k, pi_v = _rot(pi_k, ch.device), _rot(pi_v, ch.device)
    cs = ch.c_struct()
    check(lib().odmkv_dequant_chunk(ctypes.byref(cs), dtype_code(ch.dtype), ptr(pi_k), ptr(pi_v), ptr(codebook_table(ch.device)),
                                    ptr(K_out), ptr(V_out), dtype_code(K_out.dtype), K_out.shape[2], int(include_exact),
                                    stream_ptr(ch.device)), "odmkv_dequant_chunk")


def _row_start(ch: PackedChunk, cls: int) -> Tuple[torch.Tensor, int]:
    cnt = ch.seg_count_host()[cls].astype(np.int64)
    start = np.concatenate([[0], np.cumsum(cnt)[:-1]]).astype(np.int32)
    return torch.from_numpy(start).to(ch.device), int(cnt.sum())


def export_bank(ch: PackedChunk, bits: int):
    """Bank of one quantised level in the reference layout: (positions int64 [N, 3], packed key
    indices uint8 [N, ref_bytes], key norms, packed value indices, value norms)."""
    li = QLEVEL_BITS.index(bits)
    row_start, n = _row_start(ch, li + 1)
    dev = ch.device
    ik = torch.empty(n, REF_CODE_BYTES[li], dtype=torch.uint8, device=dev)
    iv = torch.empty_like(ik)
    nk = torch.empty(n, dtype=torch.float32, device=dev)
    nv = torch.empty_like(nk)
    pos = torch.empty(n, 3, dtype=torch.int64, device=dev)
    if n:
        cs = ch.c_struct()
        check(lib().odmkv_export_bank(ctypes.byref(cs), li + 1, ptr(row_start), ptr(ik), ptr(iv), ptr(nk), ptr(nv), ptr(pos),
                                      stream_ptr(dev)), "odmkv_export_bank")
    return pos, ik, nk, iv, nv


def export_positions(ch: PackedChunk, cls: int) -> torch.Tensor:
    """(b, h, t) rows of the evicted list (cls 0) or the exact bank (cls 5), row-major order."""
    row_start, n = _row_start(ch, cls)
    pos = torch.empty(n, 3, dtype=torch.int64, device=ch.device)
    if n:
        cs = ch.c_struct()
        check(lib().odmkv_export_positions(ctypes.byref(cs), cls, ptr(row_start), ptr(pos), stream_ptr(ch.device)),
              "odmkv_export_positions")
    return pos


def export_exact_rows(ch: PackedChunk) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Exact bank rows compacted in (b, h, t) order: positions, keys [N, 128], values [N, 128]."""
    pos = export_positions(ch, 5)
    cnt = ch.seg_count_host()[5]
    start = ch.seg_start.cpu().numpy()[5]
    idx = np.concatenate([np.arange(s, s + c) for s, c in zip(start, cnt)]) if len(cnt) else np.zeros(0, np.int64)
    idx_t = torch.from_numpy(idx.astype(np.int64)).to(ch.device)
    return pos, ch.exact_k[idx_t], ch.exact_v[idx_t]


# ---------------------------------------------------------------------------------------------
# decode attention
# ---------------------------------------------------------------------------------------------

_LUT_SCALES = None


def lut_scales():
    """Per level (2, 3, 4 bits) a factor s in [1, 2) that minimises the worst relative error of
    fp16(c * s) / s over the level's centroids; the tensor-core kernel stores fp16(c * s) in its tables."""
    global _LUT_SCALES
    if _LUT_SCALES is None:
        cand = np.linspace(1.0, 2.0, 40001, dtype=np.float64)[:-1]
        best = []
        for b in QLEVEL_BITS[:3]:
            c = codebook_f32(b).astype(np.float64)
            prod = (c[None, :] * cand[:, None]).astype(np.float32)
            back = prod.astype(np.float16).astype(np.float64) / cand[:, None]
            err = np.abs(back - c[None, :]) / np.abs(c[None, :])
            best.append(float(np.float32(cand[int(np.argmin(err.max(axis=1)))])))
        _LUT_SCALES = (ctypes.c_float * 3)(*best)
    return _LUT_SCALES


def decode_attn(q: torch.Tensor, chunks: Sequence[PackedChunk], pi_k: torch.Tensor, pi_v: torch.Tensor,
                tail_k: Optional[torch.Tensor] = None, tail_v: Optional[torch.Tensor] = None, tail_len: int = 0,
                scale: Optional[float] = None, n_splits: int = 0, out_dtype: Optional[torch.dtype] = None,
                return_lse: bool = False, cache_dtype: Optional[torch.dtype] = None, plain: bool = False,
                tail_len_dev: Optional[torch.Tensor] = None, tail_len_add: int = 0):
    """q [B, H*G, 128] -> out [B, H*G, 128]: softmax(q K_hat^T scale) V_hat over every token stored in
    ``chunks`` plus the first ``tail_len`` tokens of the dense tail [B, H, cap, 128].

    Calls ``odmkv_decode_attn_mma`` (tensor cores for the 2-, 3- and 4-bit banks).  ``plain=True`` calls
    ``odmkv_decode_attn`` instead, the CUDA-core reader of every level that the tests use as a second opinion.
    With ``tail_len_dev`` (int32 device tensor of one element) the tail length is ``tail_len_dev + tail_len_add``,
    read on the device when the kernel runs, and ``tail_len`` is only its upper bound
    (``odmkv_decode_attn_mma_devtail``): the form a captured decode step uses."""
    require_cuda(q, "query")
    if q.dim() != 3 or q.shape[-1] != HEAD_DIM:
        raise ValueError(f"expected query [B, Hq, {HEAD_DIM}], got {tuple(q.shape)}")
    B, Hq, _ = q.shape
    if chunks:
        H = chunks[0].H
        cdt = chunks[0].dtype
    elif tail_k is not None:
        H = tail_k.shape[1]
        cdt = tail_k.dtype
    else:
        raise ValueError("decode_attn needs at least one chunk or a tail")
    if cache_dtype is not None:
        cdt = cache_dtype
    if Hq % H:
        raise ValueError(f"query heads {Hq} not a multiple of KV heads {H}")
    G = Hq // H
    dev = q.device
    q = q.contiguous()
    pi_k, pi_v = _rot(pi_k, dev), _rot(pi_v, dev)
    L = lib()
    if n_splits <= 0:
        per_head = sum(c.stored_tokens() for c in chunks) // max(B * H, 1) + tail_len
        n_splits = L.odmkv_decode_default_splits(B, H, per_head)
    if plain:
        n_splits = min(n_splits, 64)
    out = torch.empty(B, Hq, HEAD_DIM, dtype=out_dtype or q.dtype, device=dev)
    lse = torch.empty(B, Hq, dtype=torch.float32, device=dev) if return_lse else None
    ws = _ws(L.odmkv_decode_workspace_bytes(B, H, G, n_splits), dev)
    arr = (Chunk * max(len(chunks), 1))()
    for i, c in enumerate(chunks):
        arr[i] = c.c_struct()
    cap = 0 if tail_k is None else tail_k.shape[2]
    scale = (1.0 / HEAD_DIM ** 0.5) if scale is None else float(scale)
    common = (ptr(q), dtype_code(q.dtype), arr, len(chunks), dtype_code(cdt), ptr(tail_k), ptr(tail_v), int(tail_len), int(cap),
              ptr(pi_k), ptr(pi_v), ptr(codebook_table(dev)), B, H, G, scale, ptr(out), dtype_code(out.dtype), ptr(lse),
              int(n_splits), ptr(ws), ws.numel())
    if tail_len_dev is not None:
        if plain or tail_k is None:
            raise ValueError("a device-side tail length needs the tensor-core path and a tail buffer")
        require_cuda(tail_len_dev, "tail_len_dev")
        if tail_len_dev.dtype != torch.int32 or tail_len_dev.numel() != 1:
            raise ValueError("tail_len_dev must be one int32 element")
        check(L.odmkv_decode_attn_mma_devtail(ptr(q), dtype_code(q.dtype), arr, len(chunks), dtype_code(cdt), ptr(tail_k), ptr(tail_v),
                                              ptr(tail_len_dev), int(tail_len_add), int(tail_len), int(cap), ptr(pi_k), ptr(pi_v),
                                              ptr(codebook_table(dev)), B, H, G, scale, ptr(out), dtype_code(out.dtype), ptr(lse),
                                              int(n_splits), ptr(ws), ws.numel(), lut_scales(), stream_ptr(dev)),
              "odmkv_decode_attn_mma_devtail")
    elif plain:
        check(L.odmkv_decode_attn(*common, stream_ptr(dev)), "odmkv_decode_attn")
    else:
        check(L.odmkv_decode_attn_mma(*common, lut_scales(), stream_ptr(dev)), "odmkv_decode_attn_mma")
    return (out, lse) if return_lse else out
