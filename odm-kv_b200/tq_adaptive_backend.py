"""Mixed-precision KV cache state: bit-width-segregated banks held as packed chunks.

Mirrors ``TurboQuantAdaptiveKVCacheState`` of the reference (kvquant/tq_adaptive_backend.py:245-541)
with the "mse" key and value quantisers.  Storage differs from the reference's growing per-level
tensors: each ``prefill`` / ``append`` / ``flush_buffer`` call produces one immutable packed *chunk*
(``ops.PackedChunk``) and recent decode tokens live in a preallocated dense *tail*; decode attention
reads chunks and tail directly.  The reference's bank views (``_quantized_banks``, ``_exact_bank``,
``_masked_positions``) are available as exports in its byte layout.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from . import ops
from ._lib import HEAD_DIM, QLEVEL_BITS
from .tq_backend import MSEQuantized, random_rotation

__all__ = ["TurboQuantAdaptiveKVCacheState", "ExactBankView", "QuantizedBankView"]


@dataclass
class ExactBankView:
    positions: torch.Tensor
    keys: Optional[torch.Tensor]
    values: Optional[torch.Tensor]

    @property
    def size(self) -> int:
        return int(self.positions.shape[0])


@dataclass
class QuantizedBankView:
    bits: int
    positions: torch.Tensor
    key_quantized: Optional[MSEQuantized]
    value_quantized: Optional[MSEQuantized]

    @property
    def size(self) -> int:
        return int(self.positions.shape[0])


class TurboQuantAdaptiveKVCacheState:
    def __init__(self, head_dim: int, bit_levels, value_group_size: int = 32, device=None, dtype=torch.float16,
                 key_quantizer: str = "mse", value_quantizer: str = "mse", seed: int = 42, outlier_indices=None,
                 regular_indices=None, outlier_min_bits: int = 4, tail_capacity: int = 256):
        if head_dim != HEAD_DIM:
            raise ValueError(f"Expected head_dim {HEAD_DIM}, got {head_dim}")
        if str(key_quantizer).lower() not in ("mse", "turboquant_mse", "turboquantmse") or \
                str(value_quantizer).lower() not in ("mse", "turboquant", "turboquant_mse"):
            raise NotImplementedError("only the Lloyd-Max (mse) key and value quantisers are implemented")
        if outlier_indices is not None:
            raise NotImplementedError("outlier-channel separation is not implemented")
        levels = tuple(sorted(set(int(b) for b in bit_levels)))
        bad = [b for b in levels if b not in (0, 16) and b not in QLEVEL_BITS]
        if bad:
            raise ValueError(f"unsupported bit levels {bad}; quantised levels must be in {QLEVEL_BITS}")
        self.head_dim = head_dim
        self.bit_levels = levels
        self.value_group_size = value_group_size
        self.device = torch.device(device) if device is not None else torch.device("cuda")
        self.dtype = dtype
        self.key_quantizer, self.value_quantizer = "mse", "mse"
        self.seed = seed
        # key rotation seed = seed, value rotation seed = seed + 2000 (tq_adaptive_backend.py:115-133)
        self.pi_k = random_rotation(head_dim, self.device, torch.float32, seed=seed)
        self.pi_v = random_rotation(head_dim, self.device, torch.float32, seed=seed + 2000)
        self._tail_capacity0 = int(tail_capacity)
        self._reset()

    # ------------------------------------------------------------------ bookkeeping
    def _reset(self) -> None:
        self.batch_size = 0
        self.num_heads = 0
        self.seq_len = 0
        self.chunks: List[ops.PackedChunk] = []
        self.tail_k: Optional[torch.Tensor] = None
        self.tail_v: Optional[torch.Tensor] = None
        self.tail_start = 0      # sequence position of the first tail token
        self.tail_len = 0
        self._tail_len_dev = None   # int32 [1] on the device while a captured decode step owns the tail counter
        self._tail_room = 0

    def _validate_shapes(self, keys, values, bits=None) -> None:
        if keys.shape != values.shape:
            raise ValueError(f"Mismatched key/value shapes: {keys.shape} vs {values.shape}")
        if keys.dim() != 4:
            raise ValueError(f"Expected keys/values with shape [B, H, T, D], got {keys.shape}")
        if bits is not None and bits.shape != keys.shape[:3]:
            raise ValueError(f"Expected bits shape {keys.shape[:3]}, got {bits.shape}")
        if keys.shape[-1] != self.head_dim:
            raise ValueError(f"Expected head_dim {self.head_dim}, got {keys.shape[-1]}")
        if self.batch_size == 0:
            self.batch_size, self.num_heads = int(keys.shape[0]), int(keys.shape[1])
        elif self.batch_size != int(keys.shape[0]) or self.num_heads != int(keys.shape[1]):
            raise ValueError(f"Adaptive backend state shape changed from (B={self.batch_size}, H={self.num_heads}) "
                             f"to (B={keys.shape[0]}, H={keys.shape[1]})")

    def _ensure_tail(self, need: int) -> None:
        cap = 0 if self.tail_k is None else self.tail_k.shape[2]
        if need <= cap:
            return
        new_cap = max(self._tail_capacity0, cap)
        while new_cap < need:
            new_cap *= 2
        tk = torch.zeros(self.batch_size, self.num_heads, new_cap, self.head_dim, dtype=self.dtype, device=self.device)
        tv = torch.zeros_like(tk)
        if self.tail_k is not None and self.tail_len:
            tk[:, :, : self.tail_len] = self.tail_k[:, :, : self.tail_len]
            tv[:, :, : self.tail_len] = self.tail_v[:, :, : self.tail_len]
        self.tail_k, self.tail_v = tk, tv

    # ------------------------------------------------------------------ writes
    def prefill(self, keys: torch.Tensor, values: torch.Tensor, bits: torch.Tensor) -> None:
        self._reset()
        self.append(keys, values, bits)

    def append(self, keys: torch.Tensor, values: torch.Tensor, bits: torch.Tensor) -> None:
        """Route new tokens by their bit level (tq_adaptive_backend.py:350-374): one packed chunk."""
        self._validate_shapes(keys, values, bits)
        if self.tail_len:
            raise RuntimeError("append() after exact tail tokens: flush or truncate the decode buffer first")
        if keys.shape[2] == 0:
            return
        chunk = ops.quantize_pack(keys.to(self.dtype), values.to(self.dtype), bits, self.pi_k, self.pi_v, t_offset=self.seq_len)
        self.chunks.append(chunk)
        self.seq_len += int(keys.shape[2])
        self.tail_start = self.seq_len
        self._bound_chunks()

    def append_all_exact(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """Keep new tokens verbatim (tq_adaptive_backend.py:380-425): they go to the dense tail."""
        self._validate_shapes(keys, values)
        T = int(keys.shape[2])
        if T == 0:
            return
        if self.tail_len == 0:
            self.tail_start = self.seq_len
        if self._tail_len_dev is not None:
            self._write_tail_at_counter(keys, values)
            self._tail_len_dev.add_(T)
        else:
            self._ensure_tail(self.tail_len + T)
            self.tail_k[:, :, self.tail_len:self.tail_len + T] = keys
            self.tail_v[:, :, self.tail_len:self.tail_len + T] = values
        self.tail_len += T
        self.seq_len += T

    def stage_pending(self, keys: torch.Tensor, values: torch.Tensor) -> int:
        """Copy tokens that a forward pass has produced but the hook has not appended yet right behind
        the tail, without committing them; returns the tail length a decode call should attend."""
        T = int(keys.shape[2])
        self._validate_shapes(keys, values)
        if self._tail_len_dev is not None:
            self._write_tail_at_counter(keys, values)
            return self.tail_len + T
        self._ensure_tail(self.tail_len + T)
        self.tail_k[:, :, self.tail_len:self.tail_len + T] = keys
        self.tail_v[:, :, self.tail_len:self.tail_len + T] = values
        return self.tail_len + T

    # ------------------------------------------------------------------ device-side tail counter (captured decode steps)
    def begin_device_tail(self, room: int) -> None:
        """Switch the tail bookkeeping to a counter in device memory, for a decode step that is captured into a
        CUDA graph and replayed while the tail grows by one token per replay: tail writes go to the slot the counter
        names and the decode kernels read the tail length from it.  ``room`` = tokens the tail may still take before
        ``end_device_tail`` (the buffer is grown now, never while the counter is in use).  The host counters keep
        advancing as usual in an eager pass; after a replay the caller advances them with ``advance_host(1)``."""
        if self.batch_size == 0:
            raise RuntimeError("begin_device_tail() needs a prefilled state")
        self._ensure_tail(self.tail_len + int(room) + 1)
        self._tail_room = self.tail_len + int(room) + 1
        if self._tail_len_dev is None:
            self._tail_len_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._tail_len_dev.fill_(self.tail_len)

    def end_device_tail(self) -> None:
        self._tail_len_dev = None

    def advance_host(self, n: int = 1) -> None:
        """Mirror on the host what a replayed decode step did on the device: ``n`` tokens joined the tail."""
        if self.tail_len == 0:
            self.tail_start = self.seq_len
        self.tail_len += int(n)
        self.seq_len += int(n)

    def _write_tail_at_counter(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        T = int(keys.shape[2])
        if T != 1:
            raise ValueError("the device-side tail counter serves single-token decode steps")
        if self.tail_len + T > self._tail_room:
            raise RuntimeError("the tail outgrew the room reserved by begin_device_tail()")
        idx = self._tail_len_dev.to(torch.int64)
        self.tail_k.index_copy_(2, idx, keys.to(self.dtype))
        self.tail_v.index_copy_(2, idx, values.to(self.dtype))

    def truncate(self, seq_len: int) -> None:
        """Drop every token at position >= seq_len (tq_adaptive_backend.py:427-437)."""
        seq_len = int(seq_len)
        if seq_len >= self.seq_len:
            return
        self.seq_len = seq_len
        self.tail_len = max(0, min(self.tail_len, seq_len - self.tail_start))
        kept = []
        for ch in self.chunks:
            if ch.t_offset >= seq_len:
                continue
            if ch.t_offset + ch.T > seq_len:
                ch = self._truncate_chunk(ch, seq_len)
            kept.append(ch)
        self.chunks = kept
        if self.tail_len == 0:
            self.tail_start = self.seq_len

    def _truncate_chunk(self, ch: ops.PackedChunk, seq_len: int) -> ops.PackedChunk:
        """Positions inside a segment ascend, so truncation only shortens every segment."""
        starts = ch.seg_start.cpu().numpy()
        counts = ch.seg_count_host().copy()
        pos_arrays = [ch.evicted_pos] + list(ch.pos) + [ch.exact_pos]
        for c in range(6):
            pos = pos_arrays[c].cpu().numpy()
            for bh in range(ch.B * ch.H):
                s, n = int(starts[c, bh]), int(counts[c, bh])
                counts[c, bh] = int(np.searchsorted(pos[s:s + n], seq_len, side="left"))
        new = ops.PackedChunk(B=ch.B, H=ch.H, T=seq_len - ch.t_offset, t_offset=ch.t_offset, dtype=ch.dtype, device=ch.device,
                              seg_start=ch.seg_start, seg_count=torch.from_numpy(counts).to(ch.device), totals=ch.totals,
                              k_codes=ch.k_codes, v_codes=ch.v_codes, k_norm=ch.k_norm, v_norm=ch.v_norm, pos=ch.pos,
                              exact_k=ch.exact_k, exact_v=ch.exact_v, exact_pos=ch.exact_pos, evicted_pos=ch.evicted_pos)
        return new

    # ------------------------------------------------------------------ decode buffer
    def get_buffer_tokens(self, buffer_start_seq: int):
        """Buffered tokens (position >= buffer_start_seq) as (positions [N, 3], keys [N, d], values [N, d])
        in (b, h, t) row-major order (tq_adaptive_backend.py:466-479)."""
        lo = max(int(buffer_start_seq) - self.tail_start, 0)
        n = self.tail_len - lo
        if self.tail_k is None or n <= 0:
            empty = torch.empty(0, self.head_dim, device=self.device, dtype=self.dtype)
            return torch.empty((0, 3), dtype=torch.long, device=self.device), empty, empty.clone()
        B, H = self.batch_size, self.num_heads
        k = self.tail_k[:, :, lo:self.tail_len].reshape(-1, self.head_dim)
        v = self.tail_v[:, :, lo:self.tail_len].reshape(-1, self.head_dim)
        b_idx = torch.arange(B, device=self.device).view(B, 1, 1).expand(B, H, n).reshape(-1)
        h_idx = torch.arange(H, device=self.device).view(1, H, 1).expand(B, H, n).reshape(-1)
        t_idx = (torch.arange(n, device=self.device) + self.tail_start + lo).view(1, 1, n).expand(B, H, n).reshape(-1)
        return torch.stack([b_idx, h_idx, t_idx], dim=-1).to(torch.long), k, v

    def buffer_view(self, buffer_start_seq: int):
        """Dense view of the buffered tokens: keys, values [B, H, n, d] (no copy)."""
        lo = max(int(buffer_start_seq) - self.tail_start, 0)
        return self.tail_k[:, :, lo:self.tail_len], self.tail_v[:, :, lo:self.tail_len]

    def flush_buffer(self, buffer_start_seq: int, new_bits: torch.Tensor) -> Optional[ops.PackedChunk]:
        """Re-quantise the buffered tokens with their new bit levels (tq_adaptive_backend.py:481-532).
        ``new_bits`` is flat [N] in the order of ``get_buffer_tokens`` or shaped [B, H, n]."""
        lo = max(int(buffer_start_seq) - self.tail_start, 0)
        n = self.tail_len - lo
        if self.tail_k is None or n <= 0:
            return None
        B, H = self.batch_size, self.num_heads
        bits = new_bits.to(device=self.device, dtype=torch.int32).reshape(B, H, n)
        known = torch.zeros_like(bits, dtype=torch.bool)
        for level in self.bit_levels:
            known |= bits == level
        bits = torch.where(known, bits, torch.full_like(bits, 16))   # unrouted tokens stay exact (529-532)
        k = self.tail_k[:, :, lo:self.tail_len].contiguous()
        v = self.tail_v[:, :, lo:self.tail_len].contiguous()
        if lo > 0:
            # Tokens in front of the buffer (a pinned multi-token pass) stay exact but leave the tail as a chunk of
            # their own, so that the tail is empty afterwards and tail index i keeps meaning position tail_start + i.
            pinned = torch.full((B, H, lo), 16, dtype=torch.int32, device=self.device)
            self.chunks.append(ops.quantize_pack(self.tail_k[:, :, :lo].contiguous(), self.tail_v[:, :, :lo].contiguous(), pinned,
                                                 self.pi_k, self.pi_v, t_offset=self.tail_start))
        chunk = ops.quantize_pack(k, v, bits, self.pi_k, self.pi_v, t_offset=self.tail_start + lo)
        self.chunks.append(chunk)
        self.tail_len = 0
        self.tail_start = self.seq_len
        self._bound_chunks()
        return chunk

    def compact(self, keep_first: int = 1) -> None:
        """Merge the chunks after the first ``keep_first`` into one (the reference's banks simply grow with every flush,
        kvquant/tq_adaptive_backend.py:481-532; here a state holds a bounded list of immutable chunks instead)."""
        if len(self.chunks) - keep_first < 2:
            return
        merged = ops.compact_chunks(self.chunks[keep_first:])
        self.chunks = self.chunks[:keep_first] + [merged]

    def _bound_chunks(self) -> None:
        """Keeps the chunk list within what one decode call accepts: the flushed chunks are merged when the list is full."""
        if len(self.chunks) >= ops._lib.MAX_CHUNKS:
            self.compact(keep_first=1)

    # ------------------------------------------------------------------ reads
    def materialize(self):
        """Dense dequantised cache [B, H, seq_len, d] in the cache dtype; evicted rows are zero
        (tq_adaptive_backend.py:439-452)."""
        keys = torch.zeros(self.batch_size, self.num_heads, self.seq_len, self.head_dim, device=self.device, dtype=self.dtype)
        values = torch.zeros_like(keys)
        self._materialize_into(keys, values, include_exact=True)
        return keys, values

    def materialize_fp32(self):
        """Same as ``materialize`` but fp32, i.e. the values before the cast to the cache dtype."""
        keys = torch.zeros(self.batch_size, self.num_heads, self.seq_len, self.head_dim, device=self.device, dtype=torch.float32)
        values = torch.zeros_like(keys)
        self._materialize_into(keys, values, include_exact=True)
        return keys, values

    def materialize_quantized_into(self, keys: torch.Tensor, values: torch.Tensor, chunks=None) -> None:
        """Overwrite only the quantised positions of existing dense tensors (tq_adaptive_backend.py:454-464)."""
        self._materialize_into(keys, values, include_exact=False, chunks=chunks)

    def _materialize_into(self, keys, values, include_exact: bool, chunks=None) -> None:
        if not keys.is_contiguous() or not values.is_contiguous():
            raise ValueError("dense cache tensors must be contiguous")
        for ch in (self.chunks if chunks is None else chunks):
            ops.dequant_chunk_into(ch, self.pi_k, self.pi_v, keys, values, include_exact)
        if include_exact and self.tail_len:
            s = self.tail_start
            keys[:, :, s:s + self.tail_len] = self.tail_k[:, :, : self.tail_len].to(keys.dtype)
            values[:, :, s:s + self.tail_len] = self.tail_v[:, :, : self.tail_len].to(values.dtype)

    def keep_mask(self) -> torch.Tensor:
        """[B, H, seq_len] bool: False at evicted positions."""
        keep = torch.ones(self.batch_size, self.num_heads, self.seq_len, dtype=torch.bool, device=self.device)
        mp = self._masked_positions
        if mp.numel():
            keep[mp[:, 0], mp[:, 1], mp[:, 2]] = False
        return keep

    def masked_key_indices(self):
        """(b, h, t) index tensors of the evicted tokens, or None.  Chunks are immutable, so the result is kept until
        the chunk list changes (a flush, an append or a truncation)."""
        version = tuple(id(c) for c in self.chunks)
        cached = getattr(self, "_masked_cache", None)
        if cached is not None and cached[0] == version:
            return cached[1]
        mp = self._masked_positions
        out = None if mp.numel() == 0 else (mp[:, 0], mp[:, 1], mp[:, 2])
        self._masked_cache = (version, out)
        return out

    def decode_attention(self, query: torch.Tensor, scale: Optional[float] = None, pending_k=None, pending_v=None,
                         out_dtype=None) -> torch.Tensor:
        """softmax(q K_hat^T scale) V_hat over the stored cache for one query per head.
        query [B, Hq, d]; optional pending_k/v [B, H, t, d] are attended as well (tokens of the running
        forward pass that have not been appended yet).  Returns [B, Hq, d]."""
        tail_len = self.tail_len
        n_pending = 0
        if pending_k is not None:
            if self.batch_size == 0:
                self.batch_size, self.num_heads = int(pending_k.shape[0]), int(pending_k.shape[1])
            n_pending = int(pending_k.shape[2])
            tail_len = self.stage_pending(pending_k, pending_v)
        if len(self.chunks) > ops._lib.MAX_CHUNKS:
            self.compact(keep_first=1)
        if self._tail_len_dev is not None:
            return ops.decode_attn(query, self.chunks, self.pi_k, self.pi_v, tail_k=self.tail_k, tail_v=self.tail_v,
                                   tail_len=self._tail_room, scale=scale, out_dtype=out_dtype, cache_dtype=self.dtype,
                                   tail_len_dev=self._tail_len_dev, tail_len_add=n_pending)
        return ops.decode_attn(query, self.chunks, self.pi_k, self.pi_v, tail_k=self.tail_k, tail_v=self.tail_v,
                               tail_len=tail_len, scale=scale, out_dtype=out_dtype, cache_dtype=self.dtype)

    def packed_bytes(self) -> int:
        return sum(c.packed_bytes() for c in self.chunks) + \
            2 * self.tail_len * self.batch_size * self.num_heads * self.head_dim * torch.empty(0, dtype=self.dtype).element_size()

    # ------------------------------------------------------------------ reference-layout views
    @property
    def _masked_positions(self) -> torch.Tensor:
        parts = [ops.export_positions(c, 0) for c in self.chunks]
        parts = [p for p in parts if p.numel()]
        return torch.cat(parts, dim=0) if parts else torch.empty((0, 3), dtype=torch.long, device=self.device)

    @property
    def _quantized_banks(self) -> dict:
        banks = {}
        for bits in self.bit_levels:
            if bits in (0, 16):
                continue
            rows = [ops.export_bank(c, bits) for c in self.chunks]
            rows = [r for r in rows if r[0].numel()]
            if not rows:
                banks[bits] = QuantizedBankView(bits, torch.empty((0, 3), dtype=torch.long, device=self.device), None, None)
                continue
            pos = torch.cat([r[0] for r in rows])
            kq = MSEQuantized(torch.cat([r[1] for r in rows]), torch.cat([r[2] for r in rows]), bits)
            vq = MSEQuantized(torch.cat([r[3] for r in rows]), torch.cat([r[4] for r in rows]), bits)
            banks[bits] = QuantizedBankView(bits, pos, kq, vq)
        return banks

    @property
    def _exact_bank(self) -> ExactBankView:
        rows = [ops.export_exact_rows(c) for c in self.chunks]
        rows = [r for r in rows if r[0].numel()]
        pos = [r[0] for r in rows]
        ks = [r[1] for r in rows]
        vs = [r[2] for r in rows]
        if self.tail_len:
            # decode appends arrive one position at a time, each as (b, h) rows
            B, H, n = self.batch_size, self.num_heads, self.tail_len
            t_idx = (torch.arange(n, device=self.device) + self.tail_start).view(n, 1, 1).expand(n, B, H).reshape(-1)
            b_idx = torch.arange(B, device=self.device).view(1, B, 1).expand(n, B, H).reshape(-1)
            h_idx = torch.arange(H, device=self.device).view(1, 1, H).expand(n, B, H).reshape(-1)
            pos.append(torch.stack([b_idx, h_idx, t_idx], dim=-1).to(torch.long))
            ks.append(self.tail_k[:, :, :n].permute(2, 0, 1, 3).reshape(-1, self.head_dim))
            vs.append(self.tail_v[:, :, :n].permute(2, 0, 1, 3).reshape(-1, self.head_dim))
        if not pos:
            return ExactBankView(torch.empty((0, 3), dtype=torch.long, device=self.device), None, None)
        return ExactBankView(torch.cat(pos), torch.cat(ks), torch.cat(vs))
