"""``TurboQuantPerTokenBackendPress``: score -> allocate -> quantise into a packed side-car state.

Mirrors the reference's ``kvquant/adaptive_backend_press.py`` (hook orchestration, 327-458; prefill
finalisation, 292-325; decode-buffer flush, 464-665) and the parts of ``kvquant/press.py`` it inherits
(``_compute_bits`` 235-270, ``_build_sink_mask`` 218-224, context manager 637-692), for the settings the
reference's experiments use: Lloyd-Max ("mse") key and value quantisers, no outlier channels.

Differences that do not change results:
  * with ``layerwise=True`` every layer is compressed in its own hook instead of after the last layer
    (each layer's Lagrangian is independent), so full-precision KV of earlier layers is not kept around;
  * all samples of a batch are scored and allocated in one launch each;
  * decode steps attend over the packed state directly (see ``attention_patch``); by default the dense HF cache is
    still kept in sync like the reference does, so code that reads ``cache.layers[i].keys`` keeps working; with
    ``packed_cache=True`` a compressed layer drops its dense tensors and stops growing by concatenation
    (``packed_cache.PackedCacheLayer``).
"""
from __future__ import annotations

import contextlib
import inspect
import math
import sys
from typing import Optional

import torch
from torch import nn

from . import ops
from .allocator import calibrate_epsilon, optimal_scores_to_bits, ratio_scores_to_bits, scores_to_bits
from .attention_patch import patch_attention_functions
from .scorer import (BaseScorer, RiskScorer, _aligned_rotary_outputs, _apply_rotary_pos_emb_q, _get_query_states)
from .tq_adaptive_backend import TurboQuantAdaptiveKVCacheState

__all__ = ["TurboQuantPerTokenBackendPress"]


class TurboQuantPerTokenBackendPress:
    def __init__(self, *, value_group_size: int = 32, key_quantizer: str = "prod", value_quantizer: str = "minmax",
                 scorer: Optional[BaseScorer] = None, bit_levels: tuple = (0, 2, 4, 8, 16), ratios: Optional[tuple] = None,
                 target_avg_bits: Optional[float] = None, eviction_cost: float = 5.0, above_target_alpha: float = 1.0,
                 n_outlier_channels: int = 0, outlier_min_bits: int = 4, seed: int = 42, decode_quant: bool = True,
                 sink_tokens: int = 0, layerwise: bool = False, buffer_size: int = 128, initial_layers_fp16: int = 0,
                 allow_decode_eviction: bool = False, packed_cache: bool = False):
        if scorer is None:
            raise ValueError("TurboQuantPerTokenBackendPress requires an explicit scorer.")
        if str(key_quantizer).lower() not in ("mse", "turboquant_mse", "turboquantmse"):
            raise NotImplementedError("only key_quantizer='mse' is implemented (the reference's experiment setting)")
        if str(value_quantizer).lower() not in ("mse", "turboquant", "turboquant_mse"):
            raise NotImplementedError("only value_quantizer='mse' is implemented (the reference's experiment setting)")
        if n_outlier_channels > 0:
            raise NotImplementedError("outlier-channel separation is not implemented")
        invalid = [b for b in bit_levels if b not in (0, 16) and b < 1]
        if invalid:
            raise ValueError(f"TurboQuantPerTokenBackendPress does not support key bit-levels below 1: {invalid}")
        self.scorer = scorer
        self.bit_levels = tuple(bit_levels)
        self.ratios = ratios
        self.target_avg_bits = target_avg_bits
        self.eviction_cost = eviction_cost
        self.above_target_alpha = above_target_alpha
        self.n_outlier_channels = n_outlier_channels
        self.outlier_min_bits = outlier_min_bits
        self.seed = seed
        self.decode_quant = decode_quant
        self.sink_tokens = sink_tokens
        self.layerwise = layerwise
        self.quantizer = "turboquant"
        self.key_quantizer = "mse"
        self.value_quantizer = "mse"
        self.value_group_size = value_group_size
        self.allow_decode_eviction = bool(allow_decode_eviction)
        self.buffer_size = buffer_size
        self.initial_layers_fp16 = initial_layers_fp16
        # True: a compressed layer keeps no dense keys / values (packed_cache.PackedCacheLayer); False: the dense HF
        # cache stays in sync with the dequantised tokens as in the reference
        self.packed_cache = bool(packed_cache)
        if self.allow_decode_eviction:
            self._decode_bit_levels = tuple(bit_levels)
        else:
            self._decode_bit_levels = tuple(b for b in bit_levels if b != 0) or (16,)
        self._epsilon: Optional[dict] = None
        self._head_dim: Optional[int] = None
        self._prefill_hooks_fired = 0
        self._alloc_logged = False
        self._states: dict[int, TurboQuantAdaptiveKVCacheState] = {}
        self._buffer_counts: dict[int, int] = {}
        self._buffer_start_seqs: dict[int, int] = {}
        self._observed_ratios: dict = {}
        self._hooked_layer_indices: list[int] = []
        self._last_hooked_layer_idx: Optional[int] = None
        self._layer_modules: dict[int, nn.Module] = {}
        self._score_prefill_supports_kwargs = self._supports_kwargs(self.scorer.score_prefill)
        self._reset_prefill_state()

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _supports_kwargs(method) -> bool:
        params = inspect.signature(method).parameters.values()
        return any(p.kind == inspect.Parameter.VAR_KEYWORD for p in params) or any(
            p.name in {"module", "hidden_states"} for p in params)

    def _reset_prefill_state(self) -> None:
        self._prefill_scores: dict[int, torch.Tensor] = {}
        self._prefill_sink_masks: dict[int, Optional[torch.Tensor]] = {}

    def _build_sink_mask(self, H: int, T: int, device) -> Optional[torch.Tensor]:
        if self.sink_tokens <= 0:
            return None
        mask = torch.zeros(H, T, dtype=torch.bool, device=device)
        mask[:, : min(self.sink_tokens, T)] = True
        return mask

    @staticmethod
    def _get_cache_tensors(cache, layer_idx: int):
        if hasattr(cache, "key_cache") and isinstance(cache.key_cache, list):
            return cache.key_cache[layer_idx], cache.value_cache[layer_idx]
        layer = cache.layers[layer_idx]
        return layer.keys, layer.values

    @staticmethod
    def _set_cache_tensors(cache, layer_idx: int, keys, values) -> None:
        if hasattr(cache, "key_cache") and isinstance(cache.key_cache, list):
            cache.key_cache[layer_idx], cache.value_cache[layer_idx] = keys, values
            return
        cache.layers[layer_idx].keys = keys
        cache.layers[layer_idx].values = values

    def _ensure_epsilon(self, device) -> dict:
        if self._epsilon is None:
            self._epsilon = calibrate_epsilon(self._head_dim or 128, self.bit_levels, seed=self.seed, device=device,
                                              value_group_size=self.value_group_size, n_outlier=0,
                                              outlier_min_bits=self.outlier_min_bits, value_quantizer="mse")
        return self._epsilon

    def _compute_bits(self, scores: torch.Tensor, sink_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Scores of one problem -> bits (kvquant/press.py:235-270)."""
        if self.ratios is not None:
            return ratio_scores_to_bits(scores, self.bit_levels, self.ratios, sink_mask)
        if self.target_avg_bits is not None:
            eps = self._ensure_epsilon(scores.device)
            return optimal_scores_to_bits(scores, self.bit_levels, self.target_avg_bits, eps, sink_mask,
                                          eviction_cost=self.eviction_cost, n_outlier=0, head_dim=self._head_dim or 128,
                                          outlier_min_bits=self.outlier_min_bits, above_target_alpha=self.above_target_alpha)
        bits = scores_to_bits(scores, self.bit_levels)
        if sink_mask is not None:
            bits = bits.clone()
            bits[sink_mask] = 16
        return bits

    def _compute_bits_batched(self, scores: torch.Tensor, sink_mask: Optional[torch.Tensor]) -> torch.Tensor:
        """[P, H, T] scores of P independent problems -> int32 bits, one allocator launch for all of them."""
        if self.ratios is not None or self.target_avg_bits is None or self.above_target_alpha < 1.0:
            return torch.stack([self._compute_bits(s, sink_mask) for s in scores])
        eps = self._ensure_epsilon(scores.device)
        levels = sorted(set(int(b) for b in self.bit_levels))
        ev = [float(eps.get(b, 0.0)) for b in levels]
        if self.eviction_cost != 1.0 and levels[0] == 0:
            ev[0] *= self.eviction_cost
        P = scores.shape[0]
        mask = None if sink_mask is None else sink_mask.reshape(-1)
        bits, rep = ops.allocate_bits(scores.reshape(P, -1), mask, levels, ev, float(self.target_avg_bits), 16)
        self._last_alloc_report = rep
        return bits.reshape(scores.shape)

    def _log_alloc(self, bits: torch.Tensor) -> None:
        if self._alloc_logged:
            return
        self._alloc_logged = True
        total = bits.numel()
        parts = []
        for b in sorted(set(self.bit_levels) | {16}):
            cnt = int((bits == b).sum().item())
            if cnt:
                parts.append(f"{b}bit:{cnt}({cnt / total * 100:.1f}%)")
        print(f"[alloc] n={total} avg_nominal={bits.float().mean().item():.3f}  {' '.join(parts)}", file=sys.stderr, flush=True)

    def _get_or_create_state(self, layer_idx: int, keys: torch.Tensor) -> TurboQuantAdaptiveKVCacheState:
        state = self._states.get(layer_idx)
        if state is not None:
            return state
        levels = self.bit_levels
        if self.buffer_size > 0 and 16 not in levels:
            levels = tuple(sorted(set(levels) | {16}))
        # key rotation seed = press seed + 7 * layer (kvquant/adaptive_backend_press.py:123)
        state = TurboQuantAdaptiveKVCacheState(head_dim=keys.shape[-1], bit_levels=levels, value_group_size=self.value_group_size,
                                               device=keys.device, dtype=keys.dtype, key_quantizer="mse", value_quantizer="mse",
                                               seed=self.seed + layer_idx * 7, outlier_min_bits=self.outlier_min_bits)
        self._states[layer_idx] = state
        return state

    @staticmethod
    def _is_packed_layer(cache, layer_idx: int) -> bool:
        if not hasattr(cache, "layers"):
            return False
        from .packed_cache import PackedCacheLayer
        return isinstance(cache.layers[layer_idx], PackedCacheLayer)

    def _attach(self, cache, layer_idx: int, module: nn.Module, state) -> None:
        # a packed-only layer never takes the fake-key route with these indices (its masked fallback dequantises and
        # asks the state then), so the export of the evicted positions is skipped for it
        module.masked_key_indices = None if self._is_packed_layer(cache, layer_idx) else state.masked_key_indices()
        module._odmkv_state = state
        if hasattr(cache, "layers"):
            cache.layers[layer_idx]._tq_backend_state = state

    def _record_observed_ratios(self, layer_idx: int, bits: torch.Tensor) -> None:
        """Per-(layer, head) level fractions over the bulk region (kvquant/adaptive_backend_press.py:243-290)."""
        if bits.dim() != 3:
            return
        B, H_kv, T = bits.shape
        if T == 0:
            return
        start = min(int(self.sink_tokens), T) if self.sink_tokens > 0 else 0
        end = T - min(int(self.buffer_size), T) if self.buffer_size > 0 else T
        if end <= start:
            start, end = 0, T
        bulk = bits[..., start:end]
        T_bulk = bulk.shape[-1]
        if T_bulk == 0:
            return
        levels = sorted(set(self.bit_levels) | {16})
        lv = torch.tensor(levels, device=bits.device, dtype=bits.dtype)
        counts = (bulk.reshape(B * H_kv, T_bulk, 1) == lv.view(1, 1, -1)).sum(dim=1).cpu()   # one read-back
        status = getattr(self.scorer, "last_status", None)
        if status is not None and int(status.item()) != 0:   # already synchronised by the read-back above
            raise ops._lib.OdmkvError("the scorer reported an expired bounded wait: the scores of this layer are invalid")
        if bits.is_cuda and ops.quantize_status() != 0:      # the layers packed so far (the device is idle here anyway)
            raise ops._lib.OdmkvError("the quantise kernel reported an expired bounded wait: packed codes are invalid")
        for row_idx in range(B * H_kv):
            h = row_idx % H_kv
            row = counts[row_idx]
            total = int(row.sum())
            if total == 0:
                continue
            fr = (row.float() / total).tolist()
            self._observed_ratios[(layer_idx, h)] = tuple((b, f) for b, f in zip(levels, fr) if row[levels.index(b)] > 0)

    # ------------------------------------------------------------------ prefill
    def _score_layer(self, module, hidden_states, keys, values, layer_idx: int) -> torch.Tensor:
        """Scores [B, H, T] of one layer."""
        if isinstance(self.scorer, RiskScorer) and keys.is_cuda:
            scores = self.scorer.score_prefill_batched(keys, values, layer_idx, module=module, hidden_states=hidden_states)
            self._prefill_hooks_fired += keys.shape[0]
            return scores.float()
        out = []
        for b in range(keys.shape[0]):
            if self._score_prefill_supports_kwargs:
                s = self.scorer.score_prefill(keys[b], values[b], layer_idx, module=module, hidden_states=hidden_states[b:b + 1])
            else:
                s = self.scorer.score_prefill(keys[b], values[b], layer_idx)
            out.append(s)
            self._prefill_hooks_fired += 1
        return torch.stack(out, dim=0).float()

    def _compress_layer(self, cache, layer_idx: int, module, keys, values, bits: torch.Tensor) -> None:
        """Window override, quantise into the state, write dequantised tokens back (292-325)."""
        self._record_observed_ratios(layer_idx, bits)
        if layer_idx < self.initial_layers_fp16:
            bits = torch.full_like(bits, 16)
        elif self.buffer_size > 0:
            bits = bits.clone()
            bits[..., -min(self.buffer_size, bits.shape[-1]):] = 16
        state = self._get_or_create_state(layer_idx, keys)
        state.prefill(keys, values, bits.to(dtype=torch.int32, device=keys.device))
        if self.packed_cache and hasattr(cache, "layers") and keys.is_cuda:
            from .packed_cache import convert_layer
            convert_layer(cache.layers[layer_idx], state)   # no dense write-back: the packed state is the cache
            self._attach(cache, layer_idx, module, state)
            module._odmkv_packed_cache = True
            if self.buffer_size > 0:
                self._buffer_start_seqs[layer_idx] = int(state.seq_len)
                self._buffer_counts[layer_idx] = 0
            return
        if keys.is_contiguous() and values.is_contiguous():
            state.materialize_quantized_into(keys, values)
        else:
            k2, v2 = keys.contiguous(), values.contiguous()
            state.materialize_quantized_into(k2, v2)
            self._set_cache_tensors(cache, layer_idx, k2, v2)
        self._attach(cache, layer_idx, module, state)
        if self.buffer_size > 0:
            self._buffer_start_seqs[layer_idx] = int(keys.shape[2])
            self._buffer_counts[layer_idx] = 0

    def _finalize_global(self, cache) -> None:
        """``layerwise=False``: one Lagrangian per sample over all layers (kvquant/press.py:350-378)."""
        layers = sorted(self._prefill_scores)
        B = self._prefill_scores[layers[0]].shape[0]
        dev = self._prefill_scores[layers[0]].device
        flat = torch.cat([self._prefill_scores[i].reshape(B, -1).to(dev) for i in layers], dim=1)
        masks = []
        for i in layers:
            m = self._prefill_sink_masks[i]
            n = self._prefill_scores[i][0].numel()
            masks.append(torch.zeros(n, dtype=torch.bool, device=dev) if m is None else m.reshape(-1).to(dev))
        mask = torch.cat(masks) if any(self._prefill_sink_masks[i] is not None for i in layers) else None
        bits_all = self._compute_bits_batched(flat.unsqueeze(1), None if mask is None else mask.unsqueeze(0)).reshape(B, -1)
        cursor = 0
        for i in layers:
            shape = self._prefill_scores[i].shape
            n = int(self._prefill_scores[i][0].numel())
            keys, values = self._get_cache_tensors(cache, i)
            bits = bits_all[:, cursor:cursor + n].reshape(shape).to(keys.device)
            cursor += n
            self._compress_layer(cache, i, self._layer_modules[i], keys, values, bits)
        self._reset_prefill_state()

    # ------------------------------------------------------------------ hook
    def _forward_hook(self, module: nn.Module, args, kwargs, output):
        cache = kwargs.get("past_key_values")
        hidden_states = kwargs.get("hidden_states")
        if hidden_states is None and args:
            hidden_states = args[0]
        if cache is None or hidden_states is None:
            return output
        layer_idx = int(module.layer_idx)
        self._layer_modules[layer_idx] = module
        keys, values = self._get_cache_tensors(cache, layer_idx)
        if self._head_dim is None:
            self._head_dim = keys.shape[-1]
        q_len, cache_len = hidden_states.shape[1], keys.shape[2]
        packed = self._is_packed_layer(cache, layer_idx)   # keys / values are then the new tokens only

        if cache_len == q_len and not packed:       # fresh prefill
            scores = self._score_layer(module, hidden_states, keys, values, layer_idx)
            sink_mask = self._build_sink_mask(keys.shape[1], keys.shape[2], keys.device)
            if self.layerwise:
                bits = self._compute_bits_batched(scores, sink_mask)
                self._log_alloc(bits[0])
                self._compress_layer(cache, layer_idx, module, keys, values, bits)
            else:
                self._prefill_scores[layer_idx] = scores
                self._prefill_sink_masks[layer_idx] = sink_mask
                if self._last_hooked_layer_idx is None or layer_idx == self._last_hooked_layer_idx:
                    self._finalize_global(cache)
            return output

        if not self.decode_quant or layer_idx < self.initial_layers_fp16:
            return output

        state = self._get_or_create_state(layer_idx, keys)
        if self.buffer_size > 0:
            buf_start = self._buffer_start_seqs.get(layer_idx)
            if buf_start is not None and buf_start > state.seq_len:
                self._buffer_start_seqs[layer_idx] = state.seq_len
                self._buffer_counts[layer_idx] = 0
        new_k = keys[:, :, -q_len:, :]
        new_v = values[:, :, -q_len:, :]

        if self.buffer_size > 0:
            state.append_all_exact(new_k, new_v)
            if q_len > 1:
                # question-encoding pass: part of the prompt, pinned exact and never re-quantised (407-418)
                self._buffer_start_seqs[layer_idx] = state.seq_len
                self._attach(cache, layer_idx, module, state)
                return output
            self._buffer_counts[layer_idx] = self._buffer_counts.get(layer_idx, 0) + q_len
            if self._buffer_counts[layer_idx] >= self.buffer_size:
                self._flush_decode_buffer(state, layer_idx, cache, module, hidden_states)
                return output
            self._attach(cache, layer_idx, module, state)
            return output

        # no decode buffer: score the new tokens and route them at once (426-443)
        batch_bits = []
        for b in range(keys.shape[0]):
            if q_len == 1:
                s = self.scorer.score_decode(new_k[b, :, 0, :], new_v[b, :, 0, :], layer_idx, module=module,
                                             hidden_states=hidden_states[b:b + 1]).unsqueeze(-1)
            else:
                s = self.scorer.score_prefill(new_k[b], new_v[b], layer_idx, module=module, hidden_states=hidden_states[b:b + 1])
            batch_bits.append(scores_to_bits(s, self._decode_bit_levels))
        bits = torch.stack(batch_bits, dim=0).to(dtype=torch.int32, device=keys.device)
        n_before = len(state.chunks)
        state.append(new_k.contiguous(), new_v.contiguous(), bits)
        if not packed:
            k2, v2 = keys.contiguous(), values.contiguous()
            state.materialize_quantized_into(k2, v2, chunks=state.chunks[n_before:])
            self._set_cache_tensors(cache, layer_idx, k2, v2)
        self._attach(cache, layer_idx, module, state)
        return output

    # ------------------------------------------------------------------ decode-buffer flush
    @torch.no_grad()
    def _flush_attention(self, module, hidden_states, buf_keys: torch.Tensor, state) -> Optional[torch.Tensor]:
        """Softmax of the current (GQA-mean, RoPE'd) query over the buffered keys of every (b, h):
        buf_keys [B, H, n, d] -> [B, H, n] (kvquant/adaptive_backend_press.py:601-665)."""
        if hidden_states is None:
            return None
        try:
            q = _get_query_states(module, hidden_states)
        except (AttributeError, NotImplementedError, ValueError):
            return None
        rotary_emb = getattr(module, "rotary_emb", None)
        if rotary_emb is not None:
            pos = torch.arange(state.seq_len - 1, state.seq_len, device=q.device).unsqueeze(0)
            cos, sin = _aligned_rotary_outputs(rotary_emb, q, pos)
            q = _apply_rotary_pos_emb_q(q, cos, sin)
        B, Hq, _, d = q.shape
        H = state.num_heads
        q_kv = q[:, :, -1, :].reshape(B, H, Hq // H, d).mean(dim=2)
        logits = torch.einsum("bhd,bhnd->bhn", q_kv, buf_keys) / math.sqrt(d)
        return torch.softmax(logits, dim=-1)

    def _allocate_bits_via_cached_ratios(self, scores: torch.Tensor, layer_idx: int, allowed: set) -> Optional[torch.Tensor]:
        """Rank tiers per head from the prefill's level fractions; every sample of a head is pooled in
        (b, t) order as in the reference (kvquant/adaptive_backend_press.py:198-241, kvquant/allocator.py:46-148):
        ascending stable rank, tier sizes ``int(round(r * n))`` (Python's rounding), the last tier of a head takes the
        remainder.  scores [B, H, n].  All heads go through one sort: the tier sizes are host arithmetic, the ranks
        are compared with per-head cumulative sizes on the device."""
        B, H, n = scores.shape
        if not all((layer_idx, h) in self._observed_ratios for h in range(H)):
            return None
        n_pool = B * n
        levels = sorted(allowed)
        ends = []
        for h in range(H):
            filt = sorted((b, r) for b, r in self._observed_ratios[(layer_idx, h)] if b in allowed and r > 0)
            if not filt:
                return None
            total = sum(r for _, r in filt)
            count = {}
            cursor = 0
            for i, (b, r) in enumerate(filt):
                c = n_pool - cursor if i == len(filt) - 1 else min(int(round(r / total * n_pool)), n_pool - cursor)
                count[b] = c
                cursor += c
            acc, row = 0, []
            for b in levels:             # levels a head does not use are empty tiers
                acc += count.get(b, 0)
                row.append(acc)
            ends.append(row)
        dev = scores.device
        pooled = scores.permute(1, 0, 2).reshape(H, n_pool)
        order = torch.argsort(pooled, dim=1, stable=True)
        ranks = torch.empty_like(order)
        ranks.scatter_(1, order, torch.arange(n_pool, device=dev).expand(H, n_pool))
        tier = torch.searchsorted(torch.tensor(ends, device=dev, dtype=torch.int64), ranks, right=True)
        bits = torch.tensor(levels, device=dev, dtype=torch.int32)[tier.clamp_(max=len(levels) - 1)]
        return bits.view(H, B, n).permute(1, 0, 2).contiguous()

    def _flush_decode_buffer(self, state, layer_idx: int, cache, module, hidden_states=None) -> None:
        """Score the buffered decode tokens and re-quantise them (kvquant/adaptive_backend_press.py:464-595)."""
        buffer_start = self._buffer_start_seqs.get(layer_idx)
        if buffer_start is None:
            self._attach(cache, layer_idx, module, state)
            return
        buf_k, buf_v = state.buffer_view(buffer_start)
        n_buf = 0 if buf_k is None else buf_k.shape[2]
        if n_buf == 0:
            self._buffer_start_seqs[layer_idx] = state.seq_len
            self._buffer_counts[layer_idx] = 0
            self._attach(cache, layer_idx, module, state)
            return
        B, H = state.batch_size, state.num_heads
        attn = self._flush_attention(module, hidden_states, buf_k, state)
        if attn is not None and self.scorer is not None:
            kf = buf_k.reshape(B * H, n_buf, -1)
            vf = buf_v.reshape(B * H, n_buf, -1)
            scores = self.scorer.score_with_attn(kf, vf, attn.reshape(B * H, n_buf), module=module).float().reshape(B, H, n_buf)
        elif attn is not None:
            scores = attn.pow(2) * buf_v.float().pow(2).sum(-1)
        else:
            scores = buf_k.float().pow(2).sum(-1) + buf_v.float().pow(2).sum(-1)
        lo, hi = scores.min(), scores.max()
        scores = (scores - lo) / (hi - lo) if (hi - lo) > 1e-8 else torch.full_like(scores, 0.5)

        levels = self._decode_bit_levels
        allowed = set(levels)
        bits = None
        if self.ratios is not None:
            pairs = [(b, r) for b, r in zip(self.bit_levels, self.ratios) if b in allowed]
            if pairs:
                lv, rt = zip(*pairs)
                bits = ratio_scores_to_bits(scores.reshape(-1), tuple(lv), tuple(rt), per_head=False).reshape(B, H, n_buf)
        elif self.target_avg_bits is not None:
            bits = self._allocate_bits_via_cached_ratios(scores, layer_idx, allowed)
            if bits is None:
                eps = self._ensure_epsilon(scores.device)
                bits = optimal_scores_to_bits(scores.reshape(-1), levels, self.target_avg_bits, {b: eps.get(b, 0.0) for b in levels},
                                              eviction_cost=self.eviction_cost, head_dim=self._head_dim or 128,
                                              outlier_min_bits=self.outlier_min_bits,
                                              above_target_alpha=self.above_target_alpha).reshape(B, H, n_buf)
        if bits is None:
            bits = scores_to_bits(scores, levels)
        chunk = state.flush_buffer(buffer_start, bits)
        self._buffer_start_seqs[layer_idx] = state.seq_len
        self._buffer_counts[layer_idx] = 0
        if chunk is not None and not self._is_packed_layer(cache, layer_idx):
            keys, values = self._get_cache_tensors(cache, layer_idx)
            if keys.shape[2] >= state.seq_len:
                k2, v2 = keys.contiguous(), values.contiguous()
                state.materialize_quantized_into(k2, v2, chunks=[chunk])
                if k2 is not keys:
                    self._set_cache_tensors(cache, layer_idx, k2, v2)
        self._attach(cache, layer_idx, module, state)

    # ------------------------------------------------------------------ context manager
    @contextlib.contextmanager
    def __call__(self, model):
        """Patch the attention functions, register a forward hook on every attention layer, yield, clean up
        (kvquant/press.py:637-692, kvquant/adaptive_backend_press.py:667-682)."""
        lm = model
        if hasattr(lm, "model"):
            lm = lm.model
        if hasattr(lm, "language_model"):
            lm = lm.language_model
        self._states, self._buffer_counts, self._buffer_start_seqs = {}, {}, {}
        patch_attention_functions()
        self._reset_prefill_state()
        self._hooked_layer_indices, self._last_hooked_layer_idx, self._layer_modules = [], None, {}
        hooks = []
        try:
            for i, layer in enumerate(lm.layers):
                attn = getattr(layer, "self_attn", None)
                if attn is None or getattr(attn, "is_sliding", False):
                    continue
                if not hasattr(attn, "layer_idx"):
                    attn.layer_idx = i
                attn.masked_key_indices = None
                attn._odmkv_state = None
                attn._odmkv_packed_cache = False
                if hasattr(lm, "rotary_emb"):
                    try:
                        attn.rotary_emb = lm.rotary_emb
                    except Exception:
                        pass
                self._hooked_layer_indices.append(i)
                hooks.append(attn.register_forward_hook(self._forward_hook, with_kwargs=True))
            self._last_hooked_layer_idx = self._hooked_layer_indices[-1] if self._hooked_layer_indices else None
            yield
        finally:
            for h in hooks:
                h.remove()
            used = bool(self._states)
            # the eviction mask and packed state stay on the modules: they must keep acting during decode
            # steps issued outside the context manager; the next fresh prefill clears them.
            self._hooked_layer_indices, self._last_hooked_layer_idx, self._layer_modules = [], None, {}
            self._reset_prefill_state()
            self._states, self._buffer_counts, self._buffer_start_seqs = {}, {}, {}
        # a normal exit: the packing of the last layers has not been checked yet (this synchronises once)
        if used and torch.cuda.is_available() and ops.quantize_status() != 0:
            raise ops._lib.OdmkvError("the quantise kernel reported an expired bounded wait: packed codes are invalid")
