"""KV-unit scorers (mirrors the reference's ``kvquant/scorer.py`` and ``kvquant/attention_utils.py``).

``RiskScorer`` computes ``s = (p + eps)^2 (|v|^2 + |k|^2/d |v - o|^2)`` with the CUDA scorer kernels;
only the small query statistics (a projection of the mean hidden state and the averaged RoPE) are
tensor operations on the host side.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Optional

import torch
from torch import nn

from . import ops

__all__ = ["BaseScorer", "ExpectedAttentionScorer", "RiskScorer", "_chunked_attention_qk"]


# ---- attention helpers (kvquant/attention_utils.py) ---------------------------------------------

def _repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    if n_rep == 1:
        return hidden_states
    b, h, s, d = hidden_states.shape
    return hidden_states[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)


def _module_heads(module: nn.Module, hidden_dim: int) -> tuple[int, int]:
    cfg = getattr(module, "config", None)
    num_heads = getattr(module, "num_heads", None)
    if num_heads is None and cfg is not None:
        num_heads = getattr(cfg, "num_attention_heads", None)
    if num_heads is None:
        raise AttributeError(f"Cannot determine num_heads from {module.__class__.__name__}")
    head_dim = getattr(module, "head_dim", None)
    if head_dim is None and cfg is not None:
        head_dim = getattr(cfg, "head_dim", None)
    if head_dim is None:
        head_dim = hidden_dim // num_heads
    return int(num_heads), int(head_dim)


def _get_query_states(module: nn.Module, hidden_states: torch.Tensor) -> torch.Tensor:
    """q_proj (+ q_norm) of every position, [B, Hq, T, d] (kvquant/attention_utils.py:29-54)."""
    bsz, q_len, _ = hidden_states.shape
    num_heads, head_dim = _module_heads(module, hidden_states.shape[-1])
    if hasattr(module, "qkv_proj"):
        q = module.qkv_proj(hidden_states)[..., : num_heads * head_dim]
    elif hasattr(module, "q_proj"):
        q = module.q_proj(hidden_states)
    else:
        raise NotImplementedError(f"ExpectedAttentionScorer does not support {module.__class__.__name__}.")
    q = q.view(bsz, q_len, num_heads, head_dim).transpose(1, 2)
    if hasattr(module, "q_norm"):
        q = module.q_norm(q)
    return q


def _aligned_rotary_outputs(rotary_emb, x: torch.Tensor, position_ids: torch.Tensor):
    cos, sin = rotary_emb(x, position_ids)
    return cos.to(device=x.device, dtype=x.dtype), sin.to(device=x.device, dtype=x.dtype)


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _apply_rotary_pos_emb_q(q: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    if cos.dim() == 2:
        cos, sin = cos.unsqueeze(0), sin.unsqueeze(0)
    return (q * cos.unsqueeze(1)) + (_rotate_half(q) * sin.unsqueeze(1))


def _apply_avg_rope(module: nn.Module, mu: torch.Tensor, cov, q_len: int, n_future_positions: int):
    """mu' = R mu with R the mean over the next ``n_future_positions`` positions of the RoPE matrices
    (kvquant/attention_utils.py:57-115), in its elementwise form
    mu'_i = mean(cos)_i mu_i + mean(sin)_i rotate_half(mu)_i.  The covariance path is not implemented."""
    rotary_emb = getattr(module, "rotary_emb", None)
    if rotary_emb is None or n_future_positions <= 0:
        return mu, cov
    if cov is not None:
        raise NotImplementedError("covariance statistics are not implemented")
    position_ids = torch.arange(q_len, q_len + n_future_positions, device=mu.device).unsqueeze(0)
    cos, sin = _aligned_rotary_outputs(rotary_emb, mu, position_ids)
    cos_bar, sin_bar = cos[0].mean(dim=0), sin[0].mean(dim=0)
    return cos_bar * mu + sin_bar * _rotate_half(mu), None


def mean_query_states(module: nn.Module, hidden_states: torch.Tensor, n_sink: int) -> torch.Tensor:
    """Mean over the positions after the sinks of the projected queries, fp32 [B, Hq, d]
    (kvquant/scorer.py:184-195).  For a plain linear ``q_proj`` without ``q_norm`` the mean commutes with
    the projection, so only the mean hidden state is projected instead of every position."""
    h = hidden_states[:, n_sink:]
    num_heads, head_dim = _module_heads(module, hidden_states.shape[-1])
    proj = getattr(module, "q_proj", None)
    if isinstance(proj, nn.Linear) and not hasattr(module, "q_norm") and not hasattr(module, "qkv_proj"):
        hm = h.float().mean(dim=1)
        bias = None if proj.bias is None else proj.bias.float()
        mu = torch.nn.functional.linear(hm, proj.weight.float(), bias)
        return mu.view(h.shape[0], num_heads, head_dim)
    return _get_query_states(module, h).float().mean(dim=2)


# ---- scorers --------------------------------------------------------------------------------------

def _chunked_attention_qk(query_states: torch.Tensor, expanded_keys_t: torch.Tensor, T_kv: int, H_kv: int, n_groups: int,
                          scale: float, chunk_size: int, device, dtype):
    """Attention statistics per KV position, same signature and result as the reference's helper
    (kvquant/attention_utils.py:160-211): ``query_states`` [1, H_q, T_q, d], ``expanded_keys_t`` [1, H_q, d, T_kv] (the
    G-expanded, transposed keys the reference multiplies with) -> ``(sum_attn, max_attn, sum_sq_attn)``, each
    [H_kv, T_kv] in ``dtype``.  One pass of the tensor-core kernels (``ops.window_attn_stats``); ``chunk_size`` only
    bounded the reference's temporaries and is ignored."""
    if query_states.dim() != 4 or query_states.shape[0] != 1 or expanded_keys_t.shape[-1] != T_kv:
        raise ValueError("expected query_states [1, H_q, T_q, d] and expanded_keys_t [1, H_q, d, T_kv]")
    keys = expanded_keys_t[:, ::n_groups].transpose(-1, -2)                       # [1, H_kv, T_kv, d]
    if keys.shape[1] != H_kv:
        raise ValueError(f"expanded keys hold {expanded_keys_t.shape[1]} heads, expected {H_kv} x {n_groups}")
    cdt = query_states.dtype if query_states.dtype in (torch.float16, torch.bfloat16) else torch.float16
    s, m, q = ops.window_attn_stats(query_states.to(device=device, dtype=cdt), keys.to(device=device, dtype=cdt), scale=scale)
    return s[0].to(dtype), m[0].to(dtype), q[0].to(dtype)


def _normalize_scores(raw: torch.Tensor, *, grain: str = "layer") -> torch.Tensor:
    """Min-max normalisation with the reference's grains (kvquant/scorer.py:100-135)."""
    if raw.numel() == 0 or grain == "global":
        return raw
    if grain == "head" and raw.dim() >= 2:
        lo, hi = raw.amin(dim=-1, keepdim=True), raw.amax(dim=-1, keepdim=True)
        denom = hi - lo
        out = (raw - lo) / torch.where(denom < 1e-8, torch.ones_like(denom), denom)
        dead = denom.squeeze(-1) < 1e-8
        if dead.any():
            out[dead] = 0.5
        return out
    lo, hi = raw.min(), raw.max()
    if (hi - lo) < 1e-8:
        return torch.full_like(raw, 0.5)
    return (raw - lo) / (hi - lo)


class BaseScorer(ABC):
    """Interface every scorer implements (kvquant/scorer.py:29-97)."""

    normalize_grain: str = "layer"

    def _maybe_normalize(self, raw: torch.Tensor) -> torch.Tensor:
        return _normalize_scores(raw, grain=self.normalize_grain)

    @abstractmethod
    def score_prefill(self, keys, values, layer_idx, *, module=None, hidden_states=None) -> torch.Tensor:
        """Scores [H, T] for this layer's tokens (keys, values [H, T, d])."""

    def score_decode(self, key, value, layer_idx, *, module=None, hidden_states=None) -> torch.Tensor:
        return torch.ones(key.shape[0], device=key.device)

    def score_with_attn(self, keys, values, attn_weights, *, module=None) -> torch.Tensor:
        eps = float(getattr(self, "epsilon", 0.0) or 0.0)
        return (attn_weights + eps).pow(2) * values.float().pow(2).sum(dim=-1)


class _NormFallback(BaseScorer):
    def score_prefill(self, keys, values, layer_idx, *, module=None, hidden_states=None):
        return self._maybe_normalize(keys.norm(dim=-1) + values.norm(dim=-1))

    def score_decode(self, key, value, layer_idx, *, module=None, hidden_states=None):
        return self._maybe_normalize(key.norm(dim=-1) + value.norm(dim=-1))


class ExpectedAttentionScorer(BaseScorer):
    """Holds the query-statistics machinery shared with ``RiskScorer`` (kvquant/scorer.py:154-274).
    Its own covariance-based score is not implemented; ``RiskScorer`` is the scorer the experiments build."""

    def __init__(self, *, n_future_positions: int = 512, n_sink: int = 4, use_covariance: bool = True,
                 use_vnorm: bool = True, epsilon: float = 0.0):
        self.n_future_positions = n_future_positions
        self.n_sink = n_sink
        self.use_covariance = use_covariance
        self.use_vnorm = use_vnorm
        self.epsilon = epsilon
        self._fallback = _NormFallback()

    def _query_statistics(self, module: nn.Module, hidden_states: torch.Tensor):
        q_len = hidden_states.shape[1]
        if q_len <= self.n_sink:
            raise ValueError("not enough tokens to estimate expected attention")
        if self.use_covariance:
            raise NotImplementedError("covariance statistics are not implemented")
        mu = mean_query_states(module, hidden_states, self.n_sink)
        return _apply_avg_rope(module, mu, None, q_len, self.n_future_positions)

    def score_prefill(self, keys, values, layer_idx, *, module=None, hidden_states=None):
        raise NotImplementedError("use RiskScorer; the covariance-based expected-attention score is not implemented")

    def score_decode(self, key, value, layer_idx, *, module=None, hidden_states=None):
        return self._fallback.score_decode(key, value, layer_idx, module=module, hidden_states=hidden_states)


class RiskScorer(ExpectedAttentionScorer):
    """s = p^2 [ |v|^2 + (|k|^2 / d) |v - o|^2 ]  (kvquant/scorer.py:363-416)."""

    def __init__(self, **kw):
        kw["use_covariance"] = False
        super().__init__(**kw)

    def score_prefill_batched(self, keys: torch.Tensor, values: torch.Tensor, layer_idx: int, *, module: nn.Module,
                              hidden_states: torch.Tensor) -> torch.Tensor:
        """All samples of a layer in one launch: keys/values [B, H, T, d], hidden_states [B, T, hidden]
        -> scores [B, H, T] fp32.  Same result as calling ``score_prefill`` per sample."""
        if keys.shape[2] <= self.n_sink:
            return torch.ones(keys.shape[:3], device=keys.device, dtype=keys.dtype)
        try:
            mu, _ = self._query_statistics(module, hidden_states)
        except (AttributeError, NotImplementedError, ValueError):
            # same defensive fallback as the reference (kvquant/scorer.py:390-393): norm scoring
            return torch.stack([self._fallback.score_prefill(k, v, layer_idx) for k, v in zip(keys, values)])
        # the sweeps' status word (non-zero: a bounded wait expired, scores invalid) is kept for the caller to read
        # where it synchronises anyway (the press does, when it records the level ratios)
        scores, self.last_status = ops.score_prefill(keys, values, mu.float(), self.n_sink, float(self.epsilon), return_status=True)
        return scores if self.normalize_grain == "global" else torch.stack([self._maybe_normalize(s) for s in scores])

    def score_prefill(self, keys, values, layer_idx, *, module=None, hidden_states=None):
        if module is None or hidden_states is None:
            return self._fallback.score_prefill(keys, values, layer_idx)
        if keys.shape[1] <= self.n_sink:
            return torch.ones(keys.shape[:2], device=keys.device, dtype=keys.dtype)
        if hidden_states.dim() == 2:
            hidden_states = hidden_states.unsqueeze(0)
        return self.score_prefill_batched(keys.unsqueeze(0), values.unsqueeze(0), layer_idx, module=module,
                                          hidden_states=hidden_states)[0]

    def score_with_attn(self, keys, values, attn_weights, *, module=None):
        return ops.score_with_attn(keys, values, attn_weights, float(self.epsilon))

    def score_windowed(self, keys: torch.Tensor, values: torch.Tensor, query_window: torch.Tensor) -> torch.Tensor:
        """Risk scores from the attention the last W queries actually pay: keys / values [H, T, d], ``query_window``
        [H_q, W, d] = the position-encoded queries of positions T - W .. T - 1 -> scores [H, T] fp32.  The reference
        ships the two halves of this -- the column sums of causal softmax attention (kvquant/attention_utils.py:160-211)
        and the risk formula for given weights (kvquant/scorer.py:406-416) -- and this method composes them: the
        weight of key j is its column sum divided by the number of window queries that can see it."""
        H, T, _ = keys.shape
        W = int(query_window.shape[1])
        if W < 1 or W > T:
            raise ValueError(f"window of {W} queries over {T} keys")
        cdt = keys.dtype if keys.dtype in (torch.float16, torch.bfloat16) else torch.float16
        s, _, _ = ops.window_attn_stats(query_window.unsqueeze(0).to(cdt), keys.unsqueeze(0).to(cdt), q_offset=T - W)
        pos = torch.arange(T, device=keys.device)
        seen_by = (W - (pos - (T - W)).clamp(min=0)).to(torch.float32)          # queries r with j <= r + (T - W)
        return ops.score_with_attn(keys, values, s[0] / seen_by, float(self.epsilon))
