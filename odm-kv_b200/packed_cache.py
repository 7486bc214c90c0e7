"""Cache layer that stops carrying the dense keys and values once a layer is compressed.

transformers' ``DynamicLayer.update`` concatenates every new token onto dense ``[B, H, T, d]`` tensors
(``transformers/cache_utils.py``, ``DynamicLayer.update``), which costs O(T) bytes per token and layer and keeps the
uncompressed cache resident; the reference press inherits that and also writes the dequantised tokens back into those
tensors (kvquant/adaptive_backend_press.py:131-149).  With ``packed_cache=True`` the press converts a layer to this
class right after compressing it: the packed state (chunks plus a preallocated tail) is the only store, ``update``
hands the new tokens straight to the attention override, and ``keys`` / ``values`` are the newest tokens only -- a
small dense view that keeps code like the runner's cache rewind working (it slices ``keys`` / ``values`` and calls
``_tq_backend_state.truncate``; benchmark/core/pipeline.py:211-228).
"""
from __future__ import annotations

import torch
from transformers.cache_utils import DynamicLayer

__all__ = ["PackedCacheLayer", "convert_layer"]


class PackedCacheLayer(DynamicLayer):
    """``DynamicLayer`` whose sequence lives in ``_tq_backend_state``."""

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
        # no concatenation: the attention override attends the packed state plus these tokens, and the press hook
        # appends them to the state's tail afterwards
        self.keys, self.values = key_states, value_states
        return key_states, value_states

    def get_seq_length(self) -> int:
        state = getattr(self, "_tq_backend_state", None)
        return 0 if state is None else int(state.seq_len)

    def crop(self, max_length: int) -> None:
        state = getattr(self, "_tq_backend_state", None)
        if state is None:
            return
        if max_length < 0:
            max_length = state.seq_len - abs(max_length)
        state.truncate(max_length)

    def dense_view(self):
        """Dequantised dense cache [B, H, seq_len, d] (evicted rows zero): for callers that need the reference's layout."""
        return self._tq_backend_state.materialize()


def convert_layer(layer, state) -> None:
    """Turn a filled ``DynamicLayer`` into a ``PackedCacheLayer`` in place and release its dense tensors."""
    layer.__class__ = PackedCacheLayer
    layer._tq_backend_state = state
    empty = torch.empty(state.batch_size, state.num_heads, 0, state.head_dim, dtype=state.dtype, device=state.device)
    layer.keys, layer.values = empty, empty.clone()
