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

__all__ = ["PackedCacheLayer", "convert_layer", "GraphedDecoder"]


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


class GraphedDecoder:
    """Single-token decode steps of a model under the press, replayed from a CUDA graph.

    The reference's runner issues one eager forward pass per generated token (benchmark/core/pipeline.py:164-209),
    which for a small batch is bound by the host launching a few hundred kernels per step.  With every layer on a
    ``PackedCacheLayer`` the step has no shape that grows: the packed chunks are immutable between two flushes of
    the decode buffer and the tail is a preallocated buffer whose length lives in device memory
    (``TurboQuantAdaptiveKVCacheState.begin_device_tail``), so one captured step stays valid until the next flush.
    ``step`` replays it, advances the host-side counters the press hook would have advanced, and falls back to an
    eager pass for the step that flushes (scoring and re-quantisation run host logic); the step after a flush is
    captured again over the new chunk list.

    The batch must be free of padding (no attention mask that hides keys): a captured step cannot inspect a mask.
    ``step`` returns a buffer that the next replay overwrites.

    Use inside ``with press(model):`` after the prefill, with ``packed_cache=True``::

        dec = GraphedDecoder(model, press, cache)
        logits = dec.step(next_tokens)          # [B, 1] token ids on the device -> [B, 1, vocab]
    """

    def __init__(self, model, press, cache):
        self.model, self.press, self.cache = model, press, cache
        self.graph = None
        self.logits = None
        self.ids = None
        self.pos = None
        self._warm = False
        self._expected = None
        self.captures = 0
        self.replays = 0
        self.eager_steps = 0

    # -- bookkeeping -------------------------------------------------------------------------
    def _layer_states(self):
        states = self.press._states
        return [(i, states[i]) for i in sorted(states)]

    def _replayable(self) -> bool:
        press, layers = self.press, getattr(self.cache, "layers", None)
        if layers is None or not press._states or not press.decode_quant or press.buffer_size <= 1:
            return False
        for i, layer in enumerate(layers):
            st = press._states.get(i)
            if not isinstance(layer, PackedCacheLayer) or st is None or getattr(layer, "_tq_backend_state", None) is not st:
                return False
            if press._buffer_counts.get(i, 0) + 1 >= press.buffer_size:      # this step fills the buffer: it flushes
                return False
            start = press._buffer_start_seqs.get(i)
            if start is None or start > st.seq_len:                            # the hook would rewind its counters
                return False
        return True

    def _room(self) -> int:
        press = self.press
        return min(press.buffer_size - 1 - press._buffer_counts.get(i, 0) for i, _ in self._layer_states())

    def _signature(self):
        """What the captured step assumes about every state: lengths and the identity of the chunk list."""
        return [(st.seq_len, st.tail_len, st.tail_start, tuple(id(c) for c in st.chunks)) for _, st in self._layer_states()]

    def drop_graph(self) -> None:
        """Forget the captured step (after anything that changes a state: a flush, a rewind, a new prefill)."""
        if self.graph is not None:
            self.graph = None
            self.logits = None
        for _, st in self._layer_states():
            st.end_device_tail()

    def _forward(self, ids, pos=None):
        if pos is None:
            return self.model(input_ids=ids, past_key_values=self.cache, use_cache=True).logits
        B = ids.shape[0]
        return self.model(input_ids=ids, position_ids=pos.view(1, 1).expand(B, 1), cache_position=pos,
                          past_key_values=self.cache, use_cache=True).logits

    def _capture(self, tokens: torch.Tensor) -> None:
        press = self.press
        dev = tokens.device
        if self.ids is None or self.ids.shape != tokens.shape:
            self.ids = torch.zeros_like(tokens)
            self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        room = self._room()
        pairs = self._layer_states()
        for _, st in pairs:
            st.begin_device_tail(room)
            for chunk in st.chunks:
                chunk.stored_tokens()        # host-side counts are read once, before the capture (it may not copy)
        snap = [(st.seq_len, st.tail_len, st.tail_start) for _, st in pairs]
        counts, starts = dict(press._buffer_counts), dict(press._buffer_start_seqs)
        self.pos.fill_(pairs[0][1].seq_len)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        # recording runs the host side of the step once (hooks included) without executing a kernel: the host
        # counters it advanced are put back, the device counter did not move
        modules = list(press._layer_modules.values())
        for m in modules:
            m._odmkv_mask_known_open = True      # no padding in a batch decoded this way: the mask cannot hide a key
        try:
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.logits = self._forward(self.ids, self.pos)
        finally:
            for m in modules:
                m._odmkv_mask_known_open = False
        for (_, st), (sl, tl, ts) in zip(pairs, snap):
            st.seq_len, st.tail_len, st.tail_start = sl, tl, ts
        press._buffer_counts.clear()
        press._buffer_counts.update(counts)
        press._buffer_start_seqs.clear()
        press._buffer_start_seqs.update(starts)
        self.graph = graph
        self._expected = self._signature()
        self.captures += 1

    # -- the step ----------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        if not self._warm or not self._replayable():
            # the first step (library handles, helper stream, kernel attributes) and every flushing step run eagerly
            self.drop_graph()
            self._warm = True
            self.eager_steps += 1
            return self._forward(tokens)
        if self.graph is not None and self._signature() != self._expected:
            self.drop_graph()            # someone changed a state in between (a rewind, an eager step): capture again
        if self.graph is None or self.ids.shape != tokens.shape:
            self.drop_graph()
            self._capture(tokens)
        pairs = self._layer_states()
        self.ids.copy_(tokens)
        self.pos.fill_(pairs[0][1].seq_len)
        self.graph.replay()
        for i, st in pairs:
            st.advance_host(1)
            self.press._buffer_counts[i] = self.press._buffer_counts.get(i, 0) + 1
        self.replays += 1
        self._expected = self._signature()
        return self.logits
