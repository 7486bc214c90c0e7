"""Attention-function override (mirrors the reference's ``kvquant/attention_patch.py``).

Every entry of transformers' ``ALL_ATTENTION_FUNCTIONS`` is wrapped once.  For a decode step
(one new query per sequence) on a layer whose cache carries a packed state, the wrapper answers
with this library's decode-attention kernels, which read the packed banks directly and never see
evicted tokens.  In every other case it behaves as the reference wrapper: prefill clears the eviction
mask, and calls that still go to the stock function get a fake key written over the evicted positions
so that ``exp(q . k)`` vanishes there (kvquant/attention_patch.py:13-55).
"""
from __future__ import annotations

import functools

import torch

_PATCH_ATTR = "_kvtoken_quant_attention_patched"


def search_hyperplane(x: torch.Tensor, max_iter: int = 1000) -> torch.Tensor:
    """A key k with exp(<q, k>) ~= 0 for every query q in x: -1e5 * y / |y|^2 for a y with <q, y> > 0."""
    orig_dtype = x.dtype
    x = x.float()
    y = x.mean(dim=1)
    for _ in range(max_iter):
        mask = torch.bmm(x, y.unsqueeze(-1)) <= 0
        if not mask.any():
            return (-1e5 * y / y.norm(dim=-1, keepdim=True) ** 2).to(orig_dtype)
        y = y + (x * mask).sum(dim=1) / mask.sum(dim=1).clamp(min=1)
    raise ValueError("Could not find fake keys such that exp(<q, k>) ~= 0")


def packed_decode(module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scaling):
    """Decode attention over ``module._odmkv_state`` for query [B, Hq, 1, d].  Tokens that the running
    forward pass has already appended to the dense cache but the press hook has not yet stored
    (normally the one new token) are attended from ``key`` / ``value``."""
    state = module._odmkv_state
    n_new = key.shape[2] - state.seq_len
    pend_k = key[:, :, state.seq_len:, :] if n_new > 0 else None
    pend_v = value[:, :, state.seq_len:, :] if n_new > 0 else None
    out = state.decode_attention(query[:, :, 0, :], scale=scaling, pending_k=pend_k, pending_v=pend_v, out_dtype=query.dtype)
    return out.unsqueeze(1)   # [B, 1, Hq, d], the layout attention functions return


def packed_multi(module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, scaling):
    """A pass of several new tokens (question encoding) over a layer whose cache is packed only: query j attends the
    packed state and the new tokens 0..j, one decode call per query.  ``key`` / ``value`` hold the new tokens only."""
    state = module._odmkv_state
    outs = []
    for j in range(query.shape[2]):
        outs.append(state.decode_attention(query[:, :, j, :], scale=scaling, pending_k=key[:, :, : j + 1, :],
                                           pending_v=value[:, :, : j + 1, :], out_dtype=query.dtype))
    return torch.stack(outs, dim=1)   # [B, q_len, Hq, d]


def _mask_is_open(attention_mask) -> bool:
    """True when the mask hides no key from the query (no padding in the batch).  The packed decode kernels take
    no mask, so a call with hidden keys keeps the reference's route (fake keys + stock attention)."""
    if attention_mask is None:
        return True
    if attention_mask.dtype == torch.bool:
        return bool(attention_mask.all())
    return not bool((attention_mask != 0).any())


def _causal_or_open(attention_mask, q_len: int) -> bool:
    """True when, over the packed tokens (all but the last q_len key columns), the mask hides nothing -- i.e. it is
    absent or plain causal, which ``packed_multi`` applies itself."""
    if attention_mask is None:
        return True
    old = attention_mask[..., : attention_mask.shape[-1] - q_len]
    if old.numel() == 0:
        return True
    if attention_mask.dtype == torch.bool:
        return bool(old.all())
    return not bool((old != 0).any())


def _attention_patch(func):
    if getattr(func, _PATCH_ATTR, False):
        return func

    @functools.wraps(func)
    def wrapper(module, query, key, value, attention_mask, dropout, **kwargs):
        state = getattr(module, "_odmkv_state", None)
        if state is not None and getattr(module, "_odmkv_packed_cache", False) and query.is_cuda:
            # the layer's cache is packed only: key / value are the new tokens, everything older is in the state
            scaling = kwargs.get("scaling", None)
            if scaling is None:
                scaling = getattr(module, "scaling", None)
            # (a step that is being captured into a graph may not read the mask back; its caller vouches that the
            #  batch has no padding, and a single new token then sees every key)
            if query.shape[2] == 1 and (getattr(module, "_odmkv_mask_known_open", False) or _mask_is_open(attention_mask)):
                out = state.decode_attention(query[:, :, 0, :], scale=scaling, pending_k=key, pending_v=value, out_dtype=query.dtype)
                return out.unsqueeze(1), None
            if _causal_or_open(attention_mask, query.shape[2]):
                return packed_multi(module, query, key, value, scaling), None
            # a mask that hides keys (padding in the batch): dense dequantised cache plus the new tokens, then the
            # reference's route below (fake keys over the evicted positions, stock attention)
            Kd, Vd = state.materialize()
            key = torch.cat([Kd.to(key.dtype), key], dim=2)
            value = torch.cat([Vd.to(value.dtype), value], dim=2)
            module.masked_key_indices = state.masked_key_indices()   # packed layers do not carry them otherwise
            dense_from_packed = True
        else:
            dense_from_packed = False
        if query.shape[2] == key.shape[2] and not dense_from_packed:
            module.masked_key_indices = None
            module._odmkv_state = None
            module._odmkv_packed_cache = False
        elif (state is not None and query.shape[2] == 1 and query.is_cuda and key.shape[2] >= state.seq_len
              and getattr(module, "_odmkv_decode", True) and _mask_is_open(attention_mask)):
            scaling = kwargs.get("scaling", None)
            if scaling is None:
                scaling = getattr(module, "scaling", None)
            return packed_decode(module, query, key, value, scaling), None
        elif getattr(module, "masked_key_indices", None) is not None:
            bsz, num_heads, seq_len, head_dim = query.shape
            num_key_value_heads = key.shape[1]
            num_groups = num_heads // num_key_value_heads
            q = query.view(bsz, num_key_value_heads, num_groups, seq_len, head_dim)
            q = q.reshape(bsz * num_key_value_heads, num_groups * seq_len, head_dim)
            fake_keys = search_hyperplane(q).view(bsz, num_key_value_heads, head_dim)
            batch_indices, head_indices, seq_indices = module.masked_key_indices
            key[batch_indices, head_indices, seq_indices] = fake_keys[batch_indices, head_indices]
        if "cu_seq_lens_k" in kwargs:
            kwargs["cu_seq_lens_k"][-1] = key.shape[-2]
        return func(module, query, key, value, attention_mask, dropout, **kwargs)

    setattr(wrapper, _PATCH_ATTR, True)
    return wrapper


def patch_attention_functions() -> None:
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    for name, func in list(ALL_ATTENTION_FUNCTIONS.items()):
        if getattr(func, _PATCH_ATTR, False):
            continue
        ALL_ATTENTION_FUNCTIONS[name] = _attention_patch(func)
