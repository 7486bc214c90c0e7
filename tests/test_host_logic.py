"""Host-side logic that needs no GPU: sharding plans, rank-tier allocation, press configuration, the
attention wrapper's fallback path, and the two collectives of the sharded path on gloo ranks."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_and_plans(pkg):
    d = pkg.dist
    for n, w in ((80, 8), (7, 3), (4, 2), (5, 8)):
        spans = [d.shard_range(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    # 70B shape on 8 GPUs: layers first -> no compress collective, every rank keeps all 8 KV heads
    p = d.plan_units(80, 8, 8, 5)
    assert p["layers"] == (50, 60) and p["heads"] == (0, 8) and p["head_group"] == [5]
    # Qwen shape, 2 GPUs, head split: 4 KV heads -> 2 + 2 and the two ranks share every layer's Lagrangian
    p = d.plan_units(28, 4, 2, 1, prefer="heads")
    assert p["layers"] == (0, 28) and p["heads"] == (2, 4) and p["head_group"] == [0, 1]
    with pytest.raises(ValueError):
        d.shard_range(4, 2, 2)


def test_ratio_and_uniform_allocation_match_reference_kats(pkg, golden):
    g = golden["kats"]
    sc = torch.from_numpy(g["ratio_scores"])
    bits = pkg.allocator.ratio_scores_to_bits(sc, (2, 3, 4), (0.7, 0.25, 0.05))
    assert np.array_equal(bits.numpy(), g["ratio_bits"])
    # banker's rounding of tier sizes, last tier takes the remainder
    b = pkg.allocator.ratio_scores_to_bits(torch.arange(5.0), (2, 4), (0.5, 0.5), per_head=False)
    assert b.tolist() == [2, 2, 4, 4, 4]
    u = pkg.allocator.scores_to_bits(torch.tensor([0.0, 0.3, 0.6, 1.0]), (2, 4, 8))
    assert u.tolist() == [2, 2, 4, 8]
    assert pkg.allocator.effective_bits(2, 0) == 2.0 and pkg.allocator.effective_bits(2, 4, 128, 4) == 2 + 4 * 2 / 128


def test_make_press_applies_paper_settings(pkg):
    press = pkg.press_factory.make_press({"mode": "backend_per_token", "bits": [0, 2, 3, 4, 8, 16], "target_avg_bits": 2.0,
                                          "eviction_cost": 0.5, "n_outlier_channels": 0, "outlier_min_bits": 2}, seed=42)
    assert press.bit_levels == (0, 2, 3, 4, 8, 16) and press.target_avg_bits == 2.0 and press.eviction_cost == 0.5
    assert press.sink_tokens == 4 and press.buffer_size == 128 and press.layerwise and press.decode_quant
    assert press._decode_bit_levels == (2, 3, 4, 8, 16)
    assert press.scorer.normalize_grain == "global" and press.scorer.epsilon == 1e-2 and press.scorer.n_sink == 4
    assert not press.scorer.use_covariance
    assert pkg.press_factory.make_press({"mode": "baseline"}, 0) is None
    with pytest.raises(ValueError):
        pkg.press_factory.make_press({"mode": "nope"}, 0)
    with pytest.raises(NotImplementedError):
        pkg.adaptive_backend_press.TurboQuantPerTokenBackendPress(scorer=press.scorer, key_quantizer="prod", value_quantizer="mse")
    with pytest.raises(ValueError):
        pkg.adaptive_backend_press.TurboQuantPerTokenBackendPress(scorer=None, key_quantizer="mse", value_quantizer="mse")


def test_kernels_refuse_cpu_tensors(pkg):
    K = torch.zeros(1, 1, 8, 128)
    with pytest.raises(pkg.OdmkvError):
        pkg.ops.score_prefill(K, K, torch.zeros(1, 1, 128))
    with pytest.raises(pkg.OdmkvError):
        pkg.ops.quantize_pack(K, K, torch.zeros(1, 1, 8, dtype=torch.int32), torch.eye(128), torch.eye(128))


def test_fake_key_masks_evicted_positions(pkg):
    """The wrapper's fallback (no packed state): evicted keys are overwritten so they get zero weight."""
    torch.manual_seed(0)
    ap = pkg.attention_patch
    B, Hq, H, T, d = 1, 4, 2, 12, 16
    q = torch.randn(B, Hq, 1, d)
    k = torch.randn(B, H, T, d)
    v = torch.randn(B, H, T, d)

    class M:
        pass

    m = M()
    m.masked_key_indices = (torch.tensor([0, 0]), torch.tensor([0, 1]), torch.tensor([3, 7]))

    def plain(module, query, key, value, mask, dropout, **kw):
        kk = key.repeat_interleave(Hq // H, dim=1)
        vv = value.repeat_interleave(Hq // H, dim=1)
        w = torch.softmax(query @ kk.transpose(-1, -2) / d ** 0.5, dim=-1)
        return (w @ vv).transpose(1, 2), w

    out, w = ap._attention_patch(plain)(m, q, k.clone(), v, None, 0.0)
    assert float(w[0, :2, 0, 3].abs().max()) < 1e-30 and float(w[0, 2:, 0, 7].abs().max()) < 1e-30
    keep = torch.ones(H, T, dtype=torch.bool)
    keep[0, 3] = keep[1, 7] = False
    for hq in range(Hq):
        h = hq // (Hq // H)
        lg = (k[0, h] @ q[0, hq, 0]) / d ** 0.5
        lg[~keep[h]] = float("-inf")
        ref = torch.softmax(lg, 0) @ v[0, h]
        assert torch.allclose(out[0, 0, hq], ref, atol=1e-5)
    # prefill (q_len == k_len) clears the mask
    ap._attention_patch(plain)(m, torch.randn(B, Hq, T, d), k, v, None, 0.0)
    assert m.masked_key_indices is None


def _gloo_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import importlib
    import torch.distributed as dist
    pkg = importlib.import_module("odm-kv_b200")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # output gather: rank r owns query heads [2r, 2r+2)
        local = torch.full((3, 2, 128), float(rank)) + torch.arange(2).view(1, 2, 1)
        full = pkg.dist.gather_head_outputs(local)
        ok_gather = full.shape == (3, 2 * world, 128) and all(
            torch.equal(full[:, 2 * r:2 * r + 2], torch.full((3, 2, 128), float(r)) + torch.arange(2).view(1, 2, 1)) for r in range(world))
        # count exchange of the sharded Lagrangian: a stand-in for the kernels records what it is given
        calls = {}

        def fake_sharded(scores, mask, levels, eps, target, idx_base, all_reduce, sink_bits=16):
            t = torch.tensor([[int(scores.numel()), idx_base]], dtype=torch.int64)
            all_reduce(t)
            calls["sum"] = t.clone()
            return torch.full(scores.shape, int(t[0, 0]), dtype=torch.int32), torch.zeros(1, dtype=torch.uint8)

        pkg.ops.allocate_bits_sharded = fake_sharded
        lo, hi = pkg.dist.shard_range(4, world, rank)
        sc = torch.rand(2, hi - lo, 16)
        bits, _ = pkg.dist.allocate_bits_kv_sharded(sc, None, (0, 2), [0.5, 0.1], 1.0, head_lo=lo, T=16)
        ok_alloc = bits.shape == (2, hi - lo, 16) and int(calls["sum"][0, 0]) == 2 * 4 * 16 and \
            int(calls["sum"][0, 1]) == sum(pkg.dist.shard_range(4, world, r)[0] * 16 for r in range(world))
        ret[rank] = bool(ok_gather and ok_alloc)
    finally:
        dist.destroy_process_group()


def test_collectives_on_two_gloo_ranks():
    import torch.multiprocessing as mp
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_gloo_worker, args=(world, port, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world)), dict(ret)


def test_packed_chunk_deepcopy_rebuilds_c_view():
    """A deep copy of a packed chunk (the runner copies caches between questions) must not share or pickle
    the cached ctypes view, and its view must point at the copy's own tensors."""
    import copy
    import importlib

    import torch

    ops = importlib.import_module("odm-kv_b200").ops
    z = lambda *s, dt=torch.uint8: torch.zeros(*s, dtype=dt)
    ch = ops.PackedChunk(B=1, H=1, T=16, t_offset=0, dtype=torch.float16, device=torch.device("cpu"),
                         seg_start=z(6, 1, dt=torch.int32), seg_count=z(6, 1, dt=torch.int32), totals=[0, 16, 0, 0, 0, 0],
                         k_codes=[z(512), z(0), z(0), z(0)], v_codes=[z(512), z(0), z(0), z(0)],
                         k_norm=[z(16, dt=torch.float32)] + [z(0, dt=torch.float32)] * 3,
                         v_norm=[z(16, dt=torch.float32)] + [z(0, dt=torch.float32)] * 3,
                         pos=[z(16, dt=torch.int32)] + [z(0, dt=torch.int32)] * 3,
                         exact_k=z(0, 128, dt=torch.float16), exact_v=z(0, 128, dt=torch.float16),
                         exact_pos=z(0, dt=torch.int32), evicted_pos=z(0, dt=torch.int32))
    first = ch.c_struct()
    assert ch.c_struct() is first                       # cached
    dup = copy.deepcopy(ch)
    assert dup._c_struct is None
    view = dup.c_struct()
    assert view.k_codes[0] == dup.k_codes[0].data_ptr() != ch.k_codes[0].data_ptr()
    assert view.cap[1] == 16 and view.T == 16


def test_mask_predicates_of_the_attention_wrapper(pkg):
    """The packed decode kernels take no mask: the wrapper may use them only when the mask hides no key from a single
    query, and the per-query packed route of a multi-token pass only when nothing but the causal part is masked."""
    ap = pkg.attention_patch
    B, T, q = 2, 9, 3
    assert ap._mask_is_open(None) and ap._causal_or_open(None, q)
    full = torch.ones(B, 1, 1, T, dtype=torch.bool)
    assert ap._mask_is_open(full) and ap._mask_is_open(torch.zeros(B, 1, 1, T))
    padded = full.clone()
    padded[1, ..., :4] = False                       # left padding of sample 1
    assert not ap._mask_is_open(padded)
    additive = torch.zeros(B, 1, 1, T)
    additive[1, ..., :4] = torch.finfo(torch.float32).min
    assert not ap._mask_is_open(additive)
    causal = torch.ones(B, 1, q, T, dtype=torch.bool)
    causal[..., -q:] = torch.tril(torch.ones(q, q, dtype=torch.bool))
    assert ap._causal_or_open(causal, q) and not ap._mask_is_open(causal)
    causal_padded = causal.clone()
    causal_padded[1, ..., :4] = False
    assert not ap._causal_or_open(causal_padded, q)
