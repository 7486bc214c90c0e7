"""Pin the CPU oracle to fixtures produced by running the reference on CPU (tests/golden/make_golden.py)."""
import hashlib

import numpy as np
import pytest

LEVELS = (0, 2, 3, 4, 8, 16)


def sha(a):
    return hashlib.sha1(np.ascontiguousarray(a).tobytes()).hexdigest()


def eps_of(g):
    return {int(k): float(v) for k, v in zip(g["epsilon_levels"], g["epsilon_values"])}


def test_kats(orc, golden):
    g = golden["kats"]
    for b in (2, 3, 4, 8):
        assert np.array_equal(orc.codebook_f32(b), g[f"codebook_b{b}"])
    for s in (42, 49, 2042):
        assert np.array_equal(orc.random_rotation(128, s), g[f"pi_seed{s}"])
    assert orc.pack_indices(np.array([[0, 1, 2, 3, 0, 1, 2, 3]]), 2).tolist() == g["pack2"].tolist() == [[228, 228]]
    assert orc.pack_indices(np.arange(8)[None], 3).tolist() == g["pack3"].tolist() == [[16, 50, 84, 118]]
    assert orc.pack_indices(np.arange(8, 16)[None], 4).tolist() == g["pack4"].tolist() == [[152, 186, 220, 254]]
    for bits, vals in ((2, [0, 1, 2, 3] * 32), (3, list(range(8)) * 16), (4, list(range(16)) * 8)):
        idx = np.array([vals], np.uint8)
        assert np.array_equal(orc.unpack_indices(orc.pack_indices(idx, bits), bits, 128), idx)
    rb = np.stack([orc.ratio_scores_to_bits(r, (2, 3, 4), (0.7, 0.25, 0.05)) for r in g["ratio_scores"]])
    assert np.array_equal(rb, g["ratio_bits"])


def test_epsilon_calibration_close_to_reference(orc, golden):
    ref = eps_of(golden["kats"])
    mine = orc.calibrate_epsilon(128, LEVELS, seed=42)
    assert mine[0] == 1.0 and mine[16] == 0.0
    for b in (2, 3, 4, 8):
        assert abs(mine[b] - ref[b]) / ref[b] < 1e-5


@pytest.mark.parametrize("case", ["small_g4", "small_g7_b2"])
def test_scores_bits_banks_attention(orc, golden, case):
    g = golden[case]
    B, H, G, T, d, seed, layer = [int(v) for v in g["meta_shape"]]
    K = g["K"].astype(np.float32)
    V = g["V"].astype(np.float32)
    regen = orc.synth_inputs(H, T, G, d, 64, seed, B)
    inputs_reproduce = np.array_equal(regen[0], g["K"]) and np.array_equal(regen[3], g["qd"])
    assert inputs_reproduce, "seeded generator no longer reproduces the fixture inputs"
    eps = eps_of(g)
    sink = np.zeros((H, T), bool)
    sink[:, :4] = True
    for b in range(B):
        s = orc.score_prefill(K[b], V[b], g["mu"][b], 4, 1e-2)
        assert np.max(np.abs(s - g["scores"][b]) / np.abs(g["scores"][b])) < 1e-5
    for target in g["targets"]:
        tag = f"t{int(round(target * 10)):02d}"
        bits = np.stack([orc.optimal_scores_to_bits(g["scores"][b], LEVELS, float(target), eps, sink, eviction_cost=0.5)
                         for b in range(B)])
        assert np.array_equal(bits, g[f"{tag}_bits"].astype(np.int32))
        bits_w = bits.copy()
        bits_w[..., -128:] = 16
        pi_k = orc.random_rotation(d, 42 + 7 * layer)
        pi_v = orc.random_rotation(d, 42 + 7 * layer + 2000)
        st = orc.state_prefill(K, V, bits_w, LEVELS, 42 + 7 * layer, pi_k, pi_v)
        assert st.exact_pos.shape[0] == int(g[f"{tag}_exact_count"])
        assert st.masked.shape[0] == int(g[f"{tag}_masked_count"])
        flips_allowed = {(int(r[0]), int(r[1])): int(r[2]) for r in g[f"{tag}_code_flips"]}
        for level in (2, 3, 4, 8):
            if f"{tag}_L{level}_pos" not in g.files:
                continue
            bank = st.banks[level]
            assert np.array_equal(bank.positions.astype(np.int32), g[f"{tag}_L{level}_pos"])
            for side, idx, nrm in (("k", bank.k_idx, bank.k_norm), ("v", bank.v_idx, bank.v_norm)):
                ref_idx = orc.unpack_indices(g[f"{tag}_L{level}_{side}_packed"], level, d)
                nflip = int((ref_idx != idx).sum())
                assert nflip == flips_allowed[(level, 0 if side == "k" else 1)]
                assert np.max(np.abs(nrm - g[f"{tag}_L{level}_{side}_norms"]) / nrm) < 2e-6
        Kh, Vh, keep = orc.materialize(st)
        assert np.max(np.abs(Kh[:, :, ::16] - g[f"{tag}_Khat_sample"])) < 1e-5 * np.abs(Kh).max()
        att = orc.decode_attention(g["qd"].astype(np.float32), Kh, Vh, keep)
        assert np.max(np.abs(att - g[f"{tag}_attn"])) / np.abs(g[f"{tag}_attn"]).max() < 1e-5


def test_config0_digests(orc, golden):
    """Full config-0 shapes: inputs regenerated from the seed, outputs compared through digests."""
    g = golden["config0"]
    B, H, G, T, d, seed, layer = [int(v) for v in g["meta_shape"]]
    K16, V16, Qw16, qd16 = orc.synth_inputs(H, T, G, d, 64, seed, B)
    if (sha(K16) + sha(V16) + sha(Qw16) + sha(qd16)).encode() != bytes(g["input_sha"]):
        pytest.skip("torch's CPU generator yields different inputs here than where the fixture was made")
    K, V = K16.astype(np.float32), V16.astype(np.float32)
    mu = Qw16.astype(np.float32).mean(axis=2)
    s = orc.score_prefill(K[0], V[0], mu[0], 4, 1e-2)
    stats = g["scores_stats"]
    assert abs(s.min() - stats[0]) < 1e-6 * stats[0] and abs(s.max() - stats[1]) < 2e-6 * stats[1]
    assert abs(s.astype(np.float64).sum() - stats[2]) < 1e-6 * stats[2]
    assert np.max(np.abs(s[None][:, :, ::97] - g["scores_sample"]) / g["scores_sample"]) < 1e-5
    # bits are compared on the oracle's own scores: they agree with the reference's to ~1e-6, which can
    # move a handful of tokens, so the histogram is checked to a small tolerance and the exact digest
    # only when fed the reference's allocation inputs (done for the small cases above)
    eps = eps_of(g)
    sink = np.zeros((H, T), bool)
    sink[:, :4] = True
    for target in g["targets"]:
        tag = f"t{int(round(target * 10)):02d}"
        bits = orc.optimal_scores_to_bits(s, LEVELS, float(target), eps, sink, eviction_cost=0.5)
        hist = np.array([(bits == l).sum() for l in LEVELS])
        assert np.abs(hist - g[f"{tag}_bits_hist"]).max() <= 8
        nonsink = bits[:, 4:]
        assert abs(nonsink.sum() - target * nonsink.size) <= 0.5 + 1e-9


def test_window_attention_stats_match_reference(orc, golden):
    """The oracle's restatement of _chunked_attention_qk against the reference's own output (fp32 run)."""
    g = golden["window_g4"]
    s, m, q = orc.chunked_attention_qk(g["Q"].astype(np.float32), g["K"].astype(np.float32), np.sqrt(128.0))
    for got, want in ((s, g["sum_attn"]), (m, g["max_attn"]), (q, g["sum_sq_attn"])):
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    # every query's weights sum to one, so the column sums add up to the number of queries per KV head
    assert np.allclose(s.sum(axis=1), g["Q"].shape[1], rtol=1e-5)
