"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle and the golden fixtures."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

LEVELS = (0, 2, 3, 4, 8, 16)
QBITS = (2, 3, 4, 8)


def eps_of(g):
    return {int(k): float(v) for k, v in zip(g["epsilon_levels"], g["epsilon_values"])}


def alloc_eps(eps, eviction_cost=0.5):
    return [eps[b] * (eviction_cost if b == 0 else 1.0) for b in LEVELS]


def random_bits(rng, B, H, T, probs=(0.12, 0.5, 0.2, 0.08, 0.05, 0.05)):
    return rng.choice(np.array(LEVELS, np.int32), size=(B, H, T), p=probs).astype(np.int32)


def unpack_slot_codes(packed, bits):
    """Little-endian bit stream of 128 codes per row -> codes [n, 128]."""
    bitsarr = np.unpackbits(packed.astype(np.uint8), axis=1, bitorder="little").reshape(packed.shape[0], 128, bits)
    return (bitsarr * (1 << np.arange(bits, dtype=np.uint8))).sum(axis=2).astype(np.uint8)


@pytest.mark.parametrize("bits", QBITS)
def test_encode_pack_bit_exact_on_given_coordinates(pkg, orc, cuda, bits):
    rng = np.random.default_rng(bits)
    cent = orc.codebook_f32(bits)
    y = (rng.standard_normal((1000, 128)) / math.sqrt(128)).astype(np.float32)
    # exact centroids, exact midpoints (ties), values beyond the ends, and a NaN
    mids = ((cent[:-1].astype(np.float64) + cent[1:]) / 2).astype(np.float32)
    y[0, : min(128, cent.size)] = cent[:128]
    y[1, : min(128, mids.size)] = mids[:128]
    y[2, :4] = [-1.0, 1.0, 0.0, np.nan]
    want = orc.encode(y, cent)
    got = pkg.ops.encode_pack(torch.from_numpy(y).to(cuda), bits).cpu().numpy()
    assert np.array_equal(unpack_slot_codes(got, bits), want)


@pytest.mark.parametrize("dtype,B,H,T", [(torch.float16, 1, 2, 320), (torch.bfloat16, 2, 3, 200), (torch.float32, 1, 1, 5),
                                         (torch.float16, 1, 2, 127), (torch.float16, 2, 2, 129)])
def test_quantize_pack_and_dequant_bit_exact(pkg, orc, cuda, dtype, B, H, T):
    rng = np.random.default_rng(T)
    Kt = torch.from_numpy(rng.standard_normal((B, H, T, 128)).astype(np.float32)).to(dtype)
    Vt = torch.from_numpy((3.0 * rng.standard_normal((B, H, T, 128))).astype(np.float32)).to(dtype)
    Kt[..., :4] *= 10
    bits = random_bits(rng, B, H, T)
    pi_k, pi_v = orc.random_rotation(128, 49), orc.random_rotation(128, 2049)
    st = orc.state_prefill(Kt.float().numpy(), Vt.float().numpy(), bits, LEVELS, 49, pi_k, pi_v)
    ch = pkg.ops.quantize_pack(Kt.to(cuda), Vt.to(cuda), torch.from_numpy(bits).to(cuda), torch.from_numpy(pi_k).to(cuda),
                               torch.from_numpy(pi_v).to(cuda), t_offset=0)
    for b in QBITS:
        pos, ik, nk, iv, nv = [t.cpu().numpy() for t in pkg.ops.export_bank(ch, b)]
        bank = st.banks[b]
        assert np.array_equal(pos, bank.positions)
        assert np.array_equal(ik, orc.pack_indices(bank.k_idx, b)), f"{b}-bit key codes differ"
        assert np.array_equal(iv, orc.pack_indices(bank.v_idx, b)), f"{b}-bit value codes differ"
        assert np.array_equal(nk, bank.k_norm) and np.array_equal(nv, bank.v_norm)
    assert np.array_equal(pkg.ops.export_positions(ch, 0).cpu().numpy(), st.masked)
    epos, ek, ev = pkg.ops.export_exact_rows(ch)
    assert np.array_equal(epos.cpu().numpy(), st.exact_pos)
    assert np.array_equal(ek.float().cpu().numpy(), st.exact_k) and np.array_equal(ev.float().cpu().numpy(), st.exact_v)
    # segments start on 16-slot boundaries and padding is inert
    ss, sc = ch.seg_start.cpu().numpy(), ch.seg_count.cpu().numpy()
    assert (ss % 16 == 0).all()
    assert np.array_equal(sc.sum(axis=1), np.array([(bits == l).sum() for l in LEVELS]))
    # dequantised cache, before the cast (fp32 out) and after it (cache dtype out)
    Kh, Vh, keep = orc.materialize(st)
    Ko = torch.zeros(B, H, T, 128, dtype=torch.float32, device=cuda)
    Vo = torch.zeros_like(Ko)
    pkg.ops.dequant_chunk_into(ch, torch.from_numpy(pi_k).to(cuda), torch.from_numpy(pi_v).to(cuda), Ko, Vo, True)
    assert np.array_equal(Ko.cpu().numpy(), Kh) and np.array_equal(Vo.cpu().numpy(), Vh)
    Kc = torch.zeros(B, H, T, 128, dtype=dtype, device=cuda)
    Vc = torch.zeros_like(Kc)
    pkg.ops.dequant_chunk_into(ch, torch.from_numpy(pi_k).to(cuda), torch.from_numpy(pi_v).to(cuda), Kc, Vc, True)
    assert torch.equal(Kc.cpu(), torch.from_numpy(Kh).to(dtype)) and torch.equal(Vc.cpu(), torch.from_numpy(Vh).to(dtype))


def test_quantize_pack_rejects_bad_input(pkg, cuda):
    K = torch.zeros(1, 2, 16, 128, dtype=torch.float16, device=cuda)
    pi = torch.eye(128, device=cuda)
    with pytest.raises(ValueError):
        pkg.ops.quantize_pack(K, K[:, :1], torch.zeros(1, 2, 16, dtype=torch.int32, device=cuda), pi, pi)
    with pytest.raises(ValueError):
        pkg.ops.quantize_pack(K, K, torch.zeros(1, 2, 15, dtype=torch.int32, device=cuda), pi, pi)
    with pytest.raises(ValueError):
        pkg.ops.quantize_pack(K, K, torch.full((1, 2, 16), 5, dtype=torch.int32, device=cuda), pi, pi)
    with pytest.raises(ValueError):
        pkg.ops.quantize_pack(K[..., :64], K[..., :64], torch.zeros(1, 2, 16, dtype=torch.int32, device=cuda), pi, pi)


@pytest.mark.parametrize("dtype,B,H,G,T", [(torch.float16, 1, 2, 4, 320), (torch.bfloat16, 2, 2, 7, 200), (torch.float16, 1, 8, 4, 4096),
                                           (torch.float32, 1, 1, 1, 6), (torch.float16, 2, 4, 8, 777), (torch.float16, 1, 2, 4, 3),
                                           (torch.float16, 1, 2, 12, 300), (torch.float32, 1, 2, 4, 1500), (torch.bfloat16, 1, 1, 8, 5000)])
def test_score_prefill_matches_oracle(pkg, orc, cuda, dtype, B, H, G, T):
    K16, V16, Qw16, _ = orc.synth_inputs(H, T, G, 128, 64, 3, B)
    Kt, Vt = torch.from_numpy(K16).to(dtype), torch.from_numpy(V16).to(dtype)
    mu = Qw16.astype(np.float32).mean(axis=2)
    want = np.stack([orc.score_prefill(Kt[b].float().numpy(), Vt[b].float().numpy(), mu[b], 4, 1e-2) for b in range(B)])
    got = pkg.ops.score_prefill(Kt.to(cuda), Vt.to(cuda), torch.from_numpy(mu).to(cuda), 4, 1e-2).cpu().numpy()
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1e-30)
    assert rel.max() < 1e-4, rel.max()   # tolerance: 1e-4 relative on scores


def test_score_status_word_is_clean(pkg, orc, cuda):
    """The sweeps wait on their bulk copies with a bound and report an expired wait through a status word."""
    g = torch.Generator().manual_seed(5)
    K = torch.randn(2, 2, 3000, 128, generator=g).half().to(cuda)
    V = torch.randn(2, 2, 3000, 128, generator=g).half().to(cuda)
    mu = torch.randn(2, 8, 128, generator=g).to(cuda)
    pkg.ops.score_prefill(K, V, mu, 4, 1e-2, check_status=True)   # raises when the word is set


def test_score_prefill_matches_golden_reference(pkg, cuda, golden):
    g = golden["small_g7_b2"]
    got = pkg.ops.score_prefill(torch.from_numpy(g["K"]).to(cuda), torch.from_numpy(g["V"]).to(cuda),
                                torch.from_numpy(g["mu"]).to(cuda), 4, 1e-2).cpu().numpy()
    assert (np.abs(got - g["scores"]) / g["scores"]).max() < 1e-4


def test_score_with_attn_matches_oracle(pkg, orc, cuda):
    rng = np.random.default_rng(0)
    R, T = 6, 128
    K = rng.standard_normal((R, T, 128)).astype(np.float16)
    V = rng.standard_normal((R, T, 128)).astype(np.float16)
    lg = rng.standard_normal((R, T)).astype(np.float32) * 2
    p = np.exp(lg - lg.max(-1, keepdims=True))
    p = (p / p.sum(-1, keepdims=True)).astype(np.float32)
    want = orc.score_with_attn(K.astype(np.float32), V.astype(np.float32), p, 1e-2)
    got = pkg.ops.score_with_attn(torch.from_numpy(K).to(cuda), torch.from_numpy(V).to(cuda), torch.from_numpy(p).to(cuda), 1e-2)
    assert (np.abs(got.cpu().numpy() - want) / want).max() < 1e-4


def heavy_scores(rng, n, sigma):
    return np.exp(rng.standard_normal(n) * sigma - 2.0).astype(np.float32)


@pytest.mark.parametrize("case", ["small_g4", "small_g7_b2"])
def test_allocate_bits_bit_exact_on_reference_scores(pkg, cuda, golden, case):
    g = golden[case]
    B, H, G, T, d, seed, layer = [int(v) for v in g["meta_shape"]]
    eps = eps_of(g)
    sink = np.zeros((H, T), np.uint8)
    sink[:, :4] = 1
    scores = torch.from_numpy(g["scores"].reshape(B, H * T)).to(cuda)
    for target in g["targets"]:
        tag = f"t{int(round(target * 10)):02d}"
        bits, rep = pkg.ops.allocate_bits(scores, torch.from_numpy(sink.reshape(-1)).to(cuda), LEVELS, alloc_eps(eps), float(target))
        assert np.array_equal(bits.cpu().numpy().reshape(B, H, T), g[f"{tag}_bits"].astype(np.int32))
        for r in pkg.ops.read_reports(rep):
            assert r["done"] and r["evaluations"] == 66 and r["n_active"] == H * (T - 4)


@pytest.mark.parametrize("n,target,sigma", [(4096 * 8, 2.0, 1.0), (4096 * 8, 2.5, 2.5), (12288 * 8, 3.0, 2.5), (8192 * 8, 4.2, 3.0),
                                            (1000, 0.7, 1.0), (1000, 15.0, 3.0), (50000, 8.0, 4.0), (7, 2.0, 1.0)])
def test_allocate_bits_bit_exact_vs_oracle_heavy_tails(pkg, orc, cuda, golden, n, target, sigma):
    """Heavy-tailed scores reach the 8- and 16-bit levels; both gap-closure directions are exercised."""
    eps = eps_of(golden["kats"])
    rng = np.random.default_rng(int(n + 10 * target))
    P = 3
    s = np.stack([heavy_scores(rng, n, sigma) for _ in range(P)])
    s[1, : n // 3] = s[1, n // 3: 2 * (n // 3)]   # duplicated scores -> ties at the cuts
    sink = np.zeros(n, np.uint8)
    sink[:: max(n // 8, 1)] = 1
    info = [orc.AllocInfo() for _ in range(P)]
    want = np.stack([orc.optimal_scores_to_bits(s[p], LEVELS, target, eps, sink.astype(bool), eviction_cost=0.5, info=info[p])
                     for p in range(P)])
    bits, rep = pkg.ops.allocate_bits(torch.from_numpy(s).to(cuda), torch.from_numpy(sink).to(cuda), LEVELS, alloc_eps(eps), target)
    got = bits.cpu().numpy()
    reports = pkg.ops.read_reports(rep)
    for p in range(P):
        assert np.array_equal(got[p], want[p]), f"problem {p}: {(got[p] != want[p]).sum()} of {n} differ"
        if sink.all():
            continue   # the reference returns before searching when every token is pinned
        assert reports[p]["done"]
        assert reports[p]["evaluations"] == info[p].evaluations
        assert reports[p]["moved"] == info[p].moved
        assert reports[p]["ties_lambda"] == info[p].ties_lambda
        assert abs(reports[p]["gap_before"] - info[p].gap_before) < 1e-9


@pytest.mark.parametrize("n,target,nvals", [(30000, 2.0, 40), (30000, 3.0, 12), (70000, 5.5, 25), (5000, 2.5, 3)])
def test_allocate_bits_bit_exact_on_score_ladders(pkg, orc, cuda, golden, n, target, nvals):
    """Scores drawn from a few distinct values: the bisection ends with one value on a breakpoint of the cost lines
    (inside the band that is evaluated with the full formula), every level is a handful of long runs of equal scores,
    and the gap closure cuts inside such a run -- the cases in which the selection from the sorted scores has to walk a
    band and hand the cut among equal scores to the index passes."""
    eps = eps_of(golden["kats"])
    rng = np.random.default_rng(int(n + 100 * target + nvals))
    P = 3
    ladder = (10.0 ** rng.uniform(-6, 1, size=nvals)).astype(np.float32)
    s = np.stack([ladder[rng.integers(0, nvals, size=n)] for _ in range(P)])
    s[2] = np.sort(s[2])[::-1]                    # descending: the index order of equal scores matters for the cut
    sink = np.zeros(n, np.uint8)
    sink[:4] = 1
    info = [orc.AllocInfo() for _ in range(P)]
    want = np.stack([orc.optimal_scores_to_bits(s[p], LEVELS, target, eps, sink.astype(bool), eviction_cost=0.5, info=info[p])
                     for p in range(P)])
    bits, rep = pkg.ops.allocate_bits(torch.from_numpy(np.ascontiguousarray(s)).to(cuda), torch.from_numpy(sink).to(cuda), LEVELS,
                                      alloc_eps(eps), target)
    got = bits.cpu().numpy()
    reports = pkg.ops.read_reports(rep)
    for p in range(P):
        assert np.array_equal(got[p], want[p]), f"problem {p}: {(got[p] != want[p]).sum()} of {n} differ"
        assert reports[p]["done"] and reports[p]["moved"] == info[p].moved
        assert reports[p]["ties_lambda"] == info[p].ties_lambda and reports[p]["ties_cut"] == info[p].ties_cut


def test_allocate_bits_edge_cases(pkg, orc, cuda, golden):
    eps = eps_of(golden["kats"])
    # nan / inf / negative scores, all-sink mask, constant scores (every cut is a tie), single level
    s = np.array([[0.5, np.nan, np.inf, -1.0, 0.25, 0.75, -np.inf, 0.1] * 64], np.float32)
    want = orc.optimal_scores_to_bits(s[0], LEVELS, 2.0, eps, None, eviction_cost=0.5)
    got, _ = pkg.ops.allocate_bits(torch.from_numpy(s).to(cuda), None, LEVELS, alloc_eps(eps), 2.0)
    assert np.array_equal(got.cpu().numpy()[0], want)
    ones = np.ones((1, 4096), np.float32)
    for target in (2.0, 2.5, 5.0):
        info = orc.AllocInfo()
        want = orc.optimal_scores_to_bits(ones[0], LEVELS, target, eps, None, eviction_cost=0.5, info=info)
        got, rep = pkg.ops.allocate_bits(torch.from_numpy(ones).to(cuda), None, LEVELS, alloc_eps(eps), target)
        assert np.array_equal(got.cpu().numpy()[0], want)
        assert pkg.ops.read_reports(rep)[0]["ties_cut"] == info.ties_cut
        assert target == 2.0 or info.ties_cut >= 1
    allsink = np.ones(4096, np.uint8)
    got, _ = pkg.ops.allocate_bits(torch.from_numpy(ones).to(cuda), torch.from_numpy(allsink).to(cuda), LEVELS, alloc_eps(eps), 2.0)
    assert (got.cpu().numpy() == 16).all()
    got, _ = pkg.ops.allocate_bits(torch.from_numpy(ones).to(cuda), None, (4,), [eps[4]], 2.0)
    assert (got.cpu().numpy() == 4).all()


def test_allocate_bits_sharded_equals_single(pkg, cuda, golden):
    """Two shards of one problem, the exchange summed by hand, reproduce the single-device answer."""
    eps = eps_of(golden["kats"])
    rng = np.random.default_rng(5)
    n = 20000
    s = heavy_scores(rng, n, 2.0)[None]
    full, _ = pkg.ops.allocate_bits(torch.from_numpy(s).to(cuda), None, LEVELS, alloc_eps(eps), 3.0)
    L = pkg._lib.lib()
    ptr, st = pkg._lib.ptr, pkg._lib.stream_ptr(cuda)
    halves = [torch.from_numpy(s[:, : n // 2].copy()).to(cuda), torch.from_numpy(s[:, n // 2:].copy()).to(cuda)]
    lv, ev, K = pkg.ops._level_arrays(LEVELS, alloc_eps(eps))
    xlen = L.odmkv_alloc_exchange_len()
    wss, exs, outs = [], [], []
    for r, h in enumerate(halves):
        ws = torch.empty(L.odmkv_alloc_workspace_bytes(1, h.shape[1]), dtype=torch.uint8, device=cuda)
        ex = torch.zeros(1, xlen, dtype=torch.int64, device=cuda)
        pkg._lib.check(L.odmkv_alloc_begin(ptr(h), None, 1, h.shape[1], r * (n // 2), lv, ev, K, 3.0, 16, ptr(ws), ws.numel(), ptr(ex), st), "begin")
        wss.append(ws)
        exs.append(ex)
    for _ in range(L.odmkv_alloc_num_rounds(K)):
        for ws, ex in zip(wss, exs):
            pkg._lib.check(L.odmkv_alloc_eval(ptr(ws), ptr(ex), st), "eval")
        total = exs[0] + exs[1]
        for ws in wss:
            pkg._lib.check(L.odmkv_alloc_update(ptr(ws), ptr(total), st), "update")
    for ws, h in zip(wss, halves):
        out = torch.empty(1, h.shape[1], dtype=torch.int32, device=cuda)
        pkg._lib.check(L.odmkv_alloc_finish(ptr(ws), ptr(out), None, st), "finish")
        outs.append(out)
    assert torch.equal(torch.cat(outs, dim=1), full)


def assert_attn_close(got, want, tag=()):
    """Attention tolerance: 1e-3 "max relative error".  Outputs cross zero, so the error of an element is taken
    relative to the largest magnitude of its output row (one query head), and also relative to the largest
    magnitude of the whole tensor."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want)
    assert err.max() / np.abs(want).max() < 1e-3, (tag, "global", err.max() / np.abs(want).max())
    row = err.max(axis=-1) / np.maximum(np.abs(want).max(axis=-1), 1e-30)
    assert row.max() < 1e-3, (tag, "per row", row.max())


def build_case(pkg, orc, cuda, B, H, G, T, dtype, seed, target=None, probs=None):
    K16, V16, _, qd16 = orc.synth_inputs(H, T, G, 128, 8, seed, B)
    Kt, Vt = torch.from_numpy(K16).to(dtype), torch.from_numpy(V16).to(dtype)
    rng = np.random.default_rng(seed)
    bits = random_bits(rng, B, H, T, probs) if probs else random_bits(rng, B, H, T)
    bits[..., :4] = 16
    bits[..., -min(T, 20):] = 16
    pi_k, pi_v = orc.random_rotation(128, 42), orc.random_rotation(128, 2042)
    st = orc.state_prefill(Kt.float().numpy(), Vt.float().numpy(), bits, LEVELS, 42, pi_k, pi_v)
    pk, pv = torch.from_numpy(pi_k).to(cuda), torch.from_numpy(pi_v).to(cuda)
    ch = pkg.ops.quantize_pack(Kt.to(cuda), Vt.to(cuda), torch.from_numpy(bits).to(cuda), pk, pv)
    return st, ch, pk, pv, torch.from_numpy(qd16).to(dtype)


@pytest.mark.parametrize("plain", [True, False])
@pytest.mark.parametrize("dtype,B,H,G,T", [(torch.float16, 1, 2, 4, 320), (torch.bfloat16, 2, 2, 7, 200), (torch.float16, 1, 8, 4, 4096),
                                           (torch.float16, 2, 3, 8, 1000), (torch.float32, 1, 1, 1, 5), (torch.float16, 1, 2, 2, 129)])
def test_decode_attn_matches_dense_attention_over_dequantised_cache(pkg, orc, cuda, plain, dtype, B, H, G, T):
    st, ch, pk, pv, qd = build_case(pkg, orc, cuda, B, H, G, T, dtype, seed=11)
    Kh, Vh, keep = orc.materialize(st)
    want = orc.decode_attention(qd.float().numpy(), Kh, Vh, keep)
    for ns in (0, 1, 3):
        got = pkg.ops.decode_attn(qd.to(cuda), [ch], pk, pv, n_splits=ns, out_dtype=torch.float32, plain=plain).cpu().numpy()
        assert_attn_close(got, want, (ns,))


@pytest.mark.parametrize("plain", [True, False])
def test_decode_attn_chunks_and_tail(pkg, orc, cuda, plain):
    """Two chunks (prefill + a later flush) and a dense tail of recent tokens."""
    B, H, G, T = 2, 2, 4, 300
    K16, V16, _, qd16 = orc.synth_inputs(H, T, G, 128, 8, 21, B)
    Kt, Vt = torch.from_numpy(K16), torch.from_numpy(V16)
    rng = np.random.default_rng(2)
    bits = random_bits(rng, B, H, T)
    T1, T2 = 200, 260   # chunk 0: [0, 200), chunk 1: [200, 260), tail: [260, 300)
    pi_k, pi_v = orc.random_rotation(128, 42), orc.random_rotation(128, 2042)
    pk, pv = torch.from_numpy(pi_k).to(cuda), torch.from_numpy(pi_v).to(cuda)
    bits_full = bits.copy()
    bits_full[..., T2:] = 16
    st = orc.state_prefill(Kt.float().numpy(), Vt.float().numpy(), bits_full, LEVELS, 42, pi_k, pi_v)
    Kh, Vh, keep = orc.materialize(st)
    want = orc.decode_attention(qd16.astype(np.float32), Kh, Vh, keep)
    bt = torch.from_numpy(bits).to(cuda)
    c0 = pkg.ops.quantize_pack(Kt[:, :, :T1].to(cuda), Vt[:, :, :T1].to(cuda), bt[:, :, :T1], pk, pv, t_offset=0)
    c1 = pkg.ops.quantize_pack(Kt[:, :, T1:T2].to(cuda), Vt[:, :, T1:T2].to(cuda), bt[:, :, T1:T2], pk, pv, t_offset=T1)
    cap = 64
    tk = torch.zeros(B, H, cap, 128, dtype=torch.float16, device=cuda)
    tv = torch.zeros_like(tk)
    tk[:, :, : T - T2] = Kt[:, :, T2:].to(cuda)
    tv[:, :, : T - T2] = Vt[:, :, T2:].to(cuda)
    got = pkg.ops.decode_attn(torch.from_numpy(qd16).to(cuda), [c0, c1], pk, pv, tail_k=tk, tail_v=tv, tail_len=T - T2,
                              out_dtype=torch.float32, plain=plain, return_lse=True)
    out, lse = got[0].cpu().numpy(), got[1].cpu().numpy()
    assert_attn_close(out, want)
    # log-sum-exp against the dense logits
    Gq = qd16.shape[1] // H
    for b in range(B):
        for hq in range(H * Gq):
            lg = (Kh[b, hq // Gq] @ qd16[b, hq].astype(np.float32)) / math.sqrt(128)
            lg = lg[keep[b, hq // Gq]]
            ref = lg.max() + math.log(np.exp(lg - lg.max()).sum())
            assert abs(lse[b, hq] - ref) < 2e-3
    # positions of the second chunk carry its offset
    pos = pkg.ops.export_positions(c1, 5).cpu().numpy()
    assert pos.size == 0 or pos[:, 2].min() >= T1


@pytest.mark.parametrize("target", [2.0, 3.0])
def test_decode_attn_against_golden_reference_run(pkg, orc, cuda, golden, target):
    """End to end on the fixture inputs: compress with this library, attend, compare with the reference's
    dense attention over its own dequantised cache."""
    g = golden["small_g4"]
    tag = f"t{int(round(target * 10)):02d}"
    B, H, G, T, d, seed, layer = [int(v) for v in g["meta_shape"]]
    bits = g[f"{tag}_bits"].astype(np.int32).copy()
    bits[..., -128:] = 16
    pk = torch.from_numpy(orc.random_rotation(128, 42 + 7 * layer)).to(cuda)
    pv = torch.from_numpy(orc.random_rotation(128, 42 + 7 * layer + 2000)).to(cuda)
    ch = pkg.ops.quantize_pack(torch.from_numpy(g["K"]).to(cuda), torch.from_numpy(g["V"]).to(cuda), torch.from_numpy(bits).to(cuda), pk, pv)
    for b in (2, 3, 4):
        if f"{tag}_L{b}_pos" not in g.files:
            continue
        pos, ik, nk, iv, nv = [t.cpu().numpy() for t in pkg.ops.export_bank(ch, b)]
        assert np.array_equal(pos.astype(np.int32), g[f"{tag}_L{b}_pos"])
        allowed = {(int(r[0]), int(r[1])): int(r[2]) for r in g[f"{tag}_code_flips"]}
        assert int((orc.unpack_indices(ik, b, 128) != orc.unpack_indices(g[f"{tag}_L{b}_k_packed"], b, 128)).sum()) == allowed[(b, 0)]
        assert int((orc.unpack_indices(iv, b, 128) != orc.unpack_indices(g[f"{tag}_L{b}_v_packed"], b, 128)).sum()) == allowed[(b, 1)]
    out = pkg.ops.decode_attn(torch.from_numpy(g["qd"]).to(cuda), [ch], pk, pv, out_dtype=torch.float32).cpu().numpy()
    assert_attn_close(out, g[f"{tag}_attn"])


def test_runs_are_deterministic(pkg, orc, cuda):
    st, ch, pk, pv, qd = build_case(pkg, orc, cuda, 1, 2, 4, 700, torch.float16, seed=4)
    a = pkg.ops.decode_attn(qd.to(cuda), [ch], pk, pv, out_dtype=torch.float32)
    b = pkg.ops.decode_attn(qd.to(cuda), [ch], pk, pv, out_dtype=torch.float32)
    assert torch.equal(a, b)


def test_chunk_compaction_keeps_decode_banks_and_truncation(pkg, orc, cuda):
    """Fourteen flushes: the state merges its flushed chunks when its list is full (a decode call takes at most twelve
    chunk descriptors).  Decode attention, the dequantised cache and truncation must not notice."""
    B, H, G, T0, n_flush, m = 2, 2, 4, 200, 14, 24
    T = T0 + n_flush * m
    K16, V16, _, qd16 = orc.synth_inputs(H, T, G, 128, 8, 31, B)
    rng = np.random.default_rng(5)
    bits = random_bits(rng, B, H, T)
    bits[..., :4] = 16
    Kt, Vt, bt = torch.from_numpy(K16).to(cuda), torch.from_numpy(V16).to(cuda), torch.from_numpy(bits).to(cuda)
    State = pkg.tq_adaptive_backend.TurboQuantAdaptiveKVCacheState
    state = State(head_dim=128, bit_levels=LEVELS, device=cuda, dtype=torch.float16, key_quantizer="mse", value_quantizer="mse", seed=42)
    state.prefill(Kt[:, :, :T0].contiguous(), Vt[:, :, :T0].contiguous(), bt[:, :, :T0].contiguous())
    max_chunks = 0
    for f in range(n_flush):
        a, b = T0 + f * m, T0 + (f + 1) * m
        state.append_all_exact(Kt[:, :, a:b], Vt[:, :, a:b])
        state.flush_buffer(a, bt[:, :, a:b])
        max_chunks = max(max_chunks, len(state.chunks))
    assert max_chunks <= pkg._lib.MAX_CHUNKS and len(state.chunks) < 1 + n_flush and state.seq_len == T and state.tail_len == 0
    pi_k, pi_v = state.pi_k.cpu().numpy(), state.pi_v.cpu().numpy()
    q = torch.from_numpy(qd16).to(cuda)

    def check(T_now):
        st = orc.state_prefill(K16[:, :, :T_now].astype(np.float32), V16[:, :, :T_now].astype(np.float32), bits[:, :, :T_now], LEVELS, 42, pi_k, pi_v)
        Kh, Vh, keep = orc.materialize(st)
        want = orc.decode_attention(qd16.astype(np.float32), Kh, Vh, keep)
        assert_attn_close(state.decode_attention(q, out_dtype=torch.float32).cpu().numpy(), want, (T_now,))
        Kf, Vf = state.materialize_fp32()
        assert np.array_equal(Kf.cpu().numpy()[keep], Kh[keep]) and np.array_equal(Vf.cpu().numpy()[keep], Vh[keep])
        assert np.array_equal(state.keep_mask().cpu().numpy(), keep)
        banks = state._quantized_banks
        for level in (2, 3, 4, 8):
            assert banks[level].size == int((bits[:, :, :T_now] == level).sum())

    check(T)
    state.truncate(T0 + 5 * m + 3)       # inside the merged chunk
    check(T0 + 5 * m + 3)
    state.truncate(T0 - 7)               # inside the prefill chunk
    check(T0 - 7)
