"""Generate golden fixtures by running the reference implementation on CPU.

Run from the repository root in a container that has the reference checked out:

    python tests/golden/make_golden.py --reference /path/to/ODM-KV

The reference imports ``kvquant.tq_triton.mse_nearest_centroid``, a module its tree does not
ship.  This script registers an in-memory stand-in that follows the comment at
``kvquant/tq_backend.py:191-196`` (searchsorted, clamp, two distances, where; the lower index
wins an exact tie).  Everything else that runs is the reference's own code, on fp32 copies of
fp16 inputs (its CPU torch path).

Outputs (``tests/golden/*.npz``) hold the inputs of the small cases in full, the reference's
scores, bit allocations, banks, dequantised cache and dense decode attention, and for the larger
"config 0" case the scores, bit allocations, digests and samples (its inputs are regenerated from the seed); two
"press" cases record where the reference press puts every token of a tiny random-init Llama after prefill, an
optional question pass and decode steps through the decode buffer.  The script
also runs the oracle on the same inputs and stores how many values differ, so the fixtures
document where the oracle and the reference legitimately part (summation order of the rotation).
"""
from __future__ import annotations

import argparse
import hashlib
import math
import os
import sys
import types

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

LEVELS = (0, 2, 3, 4, 8, 16)
N_SINK = 4
WINDOW_PROTECT = 128
EVICTION_COST = 0.5
SEED = 42


def install_reference(path: str):
    sys.path.insert(0, path)
    import kvquant  # noqa: F401  (imports fine; the missing module is only needed at quantize time)

    shim = types.ModuleType("kvquant.tq_triton")

    def mse_nearest_centroid(y, centroids):
        c = centroids.contiguous()
        idx = torch.searchsorted(c, y.contiguous())
        k = c.numel()
        lo = (idx - 1).clamp(min=0)
        hi = idx.clamp(max=k - 1)
        return torch.where((y - c[lo]).abs() <= (y - c[hi]).abs(), lo, hi)

    shim.mse_nearest_centroid = mse_nearest_centroid
    sys.modules["kvquant.tq_triton"] = shim


class StubAttn(torch.nn.Module):
    """Attention-module stand-in: q_proj is the identity on a [T, Hq*d] layout, no rotary."""

    def __init__(self, num_heads, head_dim):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.q_proj = torch.nn.Identity()
        self.rotary_emb = None


def sha(a: np.ndarray) -> str:
    return hashlib.sha1(np.ascontiguousarray(a).tobytes()).hexdigest()


def run_case(name, B, H, G, T, seed, targets, store_inputs, outdir, layer_idx=0, store_scores_bits=False):
    from kvquant.scorer import RiskScorer
    from kvquant.allocator import optimal_scores_to_bits, calibrate_epsilon
    from kvquant.tq_adaptive_backend import TurboQuantAdaptiveKVCacheState
    from oracle import odmkv_oracle as orc

    d = 128
    K16, V16, Qw16, qd16 = orc.synth_inputs(H, T, G, d, 64, seed, B)
    K = torch.from_numpy(K16).float()
    V = torch.from_numpy(V16).float()
    Qw = torch.from_numpy(Qw16).float()
    qd = torch.from_numpy(qd16).float()
    Hq = H * G
    scorer = RiskScorer(n_future_positions=512, n_sink=N_SINK, use_vnorm=True, epsilon=1e-2)
    scorer.normalize_grain = "global"
    module = StubAttn(Hq, d)
    eps = calibrate_epsilon(d, LEVELS, seed=SEED, value_quantizer="mse")

    out = {
        "meta_shape": np.array([B, H, G, T, d, seed, layer_idx], np.int64),
        "input_sha": np.frombuffer((sha(K16) + sha(V16) + sha(Qw16) + sha(qd16)).encode(), np.uint8),
        "epsilon_levels": np.array(sorted(eps), np.int64),
        "epsilon_values": np.array([eps[k] for k in sorted(eps)], np.float64),
        "targets": np.array(targets, np.float64),
    }
    if store_inputs:
        out.update(K=K16, V=V16, Qw=Qw16, qd=qd16)

    # ---- scores (per sample, as the press loops: adaptive_backend_press.py:355-367)
    scores = []
    mus = []
    for b in range(B):
        hidden = torch.zeros(1, N_SINK + Qw.shape[2], Hq * d)
        hidden[0, N_SINK:] = Qw[b].permute(1, 0, 2).reshape(Qw.shape[2], Hq * d)
        s = scorer.score_prefill(K[b], V[b], layer_idx, module=module, hidden_states=hidden)
        scores.append(s.float().numpy())
        mus.append(Qw[b].mean(dim=1).numpy())
    scores = np.stack(scores)          # [B, H, T]
    mu = np.stack(mus).astype(np.float32)  # [B, Hq, d]
    out["mu"] = mu
    o_scores = np.stack([orc.score_prefill(K[b].numpy(), V[b].numpy(), mu[b], N_SINK, 1e-2) for b in range(B)])
    rel = np.abs(o_scores - scores) / np.maximum(np.abs(scores), 1e-30)
    out["scores_oracle_max_rel"] = np.array(rel.max())
    print(f"[{name}] scores: min {scores.min():.7g} max {scores.max():.7g} sum {scores.astype(np.float64).sum():.8g} "
          f"oracle max rel {rel.max():.3g}")
    if store_inputs or store_scores_bits:
        out["scores"] = scores
    if not store_inputs:
        out["scores_sample"] = scores[:, :, ::97].copy()
        out["scores_stats"] = np.array([scores.min(), scores.max(), scores.astype(np.float64).sum()], np.float64)

    sink_mask = torch.zeros(H, T, dtype=torch.bool)
    sink_mask[:, :N_SINK] = True
    pi_k = orc.random_rotation(d, SEED + 7 * layer_idx)
    pi_v = orc.random_rotation(d, SEED + 7 * layer_idx + 2000)
    out["pi_k_sha"] = np.frombuffer(sha(pi_k).encode(), np.uint8)

    for target in targets:
        tag = f"t{int(round(target * 10)):02d}"
        bits = []
        o_mismatch = 0
        for b in range(B):
            bt = optimal_scores_to_bits(torch.from_numpy(scores[b]), LEVELS, target, eps, sink_mask,
                                        eviction_cost=EVICTION_COST, n_outlier=0, head_dim=d, outlier_min_bits=2)
            bits.append(bt.numpy().astype(np.int32))
            ob = orc.optimal_scores_to_bits(scores[b], LEVELS, target, eps, sink_mask.numpy(),
                                            eviction_cost=EVICTION_COST)
            o_mismatch += int((ob != bits[-1]).sum())
        bits = np.stack(bits)  # [B, H, T]
        hist = {int(l): int((bits == l).sum()) for l in LEVELS}
        print(f"[{name}] target {target}: hist {hist} sha {sha(bits)[:16]} oracle mismatches {o_mismatch}")
        out[f"{tag}_bits_oracle_mismatch"] = np.array(o_mismatch)
        out[f"{tag}_bits_sha"] = np.frombuffer(sha(bits).encode(), np.uint8)
        out[f"{tag}_bits_hist"] = np.array([hist[l] for l in LEVELS], np.int64)
        if store_inputs or store_scores_bits:
            out[f"{tag}_bits"] = bits.astype(np.int8)

        # ---- window override + state.prefill (adaptive_backend_press.py:306-316)
        bits_w = bits.copy()
        bits_w[..., -min(WINDOW_PROTECT, T):] = 16
        state = TurboQuantAdaptiveKVCacheState(
            head_dim=d, bit_levels=LEVELS, value_group_size=32, device=torch.device("cpu"), dtype=torch.float32,
            key_quantizer="mse", value_quantizer="mse", seed=SEED + 7 * layer_idx)
        state.prefill(K, V, torch.from_numpy(bits_w))
        ost = orc.state_prefill(K.numpy(), V.numpy(), bits_w, LEVELS, SEED + 7 * layer_idx, pi_k, pi_v)
        flips = {}
        for level, bank in state._quantized_banks.items():
            n = bank.size
            if n == 0:
                continue
            assert np.array_equal(bank.positions.numpy(), ost.banks[level].positions)
            kq, vq = bank.key_quantized, bank.value_quantized
            for side, q, oidx, onorm in (("k", kq, ost.banks[level].k_idx, ost.banks[level].k_norm),
                                          ("v", vq, ost.banks[level].v_idx, ost.banks[level].v_norm)):
                packed = q.indices.numpy()
                ref_idx = orc.unpack_indices(packed, level, d)
                nflip = int((ref_idx != oidx).sum())
                maxstep = int(np.abs(ref_idx.astype(np.int32) - oidx.astype(np.int32)).max()) if n else 0
                nrel = float(np.abs(q.norms.numpy() - onorm).max() / np.abs(onorm).max())
                flips[(level, side)] = (nflip, n * d, maxstep, nrel)
                out[f"{tag}_L{level}_{side}_packed_sha"] = np.frombuffer(sha(packed).encode(), np.uint8)
                if store_inputs:
                    out[f"{tag}_L{level}_{side}_packed"] = packed
                    out[f"{tag}_L{level}_{side}_norms"] = q.norms.numpy()
            if store_inputs:
                out[f"{tag}_L{level}_pos"] = bank.positions.numpy().astype(np.int32)
            out[f"{tag}_L{level}_count"] = np.array(n)
        print(f"[{name}] target {target}: code flips oracle-vs-reference (flips, coords, max step, norm rel): {flips}")
        out[f"{tag}_code_flips"] = np.array([[l, 0 if s == 'k' else 1, *flips[(l, s)][:3]] for (l, s) in flips], np.int64)
        out[f"{tag}_exact_count"] = np.array(state._exact_bank.size)
        out[f"{tag}_masked_count"] = np.array(state._masked_positions.shape[0])

        # ---- dequantised cache before the dtype cast, dense decode attention over it
        Kh = torch.zeros(B, H, T, d)
        Vh = torch.zeros(B, H, T, d)
        keep = torch.zeros(B, H, T, dtype=torch.bool)
        eb = state._exact_bank
        if eb.size:
            p = eb.positions
            Kh[p[:, 0], p[:, 1], p[:, 2]] = eb.keys
            Vh[p[:, 0], p[:, 1], p[:, 2]] = eb.values
            keep[p[:, 0], p[:, 1], p[:, 2]] = True
        for level, bank in state._quantized_banks.items():
            if bank.size == 0:
                continue
            p = bank.positions
            Kh[p[:, 0], p[:, 1], p[:, 2]] = bank.key_quantizer.dequantize(bank.key_quantized)
            Vh[p[:, 0], p[:, 1], p[:, 2]] = bank.value_mse_quantizer.dequantize(bank.value_quantized)
            keep[p[:, 0], p[:, 1], p[:, 2]] = True
        mp = state._masked_positions
        assert not keep[mp[:, 0], mp[:, 1], mp[:, 2]].any()
        # dense fp32 attention, evicted keys excluded (attention_patch.py:30-55 gives them exp(logit) = 0)
        att = torch.zeros(B, Hq, d)
        for b in range(B):
            for h in range(H):
                qq = qd[b, h * G:(h + 1) * G]
                logits = qq @ Kh[b, h].T / math.sqrt(d)
                logits = logits.masked_fill(~keep[b, h][None, :], float("-inf"))
                att[b, h * G:(h + 1) * G] = torch.softmax(logits, dim=-1) @ Vh[b, h]
        oK, oV, okeep = orc.materialize(ost)
        oatt = orc.decode_attention(qd.numpy(), oK, oV, okeep)
        arel = float(np.abs(oatt - att.numpy()).max() / np.abs(att.numpy()).max())
        drel = float(np.abs(oK - Kh.numpy()).max() / np.abs(Kh.numpy()).max())
        print(f"[{name}] target {target}: decode attn oracle-vs-reference max rel {arel:.3g}; dequant K max rel {drel:.3g}")
        out[f"{tag}_attn"] = att.numpy()
        out[f"{tag}_attn_oracle_max_rel"] = np.array(arel)
        if store_inputs:
            out[f"{tag}_Khat_sample"] = Kh.numpy()[:, :, ::16].astype(np.float32)
            out[f"{tag}_Vhat_sample"] = Vh.numpy()[:, :, ::16].astype(np.float32)

    path = os.path.join(outdir, f"{name}.npz")
    np.savez_compressed(path, **out)
    print(f"[{name}] wrote {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


def kats(outdir):
    """Known-answer values of the small pure functions."""
    from kvquant.tq_backend import _pack_indices, random_rotation, _load_or_compute_codebook
    from kvquant.allocator import calibrate_epsilon, ratio_scores_to_bits
    out = {}
    dev = torch.device("cpu")
    for b in (2, 3, 4, 8):
        out[f"codebook_b{b}"] = _load_or_compute_codebook(b, 128, dev, torch.float32).numpy()
    for s in (42, 49, 2042):
        out[f"pi_seed{s}"] = random_rotation(128, dev, torch.float32, seed=s).numpy()
    out["pack2"] = _pack_indices(torch.tensor([[0, 1, 2, 3, 0, 1, 2, 3]]), 2).numpy()
    out["pack3"] = _pack_indices(torch.tensor([[0, 1, 2, 3, 4, 5, 6, 7]]), 3).numpy()
    out["pack4"] = _pack_indices(torch.tensor([[8, 9, 10, 11, 12, 13, 14, 15]]), 4).numpy()
    eps = calibrate_epsilon(128, LEVELS, seed=SEED, value_quantizer="mse")
    out["epsilon_levels"] = np.array(sorted(eps), np.int64)
    out["epsilon_values"] = np.array([eps[k] for k in sorted(eps)], np.float64)
    g = torch.Generator().manual_seed(5)
    sc = torch.rand(3, 128, generator=g)
    out["ratio_scores"] = sc.numpy()
    out["ratio_bits"] = ratio_scores_to_bits(sc, (2, 3, 4), (0.7, 0.25, 0.05)).numpy()
    np.savez_compressed(os.path.join(outdir, "kats.npz"), **out)
    print("wrote kats.npz")


def tiny_llama(dtype=torch.float32, layers=2):
    """The random-init model the press tests use (same seed and initialisation on either side)."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=layers, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=128, max_position_embeddings=4096, rope_theta=10000.0,
                      attn_implementation="sdpa")
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg)
    for p in model.parameters():
        torch.nn.init.normal_(p, std=0.05)
    return model.to(dtype).eval()


def press_inputs(B, T, n_question, n_decode, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 512, (B, T), generator=g)
    qids = torch.randint(0, 512, (B, n_question), generator=g) if n_question else None
    toks = torch.randint(0, 512, (B, n_decode), generator=g)   # teacher-forced decode tokens
    return ids, qids, toks


def state_bits_map(state, B, H, T_total):
    """[B, H, T_total] int8: 0 evicted, 2/3/4/8 quantised level, 16 exact, -1 not stored."""
    m = np.full((B, H, T_total), -1, np.int8)
    mp = state._masked_positions
    if mp.numel():
        mp = mp.cpu().numpy()
        m[mp[:, 0], mp[:, 1], mp[:, 2]] = 0
    for level, bank in state._quantized_banks.items():
        if bank.size:
            p = bank.positions.cpu().numpy()
            m[p[:, 0], p[:, 1], p[:, 2]] = level
    eb = state._exact_bank
    if eb.size:
        p = eb.positions.cpu().numpy()
        m[p[:, 0], p[:, 1], p[:, 2]] = 16
    return m


@torch.no_grad()
def press_case(name, B, T, n_question, n_decode, buffer_size, outdir, target=2.6):
    """The reference press on the tiny model (CPU, fp32): prefill, an optional multi-token question pass, then
    single-token decode steps through the decode buffer; records where every token ended up."""
    from transformers import DynamicCache
    from benchmark.core.press_factory import make_press
    model = tiny_llama()
    press = make_press({"mode": "backend_per_token", "bits": list(LEVELS), "target_avg_bits": target, "eviction_cost": EVICTION_COST}, seed=SEED)
    press.buffer_size = buffer_size
    ids, qids, toks = press_inputs(B, T, n_question, n_decode, seed=11)
    cache = DynamicCache()
    out = {"meta": np.array([B, T, n_question, n_decode, buffer_size, 11], np.int64), "target": np.array(target)}
    with press(model):
        model.model(input_ids=ids, past_key_values=cache)
        for li in range(len(model.model.layers)):
            out[f"prefill_bits_L{li}"] = state_bits_map(press._states[li], B, 2, T)
        if qids is not None:
            model(input_ids=qids, past_key_values=cache)
        logits = None
        for s in range(n_decode):
            logits = model(input_ids=toks[:, s:s + 1], past_key_values=cache).logits
        T_total = T + n_question + n_decode
        for li in range(len(model.model.layers)):
            st = press._states[li]
            assert st.seq_len == T_total
            out[f"final_bits_L{li}"] = state_bits_map(st, B, 2, T_total)
            out[f"buffer_L{li}"] = np.array([press._buffer_start_seqs[li], press._buffer_counts[li]], np.int64)
        out["last_logits"] = logits[:, -1].float().numpy()
    hist = {int(v): int((out["final_bits_L0"] == v).sum()) for v in np.unique(out["final_bits_L0"])}
    print(f"[{name}] final layer-0 placement {hist}, buffer {out['buffer_L0']}")
    path = os.path.join(outdir, f"{name}.npz")
    np.savez_compressed(path, **out)
    print(f"[{name}] wrote {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


def window_case(name, H, G, Tq, Tkv, seed, outdir):
    """The reference's _chunked_attention_qk (kvquant/attention_utils.py:160-211) on fp16-representable inputs in
    fp32, with the G-expanded transposed keys it expects; chunk size 64 so that the chunk loop runs more than once."""
    from kvquant.attention_utils import _chunked_attention_qk, _repeat_kv
    g = torch.Generator().manual_seed(seed)
    Q = (torch.randn(1, H * G, Tq, 128, generator=g) * 1.5).half().float()
    K = torch.randn(1, H, Tkv, 128, generator=g).half().float()
    K[:, :, :4] *= 3.0        # a few dominant early keys, as attention sinks are
    K = K.half().float()
    expanded_t = _repeat_kv(K, G).transpose(-1, -2).contiguous()
    s, m, q = _chunked_attention_qk(Q, expanded_t, Tkv, H, G, math.sqrt(128.0), 64, torch.device("cpu"), torch.float32)
    np.savez_compressed(os.path.join(outdir, name + ".npz"), Q=Q[0].numpy().astype(np.float16), K=K[0].numpy().astype(np.float16),
                        sum_attn=s.numpy(), max_attn=m.numpy(), sum_sq_attn=q.numpy(), G=np.int32(G))
    print(name, "sum", float(s.sum()), "max", float(m.max()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory that holds kvquant/)")
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden"))
    ap.add_argument("--only-press", action="store_true", help="regenerate the two press fixtures only")
    ap.add_argument("--only-window", action="store_true", help="regenerate the windowed-attention fixture only")
    args = ap.parse_args()
    torch.set_num_threads(os.cpu_count() or 1)
    install_reference(args.reference)
    if args.only_window:
        window_case("window_g4", H=2, G=4, Tq=200, Tkv=200, seed=5, outdir=args.out)
        return
    if args.only_press:
        press_case("press_b1_question", B=1, T=160, n_question=6, n_decode=40, buffer_size=16, outdir=args.out)
        press_case("press_b2", B=2, T=150, n_question=0, n_decode=36, buffer_size=16, outdir=args.out)
        return
    kats(args.out)
    run_case("small_g4", B=1, H=2, G=4, T=320, seed=1, targets=(2.0, 3.0), store_inputs=True, outdir=args.out)
    run_case("small_g7_b2", B=2, H=2, G=7, T=200, seed=2, targets=(2.0,), store_inputs=True, outdir=args.out, layer_idx=1)
    run_case("config0", B=1, H=8, G=4, T=4096, seed=0, targets=(2.0, 3.0), store_inputs=False, outdir=args.out, store_scores_bits=True)
    press_case("press_b1_question", B=1, T=160, n_question=6, n_decode=40, buffer_size=16, outdir=args.out)
    press_case("press_b2", B=2, T=150, n_question=0, n_decode=36, buffer_size=16, outdir=args.out)
    window_case("window_g4", H=2, G=4, Tq=200, Tkv=200, seed=5, outdir=args.out)


if __name__ == "__main__":
    main()
