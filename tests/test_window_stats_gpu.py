"""Column statistics of causal softmax attention (tcgen05 kernels) against the oracle and the reference fixture."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-3   # relative to the largest entry of each statistic (fp16 / bf16 inputs, fp32 accumulation, ex2.approx)


def close(got: torch.Tensor, want: np.ndarray, what: str):
    want = torch.from_numpy(np.ascontiguousarray(want)).to(got.device)
    err = (got - want).abs().max() / want.abs().max()
    assert err < TOL, (what, float(err))


def test_reference_fixture(pkg, golden, cuda):
    g = golden["window_g4"]
    Q = torch.from_numpy(g["Q"]).to(cuda).unsqueeze(0)
    K = torch.from_numpy(g["K"]).to(cuda).unsqueeze(0)
    s, m, q = pkg.ops.window_attn_stats(Q, K)
    close(s[0], g["sum_attn"], "sum")
    close(m[0], g["max_attn"], "max")
    close(q[0], g["sum_sq_attn"], "sum_sq")
    # the mirror of the reference's helper takes the G-expanded transposed keys and returns [H_kv, T_kv] tensors
    G = int(g["G"])
    H = K.shape[1]
    expanded_t = K.repeat_interleave(G, dim=1).transpose(-1, -2).contiguous()
    s2, m2, q2 = pkg.scorer._chunked_attention_qk(Q, expanded_t, K.shape[2], H, G, math.sqrt(128.0), 64, cuda, torch.float32)
    assert torch.equal(s2, s[0]) and torch.equal(m2, m[0]) and torch.equal(q2, q[0])


@pytest.mark.parametrize("B,H,G,Tq,Tkv,off,dtype", [
    (1, 2, 4, 128, 128, 0, torch.float16),        # exactly one tile
    (2, 2, 4, 300, 300, 0, torch.bfloat16),       # ragged tiles, batch
    (1, 1, 8, 130, 450, 320, torch.float16),      # window of the last 130 queries, N = 256 columns
    (1, 2, 7, 96, 700, 604, torch.float16),       # G = 7 (Qwen2.5-7B): N = 224
    (1, 1, 12, 40, 200, 160, torch.bfloat16),     # G > 8: blocks of 16 queries
    (1, 1, 1, 257, 257, 0, torch.float16),        # G = 1
    (1, 2, 4, 64, 1500, 1500 - 64, torch.float16),
    (2, 2, 4, 128, 2048, 2048 - 128, torch.bfloat16),   # the press's window shape, tensor copies
    (1, 1, 8, 256, 1024, 768, torch.float16),           # N = 256 columns, tensor copies
    (1, 2, 4, 384, 384, 0, torch.float16),              # full causal, three tiles per side
    (1, 1, 2, 100, 777, 677, torch.float16),            # ragged everything, two heads per KV head
    (1, 1, 4, 64, 1000, 200, torch.bfloat16),           # keys that no query sees (zeros)
    (2, 1, 3, 128, 5000, 4872, torch.float16),          # three heads per KV head
])
def test_against_oracle(pkg, orc, cuda, B, H, G, Tq, Tkv, off, dtype):
    g = torch.Generator().manual_seed(Tq * 7 + Tkv)
    Q = (torch.randn(B, H * G, Tq, 128, generator=g) * 1.3).to(dtype)
    K = torch.randn(B, H, Tkv, 128, generator=g)
    K[:, :, :4] *= 2.5
    K = K.to(dtype)
    L = pkg._lib.lib()
    s, m, q = pkg.ops.window_attn_stats(Q.to(cuda), K.to(cuda), q_offset=off)
    assert L.odmkv_window_stats_last_path() == 1            # tiles arrived by tensor copies
    L.odmkv_window_stats_force_thread_copies(1)             # the other staging path must give the same numbers
    try:
        s2, m2, q2 = pkg.ops.window_attn_stats(Q.to(cuda), K.to(cuda), q_offset=off)
        assert L.odmkv_window_stats_last_path() == 0
    finally:
        L.odmkv_window_stats_force_thread_copies(0)
    assert torch.equal(s, s2) and torch.equal(m, m2) and torch.equal(q, q2)
    for b in range(B):
        ws, wm, wq = orc.chunked_attention_qk(Q[b].float().numpy(), K[b].float().numpy(), math.sqrt(128.0), q_offset=off)
        close(s[b], ws, "sum")
        close(m[b], wm, "max")
        close(q[b], wq, "sum_sq")
    # size-independent property: the column sums of a KV head add up to its number of queries
    assert torch.allclose(s.sum(-1), torch.full_like(s.sum(-1), float(Tq)), rtol=1e-4)


def test_arguments(pkg, cuda):
    Q = torch.zeros(1, 4, 16, 128, dtype=torch.float16, device=cuda)
    K = torch.zeros(1, 2, 16, 128, dtype=torch.float16, device=cuda)
    with pytest.raises(NotImplementedError):
        pkg.ops.window_attn_stats(Q.float(), K.float())
    with pytest.raises(ValueError):
        pkg.ops.window_attn_stats(Q[:, :3], K)
    with pytest.raises(ValueError):
        pkg.ops.window_attn_stats(Q, K, q_offset=-1)
    s, m, q = pkg.ops.window_attn_stats(Q, K)     # all logits equal: uniform weights over the visible keys
    want = sum(1.0 / (r + 1) for r in range(16))
    assert abs(float(s[0, 0, 0]) - want) < 1e-4 and abs(float(m[0, 0, 0]) - 1.0) < 1e-6


def test_windowed_risk_scores(pkg, orc, cuda):
    """RiskScorer.score_windowed = column sums / visibility counts -> score_with_attn, against the oracle's pieces."""
    H, G, T, W = 2, 4, 600, 64
    g = torch.Generator().manual_seed(11)
    K = torch.randn(H, T, 128, generator=g).half()
    V = torch.randn(H, T, 128, generator=g).half()
    Qw = (torch.randn(H * G, W, 128, generator=g) * 1.2).half()
    scorer = pkg.scorer.RiskScorer(n_sink=4, epsilon=1e-2)
    got = scorer.score_windowed(K.to(cuda), V.to(cuda), Qw.to(cuda))
    s, _, _ = orc.chunked_attention_qk(Qw.float().numpy(), K.float().numpy(), math.sqrt(128.0), q_offset=T - W)
    seen = W - np.clip(np.arange(T) - (T - W), 0, None)
    want = orc.score_with_attn(K.float().numpy(), V.float().numpy(), (s / seen).astype(np.float32), 1e-2)
    err = np.abs(got.cpu().numpy() - want).max() / np.abs(want).max()
    assert err < TOL, err
