"""The workspace-free decode entry point (for hosts that cannot allocate device memory: a serving loop
with a frozen pool, a plug-in that only receives raw pointers) must return exactly what the regular
entry point returns -- on two calls in a row, because both calls share the library's built-in scratch
array and the second one finds the first one's leftovers in it."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

LEVELS = (0, 2, 3, 4, 8, 16)


def call_noalloc(pkg, q, chunks, pk, pv, n_splits, tail_k=None, tail_v=None, tail_len=0, out=None):
    L, lib_ = pkg._lib.lib(), pkg._lib
    B, Hq, _ = q.shape
    H = chunks[0].H
    if out is None:
        out = torch.empty(B, Hq, 128, dtype=torch.float32, device=q.device)
    arr = (lib_.Chunk * len(chunks))(*[c.c_struct() for c in chunks])
    rc = L.odmkv_decode_attn_noalloc(lib_.ptr(q), lib_.dtype_code(q.dtype), arr, len(chunks), lib_.dtype_code(chunks[0].dtype),
                                     lib_.ptr(tail_k), lib_.ptr(tail_v), tail_len, 0 if tail_k is None else tail_k.shape[2],
                                     lib_.ptr(pk), lib_.ptr(pv), lib_.ptr(pkg.ops.codebook_table(q.device)), B, H, Hq // H,
                                     1.0 / 128 ** 0.5, lib_.ptr(out), lib_.DTYPE_F32, None, n_splits, pkg.ops.lut_scales(),
                                     lib_.stream_ptr(q.device))
    return rc, out


def test_noalloc_decode_matches_regular_entry_point_twice(pkg, orc, cuda):
    rng = np.random.default_rng(9)
    pk = torch.from_numpy(orc.random_rotation(128, 42)).to(cuda)
    pv = torch.from_numpy(orc.random_rotation(128, 2042)).to(cuda)
    for B, H, G, T, ns in ((1, 2, 4, 700, 3), (2, 2, 8, 333, 2)):   # second call: other shape, stale scratch contents
        K16, V16, _, qd16 = orc.synth_inputs(H, T, G, 128, 8, 5 + B, B)
        bits = rng.choice(np.array(LEVELS, np.int32), size=(B, H, T), p=(0.1, 0.5, 0.2, 0.1, 0.05, 0.05)).astype(np.int32)
        chunk = pkg.ops.quantize_pack(torch.from_numpy(K16).to(cuda), torch.from_numpy(V16).to(cuda), torch.from_numpy(bits).to(cuda), pk, pv)
        q = torch.from_numpy(qd16).to(cuda)
        tk = torch.randn(B, H, 16, 128, device=cuda).half()
        tv = torch.randn(B, H, 16, 128, device=cuda).half()
        want = pkg.ops.decode_attn(q, [chunk], pk, pv, tail_k=tk, tail_v=tv, tail_len=5, n_splits=ns, out_dtype=torch.float32)
        got = torch.empty(B, H * G, 128, dtype=torch.float32, device=cuda)
        for rep in range(2):
            if rep == 1:
                # the second call (the helper stream, the events and the scratch address exist by now) must leave the
                # device's memory as it found it: neither torch's allocator nor the driver hands anything out
                got.zero_()
                torch.cuda.synchronize()
                alloc0, free0 = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
            rc, _ = call_noalloc(pkg, q, [chunk], pk, pv, ns, tk, tv, 5, out=got)
            assert rc == 0
            if rep == 1:
                torch.cuda.synchronize()
                assert torch.cuda.memory_allocated() == alloc0
                assert torch.cuda.mem_get_info()[0] == free0
            err = (got - want).abs().max() / want.abs().max()
            assert err < 1e-3, err   # same tolerance as the other decode tests (the kernels are the same, so it is 0 in practice)
        if B == 1:
            # and against the CPU oracle: dense attention over the dequantised cache plus the five tail tokens
            st = orc.state_prefill(K16.astype(np.float32), V16.astype(np.float32), bits, LEVELS, 42, orc.random_rotation(128, 42),
                                   orc.random_rotation(128, 2042))
            Kh, Vh, keep = orc.materialize(st)
            Kh = np.concatenate([Kh, tk[:, :, :5].float().cpu().numpy()], axis=2)
            Vh = np.concatenate([Vh, tv[:, :, :5].float().cpu().numpy()], axis=2)
            keep = np.concatenate([keep, np.ones((B, H, 5), bool)], axis=2)
            ref = orc.decode_attention(qd16.astype(np.float32), Kh, Vh, keep)
            assert np.abs(got.cpu().numpy() - ref).max() / np.abs(ref).max() < 1e-3
    # a size whose partials exceed the built-in scratch is refused, nothing runs
    assert pkg._lib.lib().odmkv_decode_attn_noalloc_scratch_bytes() == 6 << 20
    rc, _ = call_noalloc(pkg, torch.zeros(64, 8 * 8, 128, device=cuda, dtype=torch.float16),
                         [pkg.ops.quantize_pack(torch.zeros(64, 8, 16, 128, device=cuda, dtype=torch.float16),
                                                torch.zeros(64, 8, 16, 128, device=cuda, dtype=torch.float16),
                                                torch.full((64, 8, 16), 2, dtype=torch.int32, device=cuda), pk, pv)], pk, pv, 64)
    assert rc == -5
