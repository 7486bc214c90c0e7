"""Model-level run of the press: a random-init model of one of the benchmark shapes, prefill under the press,
then teacher-forced decode steps, with the packed cache as the only cache (``packed_cache=True``).

    python odm-kv_b200/model_bench.py --config config1            # Llama-3.1-8B shape, prefill 32768, 256 decode steps
    python odm-kv_b200/model_bench.py --config config1 --layers 4 --prefill 4096 --decode 16

It mirrors what the reference's runner does around the press (benchmark/core/pipeline.py:117-145, 164-209: prefill
through the backbone inside ``with press(model)``, then one forward pass per generated token), with synthetic token
ids and random-init bf16 weights N(0, 0.02) because neither datasets nor checkpoints are available.  Prints one JSON
line: compress time per layer (kernel times by stage), decode time per step and per layer, tokens per second, and
the resident cache bytes (packed against the dense bf16 cache the reference keeps).
"""
from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = {
    # name: (family, layers, hidden, intermediate, q heads, kv heads, vocab, prefill, batch, decode steps)
    "config1": ("llama", 32, 4096, 14336, 32, 8, 128256, 32768, 1, 256),
    "config3": ("qwen2", 28, 3584, 18944, 28, 4, 152064, 131072, 16, 128),
    "config4": ("llama", 80, 8192, 28672, 64, 8, 128256, 131072, 8, 128),
    "tiny": ("llama", 2, 512, 1024, 8, 2, 512, 1024, 2, 16),
}
LEVELS = (0, 2, 3, 4, 8, 16)


def build_model(torch, family, layers, hidden, inter, hq, hkv, vocab, dev):
    if family == "qwen2":
        from transformers import Qwen2Config, Qwen2ForCausalLM
        cfg = Qwen2Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                          num_attention_heads=hq, num_key_value_heads=hkv, max_position_embeddings=1 << 18,
                          rope_theta=1000000.0, attn_implementation="sdpa")
        cls = Qwen2ForCausalLM
    else:
        from transformers import LlamaConfig, LlamaForCausalLM
        cfg = LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                          num_attention_heads=hq, num_key_value_heads=hkv, head_dim=128, max_position_embeddings=1 << 18,
                          rope_theta=500000.0, attn_implementation="sdpa")
        cls = LlamaForCausalLM
    torch.manual_seed(0)
    with torch.device(dev):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            model = cls(cfg)
        finally:
            torch.set_default_dtype(prev)
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    for p in model.parameters():
        if p.dim() >= 2:
            p.data.normal_(0.0, 0.02, generator=g)
    return model.eval()


def stage_times(L):
    out = {}
    for name in ("score", "allocate", "quantize", "decode_main", "decode_rotate", "decode_side", "decode_merge"):
        tot, n = ctypes.c_double(), ctypes.c_longlong()
        L.odmkv_timing_read(name.encode(), ctypes.byref(tot), ctypes.byref(n))
        out[name] = (tot.value, n.value)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="config1", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0, help="override the depth (first layers only)")
    ap.add_argument("--prefill", type=int, default=0)
    ap.add_argument("--decode", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--target-bits", type=float, default=2.0)
    ap.add_argument("--dense-cache", action="store_true", help="keep the dense HF cache in sync (the reference's behaviour)")
    ap.add_argument("--no-press", action="store_true", help="plain model with its dense cache, for comparison")
    ap.add_argument("--graph", action="store_true", help="replay the decode step from a CUDA graph (packed cache only)")
    args = ap.parse_args()
    import torch
    from transformers import DynamicCache
    if not torch.cuda.is_available():
        raise SystemExit("model_bench.py needs a CUDA device (there is no CPU path)")
    pkg = importlib.import_module("odm-kv_b200")
    L = pkg._lib.lib()
    family, layers, hidden, inter, hq, hkv, vocab, prefill, batch, decode = SHAPES[args.config]
    layers = args.layers or layers
    prefill = args.prefill or prefill
    decode = args.decode or decode
    batch = args.batch or batch
    dev = torch.device("cuda", 0)
    model = build_model(torch, family, layers, hidden, inter, hq, hkv, vocab, dev)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, vocab, (batch, prefill), generator=g).to(dev)
    toks = torch.randint(0, vocab, (batch, decode), generator=g).to(dev)
    exp = {"mode": "backend_per_token", "bits": list(LEVELS), "target_avg_bits": args.target_bits, "eviction_cost": 0.5,
           "packed_cache": not args.dense_cache}
    press = None if args.no_press else pkg.press_factory.make_press(exp, seed=42)
    cache = DynamicCache()

    def sync():
        torch.cuda.synchronize()
        return time.perf_counter()

    import contextlib
    # one-time costs (library handles, kernel selection, the press's epsilon calibration) stay outside the timed run
    with torch.no_grad(), (press(model) if press is not None else contextlib.nullcontext()):
        wcache = DynamicCache()
        model.model(input_ids=ids[:, : min(prefill, 512)], past_key_values=wcache)
        # a buffer of two tokens makes the warm-up flush once: the kernels a flush uses (sort, scatter, ...) are loaded
        # by the driver on first use, which costs over a hundred milliseconds once per process
        saved = None if press is None else press.buffer_size
        if press is not None:
            press.buffer_size = 2
        for s in range(3):
            model(input_ids=toks[:, s:s + 1], past_key_values=wcache)
        if press is not None:
            press.buffer_size = saved
        del wcache
    torch.cuda.synchronize()
    ctx = press(model) if press is not None else contextlib.nullcontext()
    with torch.no_grad(), ctx:
        if press is not None:
            press._ensure_epsilon(dev)          # calibration (once per process) outside the timed prefill
        L.odmkv_timing_enable(1)
        t0 = sync()
        model.model(input_ids=ids, past_key_values=cache)
        t1 = sync()
        prefill_stages = stage_times(L)
        torch.cuda.empty_cache()
        mem_after_prefill = torch.cuda.memory_allocated()
        # a few untimed steps, then the timed decode loop (teacher-forced tokens)
        warm = min(3, decode)
        dec = None
        if args.graph:
            if press is None or args.dense_cache:
                raise SystemExit("--graph needs the press with the packed cache")
            dec = pkg.packed_cache.GraphedDecoder(model, press, cache)
            L.odmkv_timing_enable(0)            # event pairs around kernels do not belong in a captured step

        def one_step(s):
            tok = toks[:, s:s + 1]
            return dec.step(tok) if dec is not None else model(input_ids=tok, past_key_values=cache).logits

        for s in range(warm):
            one_step(s)
        stage_times(L)
        kinds = {"replay": [0.0, 0], "capture+replay": [0.0, 0], "eager": [0.0, 0]}
        t2 = sync()
        for s in range(warm, decode):
            if dec is None:
                logits = one_step(s)
                continue
            # per-kind times of the graphed run (one synchronisation per step, negligible against a step)
            before = (dec.captures, dec.replays)
            ta = time.perf_counter()
            logits = one_step(s)
            tb = sync()
            kind = "eager" if dec.replays == before[1] else ("capture+replay" if dec.captures != before[0] else "replay")
            kinds[kind][0] += tb - ta
            kinds[kind][1] += 1
        t3 = sync()
        decode_stages = stage_times(L)
        L.odmkv_timing_enable(0)
        n_timed = max(decode - warm, 1)
        packed_bytes = sum(st.packed_bytes() for st in press._states.values()) if press is not None else None
        chunks = max((len(st.chunks) for st in press._states.values()), default=0) if press is not None else None
    dense_bytes = 2 * layers * batch * hkv * (prefill + decode) * 128 * 2
    line = {
        "config": args.config, "family": family, "layers": layers, "hidden": hidden, "q_heads": hq, "kv_heads": hkv, "batch": batch,
        "prefill_tokens": prefill, "decode_steps": decode, "target_bits": args.target_bits,
        "mode": "no press (dense DynamicCache)" if press is None else ("press, dense cache in sync" if args.dense_cache else
                                                                      "press, packed cache only" + (", decode step replayed from a CUDA graph" if args.graph else "")),
        "graph": None if dec is None else {"captures": dec.captures, "replays": dec.replays, "eager_steps": dec.eager_steps,
                                           "ms_per_step_by_kind": {k: (v[0] * 1e3 / v[1] if v[1] else None) for k, v in kinds.items()},
                                           "steps_by_kind": {k: v[1] for k, v in kinds.items()}},
        "prefill_s": t1 - t0,
        "compress_kernel_ms_per_layer": None if press is None else {k: prefill_stages[k][0] / layers for k in ("score", "allocate", "quantize")},
        "decode_ms_per_step": (t3 - t2) * 1e3 / n_timed,
        "decode_tokens_per_s": batch * n_timed / (t3 - t2),
        "decode_attention_us_per_layer_step": None if press is None else {
            k: decode_stages[k][0] * 1e3 / max(decode_stages[k][1], 1) for k in ("decode_rotate", "decode_main", "decode_side", "decode_merge")},
        "cache_bytes": {"packed": packed_bytes, "dense_bf16": dense_bytes,
                        "ratio": None if not packed_bytes else dense_bytes / packed_bytes},
        "device_bytes_allocated_after_prefill": mem_after_prefill,
        "chunks_per_layer": chunks,
        "last_logits_finite": bool(torch.isfinite(logits).all()) if decode > warm else None,
        "data": "synthetic token ids, random-init bf16 weights N(0, 0.02)",
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
