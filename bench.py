"""Benchmark of the compress-then-decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the point the headline metric is quoted on): decode attention over a packed cache at
131 072 tokens of context, 2.0-bit average, GQA 32 query / 8 KV heads, head_dim 128, batch 8 --
synthetic seeded K/V with four x10 key channels and four attention-sink tokens, compressed by this
library's own score -> allocate -> quantise/pack path.  One step = one decode-attention call over
every (sample, KV head) of the batch.  The packed cache (~0.6 GB) is larger than L2, so successive
steps re-read it from HBM.

`value` is algorithmic packed-cache bytes per second (codes + norms + exact rows that one step must
read, summed over ranks).  The reference arm (`--impl reference`) times what the reference's decode
step costs on the host cores: dense fp32 attention over a dequantised cache of the same shape, on a
bounded sample, reported in the same unit (the same algorithmic bytes per unit divided by its time).
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LEVELS = (0, 2, 3, 4, 8, 16)
METRIC = "LUT decode-attn HBM GB/s (128K ctx, 2.0-bit avg)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--group", type=int, default=4)
    ap.add_argument("--target-bits", type=float, default=2.0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--preset", default=None, choices=["config2", "config3-layer", "config4-layer"],
                    help="head shape and batch of one layer of a BASELINE configuration: config2 = GQA 32/8 batch 8 (default), "
                         "config3-layer = 28/4 batch 16 (Qwen2.5-7B shape), config4-layer = 64/8 batch 8 (Llama-3.1-70B shape)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--window-only", action="store_true",
                    help="run only the windowed attention statistics block (tcgen05 kernels) on random keys of --ctx / --batch and print it")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of a CUDA graph replay")
    args = ap.parse_args()
    if args.preset == "config3-layer":
        args.kv_heads, args.group, args.batch = 4, 7, 16
    elif args.preset == "config4-layer":
        args.kv_heads, args.group, args.batch = 8, 8, 8
    return args


def shared_config(args) -> dict:
    """The configuration both arms report (identical keys and values)."""
    return {"workload": workload_name(args.ctx, args.batch, args.kv_heads, args.group, args.target_bits),
            "l2": "inputs larger than L2: the packed cache of a step is re-read from HBM every step, no explicit flush"}


# ------------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


def window_stats_block(args, pkg, K, dev, W=128):
    """The windowed-query variant of the score stage on the tensor cores: column statistics of the causal softmax
    attention of the last W queries over the whole context of this layer (same keys as the compress pass).  Reported
    against the tensor peak and against the special-function unit, which executes one exponential per logit and pass
    and is the actual bound (16 per clock and SM)."""
    import ctypes
    import torch
    ops, L = pkg.ops, pkg._lib.lib()
    B, H, T, G = K.shape[0], K.shape[1], K.shape[2], args.group
    g = torch.Generator(device=dev).manual_seed(77)
    Qw = (torch.randn(B, H * G, W, 128, generator=g, device=dev) * 1.2).to(K.dtype)
    for _ in range(3):
        ops.window_attn_stats(Qw, K, q_offset=T - W)
    L.odmkv_timing_enable(1)
    reps = 5
    for _ in range(reps):
        ops.window_attn_stats(Qw, K, q_offset=T - W, check_status=False)
    ms = {}
    for name in ("window_lse", "window_cols"):
        tot, n = ctypes.c_double(), ctypes.c_longlong()
        L.odmkv_timing_read(name.encode(), ctypes.byref(tot), ctypes.byref(n))
        ms[name] = tot.value / max(n.value, 1)
    L.odmkv_timing_enable(0)
    # visible (query, key) pairs: query r of the window sees T - W + r + 1 keys
    pairs = B * H * G * (W * (T - W) + W * (W + 1) // 2)
    flops = 2.0 * 2 * 128 * pairs                       # two passes of q.k over every visible pair
    total_ms = ms["window_lse"] + ms["window_cols"]
    peak, kind = measured_peak_tflops()
    try:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
    except Exception:
        sms = 148
    exp_peak = 16.0 * sms * 1.965e9                     # exponentials per second at the maximum SM clock
    return {"workload": f"last {W} queries x {T} keys, batch {B}, GQA {H * G}/{H}, fp16", "ms": total_ms, "kernel_ms": ms,
            "tflops": flops / (total_ms * 1e-3) / 1e12, "tensor_peak_tflops": peak, "tensor_frac": flops / (total_ms * 1e-3) / 1e12 / peak,
            "peak_kind": f"of {kind}", "bound": "special-function unit (one ex2 per logit and pass)",
            "exp_per_s": 2.0 * pairs / (total_ms * 1e-3), "exp_frac_of_16_per_clk_sm": 2.0 * pairs / (total_ms * 1e-3) / exp_peak,
            "key_bytes_read_once_gb": B * H * T * 256 / 1e9}


def workload_name(ctx, batch, kv_heads, group, target_bits) -> str:
    return (f"decode attention over packed cache: ctx {ctx}, batch {batch}, GQA {kv_heads * group}/{kv_heads}, d 128, target "
            f"{target_bits} bits over {list(LEVELS)}, fp16 cache")


def algorithmic_bytes_per_token_head(target_bits: float) -> float:
    """Expected bytes per stored token-head for the synthetic distribution (documentation only)."""
    return 71.0 if target_bits <= 2.0 else 104.0


def dense_attention_cpu(q, Kh, Vh, keep, scale):
    """What the reference's decode step computes on the host: dense fp32 softmax(q K^T) V with evicted
    keys masked (oracle restatement; numpy, all BLAS threads)."""
    from oracle import odmkv_oracle as orc
    return orc.decode_attention(q, Kh, Vh, keep, scale)


def cpu_reference_leg(ctx, H, G, keep_frac, bytes_per_unit, steps, warmup, seed=0):
    """Times dense fp32 decode attention on the host for a bounded sample: one sample (all KV heads) of
    the workload's context length.  Returns (GB/s in the bench's unit, seconds per step, description)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    Kh = rng.standard_normal((1, H, ctx, 128), dtype=np.float32)
    Vh = rng.standard_normal((1, H, ctx, 128), dtype=np.float32)
    keep = rng.random((1, H, ctx)) < keep_frac
    q = rng.standard_normal((1, H * G, 128), dtype=np.float32)
    scale = 1.0 / math.sqrt(128)
    for _ in range(max(warmup, 1)):
        dense_attention_cpu(q, Kh, Vh, keep, scale)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        dense_attention_cpu(q, Kh, Vh, keep, scale)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    units = H  # (sample, KV head) units processed per step
    return units * bytes_per_unit / sec / 1e9, sec, f"1 sample x {H} KV heads x {ctx} tokens, dense fp32 attention (numpy), {steps} steps"


# ------------------------------------------------------------------------------------------------
# reference arm
# ------------------------------------------------------------------------------------------------

def host_threads() -> int:
    """Every host core for the numpy/BLAS baseline, whatever the launcher exported (torch.distributed.run sets
    OMP_NUM_THREADS=1).  Must run before numpy is imported."""
    n = os.cpu_count() or 1
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(n)
    return n


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    bpt = algorithmic_bytes_per_token_head(args.target_bits)
    bytes_per_unit = bpt * args.ctx
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    gbs, sec, sample = cpu_reference_leg(args.ctx, args.kv_heads, args.group, 0.883, bytes_per_unit, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": shared_config(args),
        "detail": {"timing": "host wall clock; each step is a bounded sample (one batch element, all KV heads) scaled per (sample, KV head) unit",
                   "reference_path": "dense fp32 softmax(q K^T) V over the dequantised cache with evicted keys masked, as the reference's "
                                     "decode step does on CPU; numpy restatement (the reference is Python and is not present on the GPU box)",
                   "host_threads": cores},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_compress_leg(H, G, T, target_bits, seed=0):
    """Times the oracle's compress stages on the host for one sample (all KV heads) at context T:
    score_prefill, optimal_scores_to_bits, state_prefill (route + quantise + pack).  Returns seconds per stage."""
    import numpy as np
    from oracle import odmkv_oracle as orc
    orc.build_c()
    K16, V16, Qw16, _ = orc.synth_inputs(H, T, G, 128, 64, seed, 1)
    K, V = K16[0].astype(np.float32), V16[0].astype(np.float32)
    mu = Qw16[0].astype(np.float32).mean(axis=1)
    eps = orc.calibrate_epsilon(128, LEVELS, seed=42)
    sink = np.zeros((H, T), bool)
    sink[:, :4] = True
    pi_k, pi_v = orc.random_rotation(128, 42), orc.random_rotation(128, 2042)
    t0 = time.perf_counter()
    scores = orc.score_prefill(K, V, mu, 4, 1e-2)
    t1 = time.perf_counter()
    bits = orc.optimal_scores_to_bits(scores, LEVELS, target_bits, eps, sink, eviction_cost=0.5)
    bits[:, -128:] = 16
    t2 = time.perf_counter()
    orc.state_prefill(K[None], V[None], bits[None], LEVELS, 42, pi_k, pi_v)
    t3 = time.perf_counter()
    return {"score": t1 - t0, "allocate": t2 - t1, "quantize": t3 - t2}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def compress_rooflines(stage_ms, token_heads, packed_bytes, peak):
    """Algorithmic HBM bytes of each compress stage over its measured time.  score: K and V once in 16 bit plus
    one fp32 score (516 B per token-head); allocate: score in, bit width out (8 B); quantize: K, V and the bit
    width in (516 B), packed banks out."""
    alg = {"score": 516.0 * token_heads, "allocate": 8.0 * token_heads, "quantize": 516.0 * token_heads + packed_bytes}
    out = {}
    for k, b in alg.items():
        ms = stage_ms.get(k)
        if ms:
            gbs = b / (ms * 1e-3) / 1e9
            out[k] = {"algorithmic_bytes": b, "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak}
    return out


def synth_kv(torch, B, H, T, G, dev, seed):
    """Config-0 style synthetic cache on the device: N(0,1) fp16, key channels 0-3 x10, four sink tokens."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    K = torch.randn(B, H, T, 128, generator=g, device=dev, dtype=torch.float16)
    V = torch.randn(B, H, T, 128, generator=g, device=dev, dtype=torch.float16)
    e = torch.randn(128, generator=g, device=dev)
    e = e / e.norm()
    Qw = torch.randn(B, H * G, 64, 128, generator=g, device=dev) + 3.0 * e
    qd = (torch.randn(B, H * G, 128, generator=g, device=dev) + 3.0 * e).to(torch.float16)
    K[..., 0:4] *= 10.0
    K[:, :, 0:4, :] += ((8.0 * math.sqrt(128) / 3.0) * e).to(torch.float16)
    return K, V, Qw.mean(dim=2).float(), qd


def strong_scaling_block(args, pkg, dev, world, rank, eps_list):
    """ONE layer of the workload with its KV heads split over the ranks (strong scaling): every rank scores and packs
    its heads, the per-layer Lagrangian runs with its counts all-reduced over NCCL, every decode step all-gathers the
    per-head outputs.  All ranks draw the same layer (same seed) and keep their own heads."""
    import torch
    import torch.distributed as dist
    ops = pkg.ops
    B, H, G, T = args.batch, args.kv_heads, args.group, args.ctx
    lo, hi = pkg.dist.shard_range(H, world, rank)
    Hl = hi - lo
    # the same layer on every rank, drawn head by head so that a rank only materialises its own heads
    K = torch.empty(B, Hl, T, 128, device=dev, dtype=torch.float16)
    V = torch.empty_like(K)
    g = torch.Generator(device=dev)
    g.manual_seed(4242)
    e = torch.randn(128, generator=g, device=dev)
    e = e / e.norm()
    mu_all = torch.randn(B, H * G, 128, generator=g, device=dev) * 0.125 + 3.0 * e
    qd_all = (torch.randn(B, H * G, 128, generator=g, device=dev) + 3.0 * e).to(torch.float16)
    for h in range(H):
        gh = torch.Generator(device=dev)
        gh.manual_seed(5000 + h)
        if lo <= h < hi:
            k = torch.randn(B, T, 128, generator=gh, device=dev, dtype=torch.float16)
            k[..., 0:4] *= 10.0
            k[:, 0:4, :] += ((8.0 * math.sqrt(128) / 3.0) * e).to(torch.float16)
            K[:, h - lo] = k
            V[:, h - lo] = torch.randn(B, T, 128, generator=gh, device=dev, dtype=torch.float16)
    mu = mu_all[:, lo * G:hi * G].contiguous()
    qd = qd_all[:, lo * G:hi * G].contiguous()
    sink = torch.zeros(Hl, T, dtype=torch.bool, device=dev)
    sink[:, :4] = True
    State = pkg.tq_adaptive_backend.TurboQuantAdaptiveKVCacheState

    def compress():
        scores = ops.score_prefill(K, V, mu, 4, 1e-2)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        bits, _ = pkg.dist.allocate_bits_kv_sharded(scores, sink, LEVELS, eps_list, args.target_bits, head_lo=lo, T=T)
        a1.record()
        bits = bits.reshape(B, Hl, T).clone()
        bits[..., -128:] = 16
        st = State(head_dim=128, bit_levels=LEVELS, device=dev, dtype=torch.float16, key_quantizer="mse", value_quantizer="mse", seed=42)
        st.prefill(K, V, bits)
        return st, (a0, a1)

    st, _ = compress()
    torch.cuda.synchronize()
    dist.barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    st, (a0, a1) = compress()
    c1.record()
    torch.cuda.synchronize()
    compress_ms, alloc_ms = c0.elapsed_time(c1), a0.elapsed_time(a1)
    del K, V
    out = st.decode_attention(qd)
    gathered = torch.empty(world, *out.shape, dtype=out.dtype, device=dev)
    dist.all_gather_into_tensor(gathered, out)
    # one CUDA graph per step: the decode call's launches and the NCCL all-gather of the outputs
    graph = None
    try:
        gq = qd.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            go = st.decode_attention(gq)
            dist.all_gather_into_tensor(gathered, go)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    except Exception:
        graph = None

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            dist.all_gather_into_tensor(gathered, st.decode_attention(qd))

    for _ in range(max(args.warmup, 3)):
        one_step()
    torch.cuda.synchronize()
    dist.barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        one_step()
    s1.record()
    torch.cuda.synchronize()
    dist.barrier()
    vals = torch.tensor([s0.elapsed_time(s1) / args.steps, compress_ms, alloc_ms, float(st.chunks[0].packed_bytes())], dtype=torch.float64, device=dev)
    mx = vals.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = vals.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    step_ms, bytes_all = mx[0].item(), sm[3].item()
    return {"scaling": "strong", "what": f"one layer, {H} KV heads split over {world} ranks ({Hl} per rank), batch {B}, ctx {T}",
            "ms_per_step": step_ms, "value": bytes_all / (step_ms * 1e-3) / 1e9, "unit": "GB/s",
            "step": "CUDA graph of the decode call and the all-gather" if graph is not None else "eager decode call and all-gather",
            "collectives": "per step: NCCL all-gather of [B, Hq / N, 128] fp16 outputs; compress: NCCL all-reduce of 16 int64 counters per "
                           "allocator pass (a 64 K-bin histogram per gap-closure pass)",
            "compress_ms": mx[1].item(), "allocate_sharded_ms": mx[2].item(), "mtok_per_s": B * T / (mx[1].item() * 1e-3) / 1e6}


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = importlib.import_module("odm-kv_b200")
    ops, L = pkg.ops, pkg._lib.lib()
    B, H, G, T = args.batch, args.kv_heads, args.group, args.ctx

    # ---- build the packed cache with this library's compress path (timed: compress throughput)
    eps = pkg.allocator.calibrate_epsilon(128, LEVELS, seed=42, device=dev)
    eps_list = [eps[b] * (0.5 if b == 0 else 1.0) for b in LEVELS]
    K, V, mu, qd = synth_kv(torch, B, H, T, G, dev, seed=1000 + rank)
    sink = torch.zeros(H, T, dtype=torch.uint8, device=dev)
    sink[:, :4] = 1
    sink = sink.reshape(-1)

    State = pkg.tq_adaptive_backend.TurboQuantAdaptiveKVCacheState

    def compress():
        """score -> allocate -> window override -> state.prefill (route, quantise, pack): what the press hook does for a layer."""
        scores = ops.score_prefill(K, V, mu, 4, 1e-2)
        bits, rep = ops.allocate_bits(scores.reshape(B, H * T), sink, LEVELS, eps_list, args.target_bits)
        bits = bits.reshape(B, H, T)
        bits[..., -128:] = 16
        state = State(head_dim=128, bit_levels=LEVELS, device=dev, dtype=torch.float16, key_quantizer="mse", value_quantizer="mse", seed=42)
        state.prefill(K, V, bits)
        return state, rep

    L.odmkv_timing_enable(0)
    for _ in range(2):                # warm-up; freed so that the timed run reuses its device blocks
        warm, _ = compress()
        torch.cuda.synchronize()
        del warm
    stage_ms = {}
    L.odmkv_timing_enable(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    state, rep = compress()           # timed; also the cache the decode steps read
    chunk = state.chunks[0]
    e1.record()
    torch.cuda.synchronize()
    compress_ms = e0.elapsed_time(e1)
    import ctypes
    for name in ("score", "allocate", "quantize"):
        tot, n = ctypes.c_double(), ctypes.c_longlong()
        L.odmkv_timing_read(name.encode(), ctypes.byref(tot), ctypes.byref(n))
        stage_ms[name] = tot.value
    L.odmkv_timing_enable(0)
    window = window_stats_block(args, pkg, K, dev)
    reports = ops.read_reports(rep)
    pi_k, pi_v = state.pi_k, state.pi_v
    cnt = chunk.seg_count_host().sum(axis=1)
    stored = int(cnt[1:].sum())
    bytes_per_step = chunk.packed_bytes()
    del K, V
    torch.cuda.empty_cache()

    # ---- decode steps
    n_splits = args.splits
    q_steps = [qd.clone() for _ in range(2)]

    def step(i):
        return ops.decode_attn(q_steps[i & 1], [chunk], pi_k, pi_v, n_splits=n_splits)

    # clocks are sampled from the warm-up through the end-to-end loop: the timed region alone lasts only
    # a few milliseconds, less than one nvidia-smi sampling period
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(max(args.warmup, 3)):
        out = step(i)
    torch.cuda.synchronize()

    # The timed step is one CUDA graph of the four launches of a decode call (rotate, tensor-core kernel,
    # exact/tail kernel on a forked stream, merge), replayed once per step: no host work inside the region.
    step_mode = "cuda graph replay of one decode call"
    graph = None
    graph_err = None
    if not args.eager:
        try:
            gq = qd.clone()
            graph = torch.cuda.CUDAGraph()
            # thread-local capture mode: other threads (the NCCL watchdog under torchrun) may keep making CUDA calls
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                g_out = ops.decode_attn(gq, [chunk], pi_k, pi_v, n_splits=n_splits)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            graph_err = float((g_out.float() - out.float()).abs().max())
        except Exception as exc:
            graph, graph_err = None, repr(exc)[:200]
    if graph is None:
        step_mode = "eager launches through the C ABI"

    def timed_step(i):
        if graph is not None:
            graph.replay()
            return g_out
        return step(i)

    # Multi-GPU schedules.  Headline: every rank owns whole (layer, sample, KV head) units, so a decode step needs
    # no exchange and the outputs are gathered once after the K steps (inside the timed region).  Also measured:
    # the KV-head-sharded schedule of one layer, which all-gathers the outputs after every step.
    def timed_loop(gather_every_step):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        o = None
        for i in range(args.steps):
            o = timed_step(i)
            if world > 1 and gather_every_step:
                dist.all_gather(gathered, o)
        if world > 1 and not gather_every_step:
            dist.all_gather(gathered, o)
        b.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return a.elapsed_time(b)

    gathered = [torch.empty_like(out) for _ in range(world)] if world > 1 else None
    if world > 1:
        dist.all_gather(gathered, out)   # NCCL warm-up outside the timed region
    total_ms = timed_loop(gather_every_step=False)
    tp_ms = timed_loop(gather_every_step=True) if world > 1 else None

    # per-kernel durations: the same steps launched eagerly with an event pair around each kernel
    L.odmkv_timing_enable(1)
    ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ee0.record()
    for i in range(args.steps):
        out = step(i)
    ee1.record()
    torch.cuda.synchronize()
    eager_ms = ee0.elapsed_time(ee1) / args.steps
    tot, n = ctypes.c_double(), ctypes.c_longlong()
    L.odmkv_timing_read(b"decode_main", ctypes.byref(tot), ctypes.byref(n))
    parts_ms = {}
    for name in ("decode_rotate", "decode_side", "decode_merge"):
        t2, n2 = ctypes.c_double(), ctypes.c_longlong()
        L.odmkv_timing_read(name.encode(), ctypes.byref(t2), ctypes.byref(n2))
        parts_ms[name] = t2.value / max(n2.value, 1)
    L.odmkv_timing_enable(0)
    main_ms = tot.value / max(n.value, 1)

    # ---- end to end through the cache-state API with host buffers (pinned q in, output out)
    q_host = qd.cpu().pin_memory()
    out_host = torch.empty(B, H * G, 128, dtype=torch.float16).pin_memory()
    q_dev = torch.empty_like(qd)

    def e2e_step(plugin=True):
        """Host query in, attention output out.  plugin=True: the cache-state call the attention override makes
        (state.decode_attention); False: the tensor-level op underneath it."""
        q_dev.copy_(q_host, non_blocking=True)
        o = state.decode_attention(q_dev) if plugin else ops.decode_attn(q_dev, [chunk], pi_k, pi_v, n_splits=n_splits)
        out_host.copy_(o, non_blocking=True)

    def e2e_time(plugin):
        for _ in range(3):
            e2e_step(plugin)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step(plugin)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3

    e2e_ms = e2e_time(True)
    e2e_ops_ms = e2e_time(False)
    # the same end-to-end step (host query in, host output out) as one CUDA graph: copy node, the decode call's
    # launches, copy node
    e2e_graph_ms = None
    if not args.eager:
        try:
            eg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(eg, capture_error_mode="thread_local"):
                q_dev.copy_(q_host, non_blocking=True)
                eo = state.decode_attention(q_dev)
                out_host.copy_(eo, non_blocking=True)
            for _ in range(3):
                eg.replay()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                eg.replay()
            torch.cuda.synchronize()
            e2e_graph_ms = (time.perf_counter() - t0) * 1e3
        except Exception:
            e2e_graph_ms = None
    # keep the same decode load running until the sampler has seen it for a while
    t_load = time.perf_counter()
    while rank == 0 and time.perf_counter() - t_load < 0.6:
        for i in range(50):
            step(i)
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # ---- max over ranks, totals over ranks
    strong = strong_scaling_block(args, pkg, dev, world, rank, eps_list) if world > 1 and H % world == 0 else None
    stats = torch.tensor([total_ms, e2e_ms, float(bytes_per_step), main_ms, compress_ms, tp_ms or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, main_ms, compress_ms, tp_ms = mx[0].item(), mx[1].item(), mx[3].item(), mx[4].item(), mx[5].item()
        bytes_all = sm[2].item()
    else:
        bytes_all = float(bytes_per_step)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    value = bytes_all / (ms_per_step * 1e-3) / 1e9
    e2e_value = bytes_all / (e2e_ms / args.steps * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()
    achieved = bytes_per_step / (main_ms * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "decode_traffic.json")
    if os.path.exists(tpath):
        try:
            tj = json.load(open(tpath))
            traffic = tj["dram_bytes_per_algorithmic_byte"] * bytes_per_step
        except Exception:
            traffic = None
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "us_per_step": ms_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 codes -> f32 accumulate", "data": "synthetic",
        "config": shared_config(args),
        "detail": {"packed_cache_mb_per_rank": bytes_per_step / 1e6,
                   "timing": "CUDA events on the launching stream, max over ranks; per-kernel times from a second, eager pass of the same steps",
                   "level_counts": {str(b): int(c) for b, c in zip(LEVELS, cnt)},
                   "stored_token_heads": stored, "bytes_per_step_per_rank": bytes_per_step,
                   "n_splits": n_splits,
                   "multi_gpu": "weak scaling of independent replicas: each rank holds its own (layer, sample, KV head) units, no exchange "
                                "inside a step, outputs all-gathered once after the timed steps; the KV-head-sharded schedule of ONE layer "
                                "(strong scaling, collectives inside) is the `strong_scaling` block" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": f"of {peak_kind}", "kernel": "decode_main", "kernel_ms": main_ms,
                     "frac_of_8000": achieved / 8000.0, "other_kernels_ms": parts_ms},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": int(q_host.numel() * 2 * world),
                "d2h_bytes_per_step": int(out_host.numel() * 2 * world), "ms_per_step": e2e_ms / args.steps,
                "call": "state.decode_attention(q) of the cache-state API per step, eager, host wall clock: pinned query in, output out",
                "ops_level_ms_per_step": e2e_ops_ms / args.steps,
                "graph_replay_ms_per_step": None if e2e_graph_ms is None else e2e_graph_ms / args.steps},
        "gpu_launches": 4 * args.steps,
        "gather_per_step": None if tp_ms is None else {
            "schedule": "KV heads of one layer sharded over the ranks: outputs all-gathered (NCCL) after every step",
            "ms_per_step": tp_ms / args.steps, "value": bytes_all / (tp_ms / args.steps * 1e-3) / 1e9},
        "strong_scaling": strong,
        "step_mode": {"timed_step": step_mode, "graph_vs_eager_max_abs_diff": graph_err,
                      "eager_ms_per_step_with_kernel_events": eager_ms},
        "clocks": clocks,
        "compress": {"mtok_per_s": B * T / (compress_ms * 1e-3) / 1e6, "ms_per_layer": compress_ms, "stage_ms": stage_ms,
                     "stage_roofline": compress_rooflines(stage_ms, B * H * T, bytes_per_step, peak),
                     "tokens": B * T, "alloc_evaluations": reports[0]["evaluations"], "alloc_moved": reports[0]["moved"],
                     "ties_lambda": sum(r["ties_lambda"] for r in reports), "ties_cut": sum(r["ties_cut"] for r in reports),
                     "window_stats": window},
    }
    if not args.no_cpu_baseline and world == 1:
        cores = os.cpu_count() or 1
        gbs, sec, sample = cpu_reference_leg(T, H, G, stored / float(B * H * T), bytes_per_step / float(B * H), 5, 1)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                                "sec_per_step_of_sample": sec}
        # compress on the host: one sample at a shorter context; every stage is linear in the tokens except the
        # allocator's sort (n log n), so tokens / second carries over to the full context within a few per cent
        Tc = min(T, 8192)
        cs = cpu_compress_leg(H, G, Tc, args.target_bits)
        tot = sum(cs.values())
        line["compress"]["cpu_baseline"] = {
            "mtok_per_s": Tc / tot / 1e6, "stage_s": cs, "cores": cores, "kind": "port",
            "sample": f"1 sample x {H} KV heads x {Tc} tokens: oracle score_prefill + optimal_scores_to_bits + state_prefill (numpy + C)",
            "scaling_rule": "tokens per second measured on the sample stands for the full context (stages linear in tokens)"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_window_only(args):
    import importlib
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    dev = torch.device("cuda", 0)
    pkg = importlib.import_module("odm-kv_b200")
    g = torch.Generator(device=dev).manual_seed(1)
    K = torch.randn(args.batch, args.kv_heads, args.ctx, 128, generator=g, device=dev).half()
    print(json.dumps({"window_stats": window_stats_block(args, pkg, K, dev)}), flush=True)


def main():
    args = parse()
    if args.window_only:
        run_window_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
