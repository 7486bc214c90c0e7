"""Two-GPU checks of the sharded path (skipped on a single GPU): KV heads of one Lagrangian problem split over
two ranks with the count exchange over NCCL, and the gather of per-head attention outputs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import importlib, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ODMKV_ROOT"])
pkg = importlib.import_module("odm-kv_b200")
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
LEVELS = (0, 2, 3, 4, 8, 16)
eps = pkg.allocator.calibrate_epsilon(128, LEVELS, seed=42, device=dev)
ev = [eps[b] * (0.5 if b == 0 else 1.0) for b in LEVELS]
H, T, P = 4, 3000, 2
rng = np.random.default_rng(0)                        # same scores on every rank
scores = torch.from_numpy(np.exp(rng.standard_normal((P, H, T)) * 2 - 2).astype(np.float32)).to(dev)
sink = torch.zeros(H, T, dtype=torch.bool, device=dev); sink[:, :4] = True
full, _ = pkg.ops.allocate_bits(scores.reshape(P, -1), sink.reshape(-1), LEVELS, ev, 2.0)
lo, hi = pkg.dist.shard_range(H, world, rank)
mine, _ = pkg.dist.allocate_bits_kv_sharded(scores[:, lo:hi].contiguous(), sink[lo:hi].contiguous(), LEVELS, ev, 2.0, head_lo=lo, T=T)
assert torch.equal(mine, full.reshape(P, H, T)[:, lo:hi]), "sharded allocation differs from the single-device one"
out = torch.full((2, 4, 128), float(rank), device=dev, dtype=torch.float16)
allh = pkg.dist.gather_head_outputs(out)
assert allh.shape == (2, 4 * world, 128) and all(float(allh[0, 4 * r, 0]) == r for r in range(world))
# head-sharded decode attention: every rank packs and attends its own KV heads, the gathered outputs equal
# what one device computes over all heads
B, G, Td = 2, 4, 700
g = torch.Generator(device="cpu").manual_seed(3)            # same layer on every rank
Kf = torch.randn(B, H, Td, 128, generator=g).half().to(dev)
Vf = torch.randn(B, H, Td, 128, generator=g).half().to(dev)
q = torch.randn(B, H * G, 128, generator=g).half().to(dev)
bits = torch.from_numpy(rng.choice(np.array(LEVELS, np.int32), size=(B, H, Td), p=(0.1, 0.5, 0.25, 0.05, 0.05, 0.05)).astype(np.int32)).to(dev)
pk = pkg.tq_backend.random_rotation(128, dev, torch.float32, seed=42)
pv = pkg.tq_backend.random_rotation(128, dev, torch.float32, seed=2042)
whole = pkg.ops.decode_attn(q, [pkg.ops.quantize_pack(Kf, Vf, bits, pk, pv)], pk, pv, out_dtype=torch.float32)
mine = pkg.ops.decode_attn(q[:, lo * G:hi * G].contiguous(),
                           [pkg.ops.quantize_pack(Kf[:, lo:hi].contiguous(), Vf[:, lo:hi].contiguous(), bits[:, lo:hi].contiguous(), pk, pv)],
                           pk, pv, out_dtype=torch.float32)
gathered = pkg.dist.gather_head_outputs(mine)
assert gathered.shape == whole.shape
assert float((gathered - whole).abs().max() / whole.abs().max()) < 1e-5, "head-sharded decode differs from the single-device result"
dist.barrier()
if rank == 0:
    print("MULTI_GPU_OK")
dist.destroy_process_group()
'''


def test_kv_head_sharded_allocation_and_gather_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, ODMKV_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", "29533", str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "MULTI_GPU_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
