"""GPU, two or more devices: the N-sharded GEMM (weight rows split over the ranks, one process per GPU over NCCL)
gives, after a gather along N, the bits of the one-GPU GEMM; row-sharded quantization with the importance reduced by
column slices gives the bytes of one GPU.  Skipped when fewer than two GPUs are visible."""
import os
import pathlib
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NVFP4_ROOT"])
import nvfp4quant_test_b200.kernels as K
from nvfp4quant_test_b200 import gemm_sweep as GS
from nvfp4quant_test_b200.sharding import column_shards, row_shards, scale_slab
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)
M, N, Kd = 2048, 28672, 1024
x = GS.laplace((M, Kd), 3, dev)
w = GS.laplace((N, Kd), 4, dev)                       # every rank builds the same weight and keeps its rows
qa, sa, gsa = GS.quantize_operand("ScaleSweep", x, w)
qw, sw, gsw = GS.quantize_operand("ScaleSweep", w, x)  # tensor-wide global scale, so shards agree with the whole
alpha = (gsa * gsw).reshape(1).float()
a, b = column_shards(N, world)[rank]
lo, hi = scale_slab(a, b, Kd // 16)
part = K.nvfp4_scaled_mm(qa, qw[a:b].contiguous(), sa, sw.view(torch.uint8).reshape(-1)[lo:hi].contiguous(), alpha, torch.bfloat16)
parts = [torch.empty((M, s1 - s0), dtype=torch.bfloat16, device=dev) for s0, s1 in column_shards(N, world)]
if len({p.shape for p in parts}) == 1:
    dist.all_gather(parts, part)                      # the optional final gather along N
else:
    for r, p in enumerate(parts):
        if r == rank: p.copy_(part)
        dist.broadcast(p, src=r)
full = torch.cat(parts, 1)
want = K.nvfp4_scaled_mm(qa, qw, sa, sw, alpha, torch.bfloat16)
assert torch.equal(full, want), f"rank {rank}: {(full != want).sum().item()} outputs differ"
# row-sharded quantization of the same weight: this rank's rows quantize to the same bytes as inside the whole
ra, rb = row_shards(N, world)[rank]
qs, ss, _ = GS.quantize_operand("ScaleSweep_MSE", w[ra:rb].contiguous(), x)
qf, sf, _ = GS.quantize_operand("ScaleSweep_MSE", w, x)
import nvfp4quant_test_b200.helper as H
_, gi = H.get_nvfp4_global_scale(w, 256.0)
qs, ss = K.scalesweep_mse_nvfp4_quant_impl(w[ra:rb].contiguous(), gi)
l2, h2 = scale_slab(ra, rb, Kd // 16)
assert torch.equal(qs, qf[ra:rb]) and torch.equal(ss.view(torch.uint8).reshape(-1), sf.view(torch.uint8).reshape(-1)[l2:h2])
# importance reduced by column slices + local scales of the row shards, one all-gather: the bits of one GPU, and the
# weighted sweep of this rank's rows with them equals its rows inside the whole
from nvfp4quant_test_b200.sharding import ImportanceGather
ig = ImportanceGather(Kd, dev)
c0, c1 = ig.columns
H.channel_square_norm(x[:, c0:c1], out=ig.imp_slot)
H.get_nvfp4_global_scale(w[ra:rb].contiguous(), 256.0, out=ig.scale_slot)
imp, gs_all, gs_inv = ig.gather()
gs_one, gi_one = H.get_nvfp4_global_scale(w, 256.0)
assert torch.equal(imp, H.channel_square_norm(x)) and torch.equal(gs_all, gs_one) and torch.equal(gs_inv, gi_one)
qs, ss = K.scalesweep_weighted_mse_nvfp4_quant_impl(w[ra:rb].contiguous(), imp, gs_inv)
qf, sf = K.scalesweep_weighted_mse_nvfp4_quant_impl(w, H.channel_square_norm(x), gi_one)
assert torch.equal(qs, qf[ra:rb]) and torch.equal(ss.view(torch.uint8).reshape(-1), sf.view(torch.uint8).reshape(-1)[l2:h2])
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_n_sharded_gemm_equals_one_gpu(cuda_lib, tmp_path):
    world = min(torch.cuda.device_count(), 4)
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NVFP4_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29531", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(" ok") == world
