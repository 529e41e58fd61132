"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels against NCCL collectives + fp32 matmul.
Needs at least 2 GPUs; runs as child processes (one per GPU)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from lightron_b200.parallel import symm, comm, fused
from lightron_b200.ops import functional as OF
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl")
g = dist.new_group(list(range(world)))
dev = torch.device("cuda", rank)
def rel(a, b): return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()
torch.manual_seed(1234)           # same full tensors everywhere, each rank slices its part
for it, (M, N, K) in enumerate([(256 * world, 512, 256), (1024 * world, 1280, 512), (256 * world, 264, 192), (2048 * world, 2048, 1024)]):
    xf = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    rows = M // world
    x_local = xf[rank * rows:(rank + 1) * rows].contiguous()
    y, gathered, _ = symm.ag_gemm(x_local, w, g)
    torch.cuda.synchronize()
    assert torch.equal(gathered, xf), f"gathered mismatch it={it}"
    want = xf.float() @ w.float().t()
    assert rel(y, want) < 5e-3, f"ag_gemm rel {rel(y, want)} it={it}"
    # GEMM -> reduce-scatter with K sharded: rank r holds columns [r*K/world, ...)
    kl = K // world
    xs = xf[:, rank * kl:(rank + 1) * kl].contiguous()
    wsh = w[:, rank * kl:(rank + 1) * kl].contiguous()
    out = symm.gemm_rs(xs, wsh, g)
    torch.cuda.synchronize()
    want_rs = want[rank * rows:(rank + 1) * rows]
    assert rel(out, want_rs) < 1e-2, f"gemm_rs rel {rel(out, want_rs)} it={it}"
    # b_mn variants (backward shapes)
    wt = w.t().contiguous()                  # [K, N] storage
    y2, _, _ = symm.ag_gemm(x_local, wt, g, b_mn=True)
    assert rel(y2, want) < 5e-3
symm.check_status()
# autograd parity with the library-collective path
M, K, N = 512 * world, 256, 384
torch.manual_seed(7)
xf = torch.randn(M, K, device=dev).to(torch.bfloat16)
w1 = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
w2 = (torch.randn(K, N // world, device=dev) * 0.05).to(torch.bfloat16)
rows = M // world
res = []
for use_fused in (True, False):
    fused.set_fused(use_fused)
    x = xf[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
    a, b = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    h = fused.all_gather_linear(x, (a,), g)                      # [M, N]
    hs = h[:, rank * (N // world):(rank + 1) * (N // world)].contiguous()
    o = fused.linear_reduce_scatter(hs, b, g)                    # [rows, K]
    o.backward(torch.ones_like(o) * 0.01)
    res.append((o.detach(), x.grad, a.grad, b.grad))
for t_f, t_n in zip(*res):
    assert rel(t_f, t_n) < 2e-2, rel(t_f, t_n)
symm.check_status()
dist.barrier()
if rank == 0: print("FUSED_COMM_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ag_gemm_and_gemm_rs(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    n = 2 if n < 4 else 4
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FUSED_COMM_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


DP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from lightron_b200 import mesh
from lightron_b200.config import ModelArgs
from lightron_b200.models import LightronTransformer, init_weights
from lightron_b200.optim import DistributedAdamW
world = int(os.environ["WORLD_SIZE"])
ctx = mesh.setup_distributed(dp_size=world)
dev = ctx.device
args = ModelArgs(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=1024, intermediate_size=512, max_seq_len=128)
finals = []
for fused in ("1", "0"):
    os.environ["LIGHTRON_FUSED_DP"] = fused
    m = LightronTransformer(args, ctx, dtype=torch.bfloat16, device=dev)
    init_weights(m, 3)
    opt = DistributedAdamW(m, lr=1e-3, ctx=ctx)
    assert (opt.fused_dp is not None) == (fused == "1")
    g = torch.Generator().manual_seed(100 + ctx.rank)
    for step in range(3):
        tok = torch.randint(0, 1024, (2, 128), generator=g).to(dev)
        opt.zero_grad()
        loss = m.loss(tok, torch.roll(tok, -1, 1))
        loss.backward()
        opt.step()
        assert torch.isfinite(loss).item() and not torch.isnan(opt.master).any().item()
    torch.cuda.synchronize()
    finals.append(opt.flat_params.float().clone())
    # replicas must hold identical parameters after the step
    ref = finals[-1].clone(); dist.broadcast(ref, src=0)
    if not torch.equal(ref, finals[-1]):
        bad = (ref != finals[-1]).nonzero().flatten()
        raise AssertionError(f"replicas diverged (fused={fused}): {bad.numel()} of {ref.numel()} elements, first {bad[:4].tolist()} "
                             f"last {bad[-4:].tolist()}, shard_len {opt.buckets[0].shard_len}, max diff {(ref - finals[-1]).abs().max().item()}")
import ctypes
from lightron_b200.ops import native
buf = (ctypes.c_uint * 4)(); native.require().lb_dp_status(ctypes.cast(buf, ctypes.c_void_p)); assert buf[0] == 0, list(buf)
rel = ((finals[0] - finals[1]).norm() / finals[1].norm()).item()
assert rel < 2e-3, rel
dist.barrier()
if ctx.rank == 0: print("FUSED_DP_OK", rel)
mesh.destroy()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_dp_adamw_matches_nccl_path(tmp_path):
    script = tmp_path / "dp_worker.py"
    script.write_text(DP_WORKER)
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29542", str(script)], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FUSED_DP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
