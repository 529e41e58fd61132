"""Stand-alone peer-memory collectives against torch.distributed (NCCL) on 2 GPUs (or more)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from lightron_b200.ops import native
from lightron_b200.parallel import peer_collectives as pc
rank, n = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
comm = pc.PeerComm(dist.group.WORLD, max_bytes=16 << 20, ctas=16)     # the all-gather stages n x 2 MiB at most
g = torch.Generator(device="cuda").manual_seed(100 + rank)
for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
    for m in (8, 1000, 16384):
        for rep in range(3):                                  # calls alternate between the two halves
            x = torch.randn(n * m, 8, device="cuda", generator=g).to(dtype)
            want = [torch.empty_like(x) for _ in range(n)]
            dist.all_gather(want, x)
            assert torch.equal(comm.all_gather(x), torch.cat(want)), ("all_gather", dtype, m)
            ref = torch.empty_like(x); dist.all_to_all_single(ref, x)
            assert torch.equal(comm.all_to_all(x), ref), ("all_to_all", dtype, m)
            ref = x.float().clone(); dist.all_reduce(ref)
            got = comm.all_reduce(x, nvls=False).float()
            assert (got - ref).abs().max() <= tol * ref.abs().max().clamp_min(1), ("all_reduce", dtype, m)
            got = comm.reduce_scatter(x).float()
            assert (got - ref.view(n, -1)[rank].view_as(got)).abs().max() <= tol * ref.abs().max().clamp_min(1), ("reduce_scatter", dtype, m)
            if comm.mc_ptr:
                got = comm.all_reduce(x, nvls=True).float()
                assert (got - ref).abs().max() <= tol * ref.abs().max().clamp_min(1), ("all_reduce_nvls", dtype, m)
torch.cuda.synchronize()
assert not native.device_status()
if rank == 0:
    print("PEER_COLLECTIVES_OK nvls=%d" % (1 if comm.mc_ptr else 0), flush=True)
dist.barrier()
dist.destroy_process_group()
'''


def test_peer_collectives_match_nccl(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29571", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "PEER_COLLECTIVES_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-6000:]


EMBED_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from lightron_b200.ops import native, functional as OF
from lightron_b200.parallel import embed_fused, comm
rank, n = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
group = dist.new_group(list(range(n)))
V, H = 1024, 256
torch.manual_seed(5)
table = (torch.randn(V, H, device="cuda") * 0.1).to(torch.bfloat16)
local = V // n
for sp in (True, False):
    for T in (n * 96, n * 1000, n * 4096):
        for rep in range(3):                                   # staging buffers alternate
            tok = torch.randint(0, V, (T,), device="cuda")
            dist.broadcast(tok, 0)
            w = table[rank * local:(rank + 1) * local].clone().requires_grad_(True)
            assert embed_fused.fused_ok(w, group, T, sp)
            out = embed_fused.vocab_parallel_embedding(tok, w, group, rank * local, sp)
            want = table[tok]
            rows = T // n
            if sp:
                want = want[rank * rows:(rank + 1) * rows]
            assert torch.equal(out, want), ("forward", sp, T)
            dy_full = (torch.randn(T, H, device="cuda") * 0.1).to(torch.bfloat16)
            dist.broadcast(dy_full, 0)
            dy = dy_full[rank * rows:(rank + 1) * rows] if sp else dy_full
            out.backward(dy.contiguous())
            ref = torch.zeros(V, H, device="cuda").index_add_(0, tok, dy_full.float())[rank * local:(rank + 1) * local]
            err = (w.grad.float() - ref).norm() / ref.norm()
            assert err < 2e-2, ("backward", sp, T, float(err))       # bf16 atomics round as they add
torch.cuda.synchronize()
assert not native.device_status()
if rank == 0:
    print("PEER_EMBEDDING_OK", flush=True)
dist.barrier()
dist.destroy_process_group()
'''


def test_vocab_parallel_embedding_by_peer_stores(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "w.py"
    script.write_text(EMBED_WORKER)
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29572", str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "PEER_EMBEDDING_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-6000:]
