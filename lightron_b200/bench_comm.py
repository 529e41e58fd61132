"""Times the fused compute + collective paths of tensor parallelism against their library
counterparts and their roofline, on the 1.1B layer shapes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29620 -m lightron_b200.bench_comm [--tokens 16384]

Every number is CUDA-event time on the launching stream (3 warm-up calls, 10 timed, barrier and
synchronize on both sides), MAX over ranks.  Roofline of a fused path = the slower of the GEMM alone
(the same kernel family, measured here) and the bytes that must cross NVLink at the peer-copy rate
measured here with a plain device-to-device copy engine transfer.  Rank 0 prints a markdown table;
SM clocks are sampled with nvidia-smi while each row is timed.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--publish", action="store_true",
                    help="only measure what publishing an SM-issued peer copy costs (fence + flag per chunk) and exit")
    args = ap.parse_args()
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from bench import ClockSampler
    from lightron_b200.ops import functional as OF
    from lightron_b200.parallel import comm, symm

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    g = dist.new_group(list(range(world)))
    dev = torch.device("cuda", torch.cuda.current_device())

    def bench(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        sampler = ClockSampler(torch.cuda.current_device())
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item(), (clocks or {}).get("sm_mhz")

    T = args.tokens
    # peer copy rate: one copy-engine transfer of 256 MiB into the peer's symmetric buffer
    import torch.distributed._symmetric_memory as symm_mem
    nbytes = 256 << 20
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
    hdl = symm_mem.rendezvous(buf, group=g)
    src = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    peer = hdl.get_buffer((rank + 1) % world, (nbytes,), torch.uint8)
    t_copy, _ = bench(lambda: peer.copy_(src, non_blocking=True))
    link_gbs = nbytes / t_copy / 1e6
    # the same transfer issued by SMs (lb_peer_copy): 16-byte stores by every thread, and bulk copies
    # through shared memory issued by one thread per CTA, for several CTA counts
    from lightron_b200.ops import native
    sm_rates = []
    for mode, label in ((0, "16-byte stores"), (1, "bulk copies via shared memory")):
        for ctas in (8, 16, 32, 64, 148):
            t_sm, _ = bench(lambda: native.call("lb_peer_copy", src.data_ptr(), peer.data_ptr(), nbytes, mode, ctas,
                                                native.stream_ptr()), iters=5)
            sm_rates.append((label, ctas, nbytes / t_sm / 1e6))
    if args.publish:
        # lb_peer_copy_flagged: the same copy, every chunk followed by a system-scope fence and a release-add on a
        # flag word in the peer's memory (mode 2: the whole CTA; mode 3: a signalling warp), 64 MiB
        nb = 64 << 20
        fbuf = symm_mem.empty(1 << 20, dtype=torch.uint8, device=dev)
        fbuf.zero_()
        fh = symm_mem.rendezvous(fbuf, group=g)
        pflags = fh.get_buffer((rank + 1) % world, (1 << 20,), torch.uint8)
        lines = []
        for ctas in (16, 32):
            t, _ = bench(lambda: native.call("lb_peer_copy", src.data_ptr(), peer.data_ptr(), nb, 0, ctas, native.stream_ptr()))
            lines.append(f"plain copy, {ctas} CTAs: {nb / t / 1e6:.0f} GB/s")
            for mode in (2, 3):
                for chunk in (128 << 10, 512 << 10, 2 << 20):
                    t, _ = bench(lambda: native.call("lb_peer_copy_flagged", src.data_ptr(), peer.data_ptr(), nb, mode, ctas,
                                                     chunk, pflags.data_ptr(), native.stream_ptr()))
                    lines.append(f"mode {mode}, {ctas} CTAs, chunk {chunk >> 10} KiB: {nb / t / 1e6:.0f} GB/s")
        native.raise_on_device_status()
        if rank == 0:
            print("\n".join(lines), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    rows = []
    for name, N, K in [("qkv", 2560 // world, 2048), ("gate+up", 11264 // world, 2048), ("LM head", 32000 // world, 2048),
                       ("dgrad of down (dy gathered)", 5632 // world, 2048), ("dgrad of wo (dy gathered)", 2048 // world, 2048)]:
        x = torch.randn(T // world, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        xf = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        res = {}
        for tr in ("sm", "ce"):
            symm.AG_TRANSPORT = tr
            res[tr], mhz = bench(lambda: symm.ag_gemm(x, w, g))
        t_lib, _ = bench(lambda: OF.gemm(comm.all_gather_rows(x, g), w))
        t_gemm, _ = bench(lambda: OF.gemm(xf, w))
        t_link = (T // world) * K * 2 * (world - 1) / (link_gbs * 1e6)          # ms: bytes this rank must send
        roof = max(t_gemm, t_link)
        rows.append((f"all-gather -> GEMM, {name} (N {N}, K {K})", res["sm"], res["ce"], t_lib, t_gemm, t_link, roof, mhz))
    for name, N, K in [("wo", 2048, 2048 // world), ("down", 2048, 5632 // world), ("dgrad of qkv", 2048, 2560 // world),
                       ("dgrad of gate+up", 2048, 11264 // world)]:
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        t_f, mhz = bench(lambda: symm.gemm_rs(x, w, g))
        t_lib, _ = bench(lambda: comm.reduce_scatter_rows(OF.gemm(x, w), g))
        t_gemm, _ = bench(lambda: OF.gemm(x, w))
        t_link = (T // world) * N * 2 * (world - 1) / (link_gbs * 1e6)
        roof = max(t_gemm, t_link)
        rows.append((f"GEMM -> reduce-scatter, {name} (N {N}, K {K})", t_f, None, t_lib, t_gemm, t_link, roof, mhz))
    symm.check_status()
    if rank == 0:
        print(f"peer copy (copy engine, 256 MiB): {link_gbs:.0f} GB/s per direction; {world} ranks, {T} tokens")
        print("peer copy issued by SMs (256 MiB), GB/s per direction: " +
              "; ".join(f"{label} x {c} CTAs: {r:.0f}" for label, c, r in sm_rates))
        print("| fused path | ours, rows moved by SM stores (ms) | ours, rows moved by copy engines (ms) | library collective + GEMM (ms) "
              "| GEMM alone (ms) | bytes / link rate (ms) | roofline (ms) | best fraction of roofline | SM MHz |")
        print("|---|---|---|---|---|---|---|---|---|")
        for name, a, b, lib, gm, lk, roof, mhz in rows:
            best = min(v for v in (a, b) if v is not None)
            print(f"| {name} | {a:.3f} | {'-' if b is None else f'{b:.3f}'} | {lib:.3f} | {gm:.3f} | {lk:.3f} | {roof:.3f} | "
                  f"{roof / best:.2f} | {mhz} |")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
