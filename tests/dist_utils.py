"""Spawn helper for multi-process CPU (gloo) tests."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, q, pg_timeout_s=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        import datetime
        import torch.distributed as dist
        kw = {} if pg_timeout_s is None else {"timeout": datetime.timedelta(seconds=pg_timeout_s)}
        dist.init_process_group("gloo", rank=rank, world_size=world, **kw)
        out = fn(rank, world, *args)
    except Exception:
        q.put((rank, "err", traceback.format_exc()))
        return
    q.put((rank, "ok", out))
    try:                                   # tests that break the group on purpose have nothing left to tear down
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        pass


def run_distributed(fn, world: int, *args, timeout: float = 300.0, pg_timeout_s=None):
    """Run fn(rank, world, *args) on `world` gloo ranks; returns the list of results by rank.
    ``pg_timeout_s``: process-group timeout (a collective whose peer never joins fails after it)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q, pg_timeout_s)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, out = q.get(timeout=timeout)
            if status == "err":
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            results[rank] = out
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
