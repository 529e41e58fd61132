"""Failure detection on the host side: heartbeats through the rendezvous store, config agreement
across ranks, and a watchdog around collective calls.

The reference has only the 10-minute NCCL timeout (trainer.py:103) and shape asserts.  Here:
* ``check_config_agreement`` hashes the run config on every rank and compares through an
  all-gather, so a rank launched with another JSON fails at start-up instead of deadlocking later;
* ``Heartbeat`` lets every rank publish a monotonically increasing beat in the key-value store
  between steps; ``dead_ranks()`` lists the ranks whose beat is older than a limit, so that the
  survivors learn of a lost rank on the host, before their next launch;
* ``guarded`` runs a host function in a watchdog thread and raises ``RankFailure`` if it does not
  return in time (a collective whose peer never joined);
* ``announce_failure`` / ``failed_ranks``: a rank that leaves the training loop with an exception says
  so in the store, and a rank whose own step then fails (its collective timed out, the connection
  closed) reports THAT rank as the cause instead of its own secondary error;
* ``maybe_inject_failure``: host-side fault injection for tests (``LIGHTRON_INJECT_FAILURE=rank:step``
  makes that rank raise at the start of that step, between steps, with nothing in flight).
Recovery is a relaunch with ``training.resume`` pointing at the last periodic checkpoint.
Device-side waits are bounded inside the kernels and surface through ``lb_device_status`` /
``symm.check_status``.  Nothing here, and no test of it, faults or hangs a GPU.
"""
from __future__ import annotations

import hashlib
import json
import threading
import time
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist


class RankFailure(RuntimeError):
    pass


class InjectedFailure(RuntimeError):
    """Raised by ``maybe_inject_failure`` (tests of the detection and recovery path)."""


def maybe_inject_failure(step: int, rank: int) -> None:
    import os
    spec = os.environ.get("LIGHTRON_INJECT_FAILURE")
    if not spec:
        return
    r, s = spec.split(":")
    if int(r) == rank and int(s) == step:
        raise InjectedFailure(f"injected failure on rank {rank} before step {step}")


def announce_failure(store, rank: int, reason: str) -> None:
    try:
        store.set(f"failed/{rank}", f"{time.time():.3f}:{reason[:300]}")
    except Exception:                       # the store itself may be gone: nothing more to do
        pass


def failed_ranks(store, world_size: int, exclude: Optional[int] = None) -> Dict[int, str]:
    out: Dict[int, str] = {}
    for r in range(world_size):
        if r == exclude:
            continue
        try:
            if hasattr(store, "check") and not store.check([f"failed/{r}"]):
                continue
            out[r] = store.get(f"failed/{r}").decode().split(":", 1)[1]
        except Exception:
            continue
    return out


def check_config_agreement(cfg_dict: Dict[str, Any], group=None) -> None:
    digest = hashlib.sha256(json.dumps(cfg_dict, sort_keys=True, default=str).encode()).digest()[:8]
    mine = torch.tensor(list(digest), dtype=torch.int64)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    mine = mine.to(dev)
    allv = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(allv, mine, group=group)
    bad = [r for r, v in enumerate(allv) if not torch.equal(v.cpu(), allv[0].cpu())]
    if bad:
        raise RankFailure(f"run config differs on ranks {bad} (vs rank 0)")


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, prefix: str = "hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world_size, prefix
        self.beat_no = 0

    def beat(self) -> None:
        self.beat_no += 1
        self.store.set(f"{self.prefix}/{self.rank}", f"{self.beat_no}:{time.time():.3f}")

    def last_seen(self, rank: int) -> Optional[float]:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}/{rank}"]):
                return None
            v = self.store.get(f"{self.prefix}/{rank}").decode()
            return float(v.split(":")[1])
        except Exception:
            return None

    def dead_ranks(self, max_age_s: float) -> List[int]:
        now = time.time()
        out = []
        for r in range(self.world):
            t = self.last_seen(r)
            if t is None or now - t > max_age_s:
                out.append(r)
        return out


def guarded(fn: Callable[[], Any], timeout_s: float, what: str = "collective") -> Any:
    """Run ``fn`` in a helper thread; raise RankFailure if it has not returned after timeout_s."""
    box: Dict[str, Any] = {}

    def run():
        try:
            box["out"] = fn()
        except BaseException as e:          # noqa: BLE001 - re-raised in the caller
            box["err"] = e

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(timeout_s)
    if t.is_alive():
        raise RankFailure(f"{what} did not complete within {timeout_s:.1f}s: a peer is missing or stuck")
    if "err" in box:
        raise box["err"]
    return box.get("out")
