"""Process mesh: one process per GPU, rank = ((pp*DP + dp)*CP + cp)*TP + tp.

Parity with the reference: ``parallel/distributed.py:9-130`` (size validation, mesh order
pp,dp,cp,tp with TP innermost, group getters, EP living inside DP).  Differences: the device
type follows the backend (``gloo`` -> cpu, ``nccl`` -> cuda) so every parallel path also runs as
CPU ranks; an expert-parallel group really exists (the reference returns the DP group and never
creates an ``ep`` dim, ``parallel/distributed.py:122-130``); a ``dp x cp`` group exists because
parameters are replicated over both and gradients must be reduced over both.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelContext:
    tp_size: int = 1
    dp_size: int = 1
    cp_size: int = 1
    pp_size: int = 1
    ep_size: int = 1
    rank: int = 0
    world_size: int = 1
    device: torch.device = torch.device("cpu")
    tp_group: Optional[dist.ProcessGroup] = None
    dp_group: Optional[dist.ProcessGroup] = None
    cp_group: Optional[dist.ProcessGroup] = None
    pp_group: Optional[dist.ProcessGroup] = None
    ep_group: Optional[dist.ProcessGroup] = None     # ep_size ranks inside one dp group
    edp_group: Optional[dist.ProcessGroup] = None    # dp/ep replicas of the same experts
    dpcp_group: Optional[dist.ProcessGroup] = None   # gradient reduction group (dp x cp)
    edpcp_group: Optional[dist.ProcessGroup] = None  # gradient reduction group of expert params
    group_ranks: Dict[str, List[int]] = None

    # ---- coordinates -------------------------------------------------------------------
    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def cp_rank(self) -> int:
        return (self.rank // self.tp_size) % self.cp_size

    @property
    def dp_rank(self) -> int:
        return (self.rank // (self.tp_size * self.cp_size)) % self.dp_size

    @property
    def pp_rank(self) -> int:
        return self.rank // (self.tp_size * self.cp_size * self.dp_size)

    @property
    def ep_rank(self) -> int:
        return self.dp_rank % self.ep_size

    @property
    def pp_is_first(self) -> bool:
        return self.pp_rank == 0

    @property
    def pp_is_last(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    def coord_to_rank(self, pp: int, dp: int, cp: int, tp: int) -> int:
        return ((pp * self.dp_size + dp) * self.cp_size + cp) * self.tp_size + tp

    @property
    def pp_prev_rank(self) -> Optional[int]:
        if self.pp_is_first:
            return None
        return self.coord_to_rank(self.pp_rank - 1, self.dp_rank, self.cp_rank, self.tp_rank)

    @property
    def pp_next_rank(self) -> Optional[int]:
        if self.pp_is_last:
            return None
        return self.coord_to_rank(self.pp_rank + 1, self.dp_rank, self.cp_rank, self.tp_rank)

    @property
    def log_rank(self) -> int:
        """Rank that owns the loss: 0 without PP, first rank of the last stage with PP
        (the reference logs on ``world/pp``, trainer.py:320-324, which is only right for pp=2)."""
        return self.coord_to_rank(self.pp_size - 1, 0, 0, 0)

    @property
    def grad_replicas(self) -> int:
        return self.dp_size * self.cp_size

    def describe(self) -> str:
        return (f"PP={self.pp_size} | DP={self.dp_size} (EP={self.ep_size}) | CP={self.cp_size} | "
                f"TP={self.tp_size} | world={self.world_size}")


_CTX: Optional[ParallelContext] = None


def _enumerate_groups(pp, dp, cp, tp, ep) -> Dict[str, List[List[int]]]:
    """Rank lists of every group of every kind, in a deterministic order (pure function: unit-tested)."""
    def r(p, d, c, t):
        return ((p * dp + d) * cp + c) * tp + t
    out: Dict[str, List[List[int]]] = {k: [] for k in ("tp", "cp", "dp", "pp", "ep", "edp", "dpcp", "edpcp")}
    for p in range(pp):
        for d in range(dp):
            for c in range(cp):
                out["tp"].append([r(p, d, c, t) for t in range(tp)])
            for t in range(tp):
                out["cp"].append([r(p, d, c, t) for c in range(cp)])
        for c in range(cp):
            for t in range(tp):
                out["dp"].append([r(p, d, c, t) for d in range(dp)])
                for g in range(dp // ep):     # ep group: consecutive dp ranks
                    out["ep"].append([r(p, g * ep + e, c, t) for e in range(ep)])
                for e in range(ep):           # same experts: dp ranks congruent mod ep
                    out["edp"].append([r(p, g * ep + e, c, t) for g in range(dp // ep)])
        for t in range(tp):
            out["dpcp"].append([r(p, d, c, t) for d in range(dp) for c in range(cp)])
            for e in range(ep):
                out["edpcp"].append([r(p, g * ep + e, c, t) for g in range(dp // ep) for c in range(cp)])
    for d in range(dp):
        for c in range(cp):
            for t in range(tp):
                out["pp"].append([r(p, d, c, t) for p in range(pp)])
    return out


def setup_distributed(tp_size: int = 1, pp_size: int = 1, cp_size: int = 1, ep_size: int = 1,
                      dp_size: int = 1, backend: Optional[str] = None,
                      timeout_s: float = 600.0) -> ParallelContext:
    """Create the process groups.  Works without torchrun for world_size 1."""
    global _CTX
    expected = tp_size * pp_size * cp_size * dp_size
    if dp_size % ep_size:
        raise ValueError(f"DP size ({dp_size}) must be divisible by EP size ({ep_size})")
    if not dist.is_initialized():
        if expected == 1 and "RANK" not in os.environ:
            dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
            _CTX = ParallelContext(device=dev, group_ranks={})
            return _CTX
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group(backend=backend, init_method="env://",
                                timeout=datetime.timedelta(seconds=timeout_s))
    world, rank = dist.get_world_size(), dist.get_rank()
    if world != expected:
        raise ValueError(f"World Size Mismatch! Real: {world}, Configured: {pp_size}(PP) * {dp_size}(DP) * "
                         f"{cp_size}(CP) * {tp_size}(TP) = {expected}")
    if dist.get_backend() == "nccl":
        device = torch.device("cuda", torch.cuda.current_device())
    else:
        device = torch.device("cpu")
    ctx = ParallelContext(tp_size, dp_size, cp_size, pp_size, ep_size, rank, world, device, group_ranks={})
    sizes = dict(tp=tp_size, cp=cp_size, dp=dp_size, pp=pp_size, ep=ep_size, edp=dp_size // ep_size,
                 dpcp=dp_size * cp_size, edpcp=(dp_size // ep_size) * cp_size)
    for kind, groups in _enumerate_groups(pp_size, dp_size, cp_size, tp_size, ep_size).items():
        if sizes[kind] == 1:
            continue
        for ranks in groups:       # every rank creates every group, in the same order
            g = dist.new_group(ranks=ranks)
            if rank in ranks:
                setattr(ctx, f"{kind}_group", g)
                ctx.group_ranks[kind] = ranks
    _CTX = ctx
    if rank == 0:
        print(f"Distributed init: {ctx.describe()}", flush=True)
    return ctx


def get_context() -> ParallelContext:
    global _CTX
    if _CTX is None:
        _CTX = ParallelContext(device=torch.device("cuda", 0) if torch.cuda.is_available()
                               else torch.device("cpu"), group_ranks={})
    return _CTX


def set_context(ctx: Optional[ParallelContext]) -> None:
    global _CTX
    _CTX = ctx


def get_tp_group():
    return get_context().tp_group


def get_cp_group():
    return get_context().cp_group


def get_pp_group():
    return get_context().pp_group


def get_dp_group():
    return get_context().dp_group


def get_ep_group():
    return get_context().ep_group


def get_parallel_info() -> Dict[str, int]:
    c = get_context()
    return {"tp": c.tp_size, "pp": c.pp_size, "cp": c.cp_size, "ep": c.ep_size, "dp": c.dp_size}


def destroy() -> None:
    global _CTX
    _CTX = None
    if dist.is_initialized():
        dist.destroy_process_group()
