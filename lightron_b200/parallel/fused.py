"""Compute + collective pairs used by sequence-parallel TP.

``all_gather_linear``      rows sharded over the group -> all-gather -> GEMM   (C4 + K1/K3)
``linear_reduce_scatter``  GEMM with K sharded over the group -> reduce-scatter of rows (K2/K3 + C5)

On CUDA with ``fused_comm`` enabled these run as ONE sm_100a kernel each over NVLink peer
memory (``parallel.symm``): the all-gather is a set of peer-to-local tile copies issued by
dedicated CTAs while the tcgen05 main loop consumes row chunks as their flags arrive, and the
reduce-scatter is done by the GEMM epilogue storing partial tiles straight into the owner's
buffer.  Everywhere else (CPU ranks, fp32) they are the library collective followed by / following
the GEMM, which is also the baseline the fused kernels are measured against.

Reference call sites: ``funcol.all_gather_tensor`` before ``F.linear`` (parallel/parallel_tp.py:61-69)
and ``funcol.reduce_scatter_tensor`` after it (parallel/parallel_tp.py:100-106).
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..ops import functional as OF
from . import comm

_FUSED_ENABLED = True


def set_fused(enabled: bool) -> None:
    global _FUSED_ENABLED
    _FUSED_ENABLED = bool(enabled)


def _fused_ok(x: torch.Tensor, group, total_rows: int) -> bool:
    if not (_FUSED_ENABLED and x.is_cuda and x.dtype == torch.bfloat16 and comm.group_size(group) > 1):
        return False
    from . import symm
    return symm.supported(group) and symm.shapes_ok(total_rows, group)


def all_gather_linear(x_local: torch.Tensor, weights: Sequence[torch.Tensor], group) -> torch.Tensor:
    """x_local [T/n, K] (this rank's rows) -> [T, sum out_i] = all_gather(x) @ cat(weights)^T."""
    if _fused_ok(x_local, group, x_local.shape[0] * comm.group_size(group)):
        from . import symm
        return symm.AllGatherLinear.apply(x_local, group, *weights)
    return OF.linear(comm.gather_rows(x_local, group), *weights)


def linear_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, group) -> torch.Tensor:
    """x [T, K/n], weight [N, K/n] -> this rank's [T/n, N] rows of sum_over_ranks(x @ w^T)."""
    if _fused_ok(x, group, x.shape[0]):
        from . import symm
        return symm.LinearReduceScatter.apply(x, weight, group)
    return comm.scatter_rows(OF.linear(x, weight), group)
