"""Collective wrappers shared by every parallel strategy, plus their autograd forms.

On NCCL these are the plain library collectives (the baseline path and the bootstrap for the
fused peer-memory kernels).  On gloo (CPU ranks in tests) the collectives that gloo lacks are
composed from the ones it has, so every strategy runs unchanged on CPU: the reference cannot
(its Ulysses path needs list ``all_to_all``, parallel/parallel_cp.py:71, which gloo rejects).

Autograd pairs (Megatron "f/g" operators; the reference's ``_all_reduce`` is a raw in-place call
with no backward, parallel/parallel_tp.py:9-14, which leaves column-parallel input grads
un-reduced):
  copy_to_group      identity fwd   / all-reduce bwd
  reduce_from_group  all-reduce fwd / identity bwd
  gather_rows        all-gather fwd (dim 0) / reduce-scatter bwd
  scatter_rows       reduce-scatter fwd (dim 0) / all-gather bwd
  split_rows         keep own slice fwd / all-gather bwd
  all_to_all_rows    equal-split all-to-all, self-inverse in backward
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def group_size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


def _is_gloo(group) -> bool:
    return dist.get_backend(group) == "gloo"


def all_reduce(x: torch.Tensor, group, op=dist.ReduceOp.SUM) -> torch.Tensor:
    if group_size(group) > 1:
        dist.all_reduce(x, op=op, group=group)
    return x


def all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    assert x.shape[0] % n == 0, f"rows {x.shape[0]} not divisible by group size {n}"
    rows = x.shape[0] // n
    if _is_gloo(group):                 # gloo has no reduce_scatter: all-reduce then slice
        y = x.clone()
        dist.all_reduce(y, group=group)
        r = dist.get_rank(group)
        return y[r * rows:(r + 1) * rows].contiguous()
    out = torch.empty((rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def all_to_all_equal(x: torch.Tensor, group) -> torch.Tensor:
    """x [n*c, ...] -> chunk j goes to rank j; returns received chunks stacked in rank order."""
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty_like(x)
    if _is_gloo(group):
        _p2p_all_to_all(list(out.chunk(n)), list(x.chunk(n)), group)
    else:
        dist.all_to_all_single(out, x, group=group)
    return out


def all_to_all_var(x: torch.Tensor, send_counts: List[int], recv_counts: List[int], group) -> torch.Tensor:
    """Variable-split all-to-all over dim 0."""
    n = group_size(group)
    out = torch.empty((sum(recv_counts),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if n == 1:
        out.copy_(x)
        return out
    x = x.contiguous()
    if _is_gloo(group):
        _p2p_all_to_all(list(out.split(recv_counts)), list(x.split(send_counts)), group)
    else:
        dist.all_to_all_single(out, x, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return out


def _p2p_all_to_all(outs: List[torch.Tensor], ins: List[torch.Tensor], group) -> None:
    me = dist.get_rank(group)
    n = dist.get_world_size(group)
    outs[me].copy_(ins[me])
    reqs = []
    for off in range(1, n):
        dst = (me + off) % n
        src = (me - off) % n
        if ins[dst].numel():
            reqs.append(dist.isend(ins[dst].contiguous(), dist.get_global_rank(group, dst), group=group))
        if outs[src].numel():
            reqs.append(dist.irecv(outs[src], dist.get_global_rank(group, src), group=group))
    for r in reqs:
        r.wait()


# ---- autograd forms ----------------------------------------------------------------


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce(g.contiguous().clone(), ctx.group), None


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return all_reduce(x.contiguous().clone(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_rows(g, ctx.group), None


class _ScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_rows(g, ctx.group), None


class _SplitRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = group_size(group), group_rank(group)
        rows = x.shape[0] // n
        return x[r * rows:(r + 1) * rows].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_rows(g, ctx.group), None


class _GatherRowsReplicated(torch.autograd.Function):
    """all-gather fwd / keep own slice bwd: for consumers that compute identically on every rank
    (their input grads are already complete, not partial sums)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        n, r = group_size(ctx.group), group_rank(ctx.group)
        rows = g.shape[0] // n
        return g[r * rows:(r + 1) * rows].contiguous(), None


class _GatherCols(torch.autograd.Function):
    """all-gather on the last dim forward, keep own slice backward (LM-head ``gather_output``,
    parallel/parallel_tp.py:27-35,72)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = group_size(group)
        xt = x.reshape(-1, x.shape[-1]).t().contiguous()          # [V/t, T]
        full = all_gather_rows(xt, group)                          # [V, T]
        return full.t().contiguous().view(*x.shape[:-1], n * x.shape[-1])

    @staticmethod
    def backward(ctx, g):
        n, r = group_size(ctx.group), group_rank(ctx.group)
        c = g.shape[-1] // n
        return g[..., r * c:(r + 1) * c].contiguous(), None


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_to_all_equal(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_to_all_equal(g, ctx.group), None


class _AllToAllVar(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_counts, recv_counts, group):
        ctx.group, ctx.sc, ctx.rc = group, send_counts, recv_counts
        return all_to_all_var(x, send_counts, recv_counts, group)

    @staticmethod
    def backward(ctx, g):
        return all_to_all_var(g, ctx.rc, ctx.sc, ctx.group), None, None, None


def copy_to_group(x, group):
    return x if group_size(group) == 1 else _Copy.apply(x, group)


def reduce_from_group(x, group):
    return x if group_size(group) == 1 else _Reduce.apply(x, group)


def gather_rows(x, group):
    return x if group_size(group) == 1 else _GatherRows.apply(x, group)


def gather_rows_replicated(x, group):
    return x if group_size(group) == 1 else _GatherRowsReplicated.apply(x, group)


def scatter_rows(x, group):
    return x if group_size(group) == 1 else _ScatterRows.apply(x, group)


def split_rows(x, group):
    return x if group_size(group) == 1 else _SplitRows.apply(x, group)


def gather_cols(x, group):
    return x if group_size(group) == 1 else _GatherCols.apply(x, group)


def all_to_all_rows(x, group):
    return x if group_size(group) == 1 else _AllToAllRows.apply(x, group)


def all_to_all_var_rows(x, send_counts, recv_counts, group):
    return _AllToAllVar.apply(x, list(send_counts), list(recv_counts), group)
