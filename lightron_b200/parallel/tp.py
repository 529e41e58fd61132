"""Tensor parallelism (+ Megatron sequence parallelism).

Parity with the reference ``parallel/parallel_tp.py``: ``ColumnParallelLinear`` (weight
``[out/tp, in]``, ``:38-74``), ``RowParallelLinear`` (weight ``[out, in/tp]``, ``:77-113``) and
``VocabParallelEmbedding`` (rows ``[V/tp, dim]``, masked lookup + all-reduce, ``:116-143``).
Differences: the collectives are autograd-aware (the reference's backward omits the
column-linear input-grad all-reduce); ``sequence_parallel=True`` is really usable (rows of the
flattened ``[tokens, hidden]`` activation are sharded across the group); on CUDA the
sequence-parallel all-gather / reduce-scatter are fused into the GEMM kernels through peer
memory (``parallel.fused``) instead of being separate NCCL calls.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import mesh
from ..ops import functional as OF
from . import comm


def _seq_to_rows(x: torch.Tensor):
    """[B, S_local, H] -> ([S_local*B... rows], restore) so that the sharded dim is dim 0."""
    if x.dim() == 2:
        return x, None
    B, S, H = x.shape
    return x.transpose(0, 1).reshape(S * B, H), (B, S)


def _rows_to_seq(x: torch.Tensor, meta, n_scale: float = 1.0):
    if meta is None:
        return x
    B, S = meta
    S = int(S * n_scale)
    return x.view(S, B, x.shape[-1]).transpose(0, 1)


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, gather_output: bool = False,
                 sequence_parallel: bool = False, group="auto", dtype=None, device=None):
        super().__init__()
        self.group = mesh.get_tp_group() if group == "auto" else group
        self.tp = comm.group_size(self.group)
        assert out_features % self.tp == 0, f"out_features {out_features} not divisible by tp {self.tp}"
        self.in_features, self.out_features = in_features, out_features
        self.out_local = out_features // self.tp
        self.gather_output = gather_output
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.weight = nn.Parameter(torch.empty(self.out_local, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(self.out_local, dtype=dtype, device=device)) if bias else None
        self.weight.tp_shard_dim = 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            rows, meta = _seq_to_rows(x)
            from . import fused
            y = fused.all_gather_linear(rows, (self.weight,), self.group)
            y = _rows_to_seq(y, meta, self.tp)
        else:
            y = OF.linear(comm.copy_to_group(x, self.group), self.weight)
        if self.bias is not None:
            y = y + self.bias
        if self.gather_output:
            y = comm.gather_cols(y, self.group)
        return y


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, input_is_parallel: bool = True,
                 sequence_parallel: bool = False, group="auto", dtype=None, device=None):
        super().__init__()
        self.group = mesh.get_tp_group() if group == "auto" else group
        self.tp = comm.group_size(self.group)
        assert in_features % self.tp == 0, f"in_features {in_features} not divisible by tp {self.tp}"
        self.in_features, self.out_features = in_features, out_features
        self.in_local = in_features // self.tp
        self.input_is_parallel = input_is_parallel
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.weight = nn.Parameter(torch.empty(out_features, self.in_local, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.weight.tp_shard_dim = 1

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.input_is_parallel and self.tp > 1:
            r = comm.group_rank(self.group)
            x = x[..., r * self.in_local:(r + 1) * self.in_local]
        if self.sequence_parallel:
            rows, meta = _seq_to_rows(x)
            from . import fused
            y = fused.linear_reduce_scatter(rows, self.weight, self.group)
            y = _rows_to_seq(y, meta, 1.0 / self.tp)
        else:
            y = comm.reduce_from_group(OF.linear(x, self.weight), self.group)
        if self.bias is not None:
            y = y + self.bias
        return y


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, group="auto", sequence_parallel: bool = False,
                 dtype=None, device=None):
        super().__init__()
        self.group = mesh.get_tp_group() if group == "auto" else group
        self.tp = comm.group_size(self.group)
        assert num_embeddings % self.tp == 0
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.local = num_embeddings // self.tp
        self.vocab_start = comm.group_rank(self.group) * self.local
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.weight = nn.Parameter(torch.empty(self.local, embedding_dim, dtype=dtype, device=device))
        self.weight.tp_shard_dim = 0

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            from . import embed_fused
            sp = self.sequence_parallel and tokens.dim() == 1
            if (tokens.dim() == 1 or not self.sequence_parallel) and embed_fused.fused_ok(self.weight, self.group, tokens.numel(), sp):
                out = embed_fused.vocab_parallel_embedding(tokens, self.weight, self.group, self.vocab_start, sp)
                return out if sp else out.view(*tokens.shape, self.embedding_dim)
        part = OF.embedding(tokens, self.weight, self.vocab_start)
        if self.tp == 1:
            return part
        if self.sequence_parallel:
            rows, meta = _seq_to_rows(part) if part.dim() == 3 else (part, None)
            return _rows_to_seq(comm.scatter_rows(rows.contiguous(), self.group), meta, 1.0 / self.tp)
        return comm.reduce_from_group(part, self.group)


class Linear(nn.Module):
    """Unsharded bias-free linear holding ``weight`` [out, in] (same state_dict key as nn.Linear)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype=None, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        y = OF.linear(x, self.weight)
        return y if self.bias is None else y + self.bias
