"""Expert parallelism: token dispatch / combine around the local experts.

Parity with the reference ``parallel/parallel_ep.py``: ``dispatch`` expands tokens x top-k,
orders the copies by destination rank, exchanges counts and then payloads with a variable
all-to-all (``:73-137``); ``combine`` reverses it and restores the original order (``:139-182``).
What the reference leaves broken is done here: an EP group exists, the local (ep=1) path works,
received tokens are grouped by local expert and every local expert is applied (the reference runs
``experts[0]`` on everything, model/model.py:109), and the exchange is differentiable.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from . import comm


@dataclass
class DispatchMeta:
    order: torch.Tensor              # [N*k] argsort of the flat (token, slot) copies by expert id
    send_counts: List[int]           # copies sent to each ep rank
    recv_counts: List[int]           # copies received from each ep rank
    local_order: Optional[torch.Tensor]   # permutation grouping received copies by local expert
    expert_counts: List[int]         # received copies per local expert (after grouping)
    n_tokens: int
    topk: int


class ExpertParallel:
    def __init__(self, num_experts: int, group=None):
        self.num_experts = num_experts
        self.group = group
        self.ep_size = comm.group_size(group)
        self.ep_rank = comm.group_rank(group)
        assert num_experts % self.ep_size == 0, "num_experts must be divisible by ep_size"
        self.local_experts = num_experts // self.ep_size
        self.first_expert = self.ep_rank * self.local_experts

    def dispatch(self, x: torch.Tensor, indices: torch.Tensor) -> Tuple[torch.Tensor, DispatchMeta]:
        """x [N, H], indices [N, k] (global expert ids) -> (tokens for the local experts grouped by
        expert [R, H], metadata)."""
        N, k = indices.shape
        flat_e = indices.reshape(-1)
        order = torch.argsort(flat_e, stable=True)              # groups by expert, hence by rank
        counts_e = torch.bincount(flat_e, minlength=self.num_experts)
        src_tok = torch.div(order, k, rounding_mode="floor")
        sent = x.index_select(0, src_tok)                       # [N*k, H], differentiable gather
        if self.ep_size == 1:
            meta = DispatchMeta(order, [N * k], [N * k], None, counts_e.tolist(), N, k)
            return sent, meta
        send_per_expert = counts_e.view(self.ep_size, self.local_experts)
        recv_per_expert = comm.all_to_all_equal(send_per_expert.contiguous(), self.group)  # [src, local_e]
        send_counts = send_per_expert.sum(1).tolist()
        recv_mat = recv_per_expert.view(self.ep_size, self.local_experts)
        recv_counts = recv_mat.sum(1).tolist()
        recv = comm.all_to_all_var_rows(sent, send_counts, recv_counts, self.group)
        # received layout: for src rank s: [expert 0 copies, expert 1 copies, ...]; regroup by expert
        if self.local_experts > 1:
            e_of = torch.repeat_interleave(
                torch.arange(self.local_experts, device=x.device).repeat(self.ep_size), recv_mat.reshape(-1))
            local_order = torch.argsort(e_of, stable=True)
            recv = recv.index_select(0, local_order)
        else:
            local_order = None
        meta = DispatchMeta(order, send_counts, recv_counts, local_order, recv_mat.sum(0).tolist(), N, k)
        return recv, meta

    def combine(self, y: torch.Tensor, meta: DispatchMeta) -> torch.Tensor:
        """y [R, H] (expert outputs in dispatch order) -> [N, k, H] in the original token order."""
        if self.ep_size > 1:
            if meta.local_order is not None:
                inv = torch.empty_like(meta.local_order)
                inv[meta.local_order] = torch.arange(meta.local_order.numel(), device=y.device)
                y = y.index_select(0, inv)
            y = comm.all_to_all_var_rows(y, meta.recv_counts, meta.send_counts, self.group)
        inv = torch.empty_like(meta.order)
        inv[meta.order] = torch.arange(meta.order.numel(), device=y.device)
        out = y.index_select(0, inv)
        return out.view(meta.n_tokens, meta.topk, y.shape[-1])

    def apply_experts(self, tokens: torch.Tensor, meta: DispatchMeta, experts: List[Callable]) -> torch.Tensor:
        """Run local expert ``e`` on its contiguous segment of ``tokens``."""
        counts = meta.expert_counts
        if self.ep_size == 1:
            counts = counts[self.first_expert:self.first_expert + self.local_experts]
        outs, off = [], 0
        for e, c in enumerate(counts):
            if c:
                outs.append(experts[e](tokens[off:off + c]))
            off += c
        if not outs:
            return tokens * 0.0
        return torch.cat(outs, dim=0)
