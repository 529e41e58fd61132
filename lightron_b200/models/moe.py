"""Sparse mixture-of-experts feed-forward with expert parallelism.

Parity: ``MoEFeedForward`` in the reference's ``model/model.py:72-116``: a bias-free ``gate`` linear,
softmax over experts then top-k (``:96-98``), dispatch, expert SwiGLU MLPs, combine and a sum over
the k slots weighted by the (un-renormalised) router probabilities (``:115``).  Completed here:
each rank allocates only its own experts (the reference allocates all of them on every rank,
``:88``), every local expert is applied to its own tokens (``:109`` applies expert 0 to all) and a
Switch-style load-balance auxiliary loss ``E * sum_e f_e * P_e`` is produced.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelArgs
from ..ops import functional as OF
from ..parallel.ep import ExpertParallel
from ..parallel.tp import Linear


class MoEFeedForward(nn.Module):
    def __init__(self, args: ModelArgs, ctx, **kw):
        super().__init__()
        from .llama import MLP
        self.num_experts = args.moe_num_experts
        self.topk = args.moe_topk
        self.gate = Linear(args.dim, self.num_experts, **kw)
        group = ctx.ep_group if args.ep_size > 1 else None
        self.ep = ExpertParallel(self.num_experts, group)
        lo = self.ep.first_expert
        self.experts = nn.ModuleDict({str(e): MLP(args, ctx, **kw) for e in range(lo, lo + self.ep.local_experts)})
        for p in self.experts.parameters():
            p.is_expert = True
        self.sp = args.sequence_parallel and args.tp_size > 1
        self.tp_group = ctx.tp_group if args.tp_size > 1 else None
        self.last_aux_loss = None
        self.capacity_factor = args.moe_capacity_factor
        self.pp_size = getattr(ctx, "pp_size", 1)
        self.layer_key = id(self)

    def _fused_ok(self, x: torch.Tensor) -> bool:
        """The kernel chain of ``parallel.ep_fused`` (router, peer-memory dispatch / combine, ragged
        expert GEMMs, no host synchronisation): CUDA bf16, experts not tensor-parallel, parameters in
        the flat arena, and no pipeline parallelism (several micro-batches between a layer's forward
        and backward would share the layer's exchange buffers)."""
        from ..parallel import ep_fused
        if self.tp_group is not None or self.pp_size > 1:
            return False
        mlps = list(self.experts.values())
        if not all(OF._rows_adjacent((m.w1.weight, m.w3.weight)) for m in mlps):
            return False
        return ep_fused.supported(x, self.ep.group, self.num_experts, self.topk, self.ep.local_experts)

    def _apply_experts(self, tokens: torch.Tensor, meta) -> torch.Tensor:
        """Local expert e on its contiguous segment of ``tokens``: one grouped GEMM launch for the
        gate+up projections of all local experts, SwiGLU, one for the down projections (K14 of the
        kernel list: the reference runs a single expert, model/model.py:109).  With tensor-parallel
        experts, or before the parameters sit in the flat arena, experts run one after the other."""
        mlps = list(self.experts.values())
        up = [(m.w1.weight, m.w3.weight) for m in mlps]
        down = [(m.w2.weight,) for m in mlps]
        if self.tp_group is None and tokens.shape[0] > 0 and OF.grouped_linear_ok(tokens, up) \
                and OF.grouped_linear_ok(tokens, down):
            counts = meta.expert_counts
            if self.ep.ep_size == 1:
                counts = counts[self.ep.first_expert:self.ep.first_expert + self.ep.local_experts]
            counts = [int(c) for c in counts]
            gu = OF.grouped_linear(tokens, counts, up)
            return OF.grouped_linear(OF.swiglu(gu), counts, down)
        experts = [lambda t, m=m: m(t, sp=False) for m in mlps]
        return self.ep.apply_experts(tokens, meta, experts)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [T, H] -> [T, H]."""
        from ..parallel import comm
        if self.sp:                       # experts see whole tokens; gather the row shards first
            x = comm.gather_rows_replicated(x, self.tp_group)
        T, H = x.shape
        if self._fused_ok(x):
            from ..parallel import ep_fused
            ws = [w for m in self.experts.values() for w in (m.w1.weight, m.w3.weight, m.w2.weight)]
            out, aux = ep_fused.fused_moe(x, self.gate.weight, ws, self.num_experts, self.topk, self.ep.group,
                                          self.layer_key, self.capacity_factor)
            self.last_aux_loss = aux[0]
            if self.sp:
                out = comm.split_rows(out, self.tp_group)
            return out
        logits = OF.linear(x, self.gate.weight).float()
        probs = F.softmax(logits, dim=-1)
        weights, indices = torch.topk(probs, self.topk, dim=-1)
        # load-balance loss: fraction of routed copies per expert x mean router probability
        with torch.no_grad():
            frac = torch.bincount(indices.reshape(-1), minlength=self.num_experts).float() / (T * self.topk)
        self.last_aux_loss = self.num_experts * torch.sum(frac * probs.mean(dim=0))
        tokens, meta = self.ep.dispatch(x, indices)
        y = self._apply_experts(tokens, meta)
        y = self.ep.combine(y, meta)                             # [T, k, H]
        out = (y.float() * weights.unsqueeze(-1)).sum(dim=1).to(x.dtype)
        if self.sp:
            out = comm.split_rows(out, self.tp_group)
        return out
